// GEMM for lumen's dot_general (one contracting dimension, optional leading batch), the counterpart of the
// reference's Ampere `mma.sync` CuTe kernel behind its GEMM hook (lumen/codegen/dot_general/cuda/ampere.py:35-904,
// lumen/codegen/dot_general/cuda/mod.rs:658-757) rebuilt for Blackwell:
//
//  * gemm_tcgen05: 16-bit operands, explicit fp32 accumulation in tensor memory. Persistent, warp-specialised:
//    warp 0 issues TMA tile loads into a 4-stage ring of 128-byte-swizzled shared-memory tiles, one thread of warp 1
//    issues tcgen05.mma (128x256x16 per instruction) and commits stage/accumulator barriers, warps 2-9 drain the
//    previous tile's accumulator (tcgen05.ld) through the epilogue while the next tile's MMAs run into the other
//    half of the 512 TMEM columns. All four operand majors (row- or column-major A and B) are handled by the tensor
//    maps and the descriptor major bits, so the transposed *views* of the backward GEMMs (dA = dY.B^T, dB = A^T.dY)
//    need no copies. Every CTA loads its own operand tiles.
//  * gemm_simt: any float dtype and any strides, one thread per output element group, products and partial sums
//    rounded to fp32 one by one in contracting order (__fmul_rn / __fadd_rn): exactly the reference interpreter's
//    accumulation (lumen/reference/mod.rs:958-970). float32 operands always take this path: there is no hidden
//    TF32/bf16 narrowing.
#include <algorithm>
#include <map>
#include <mutex>

#include "device.h"
#include "sm100.cuh"

namespace lb {
namespace {

using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int kThreads = 320;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..9: epilogue
constexpr int kEpilogueWarps = 8;
constexpr int kStageBytesA = BM * BK * 2, kStageBytesB = BN * BK * 2;
constexpr int kEpilogueStageBytes = 8 * 4096;  // one 4 KB staging area per epilogue warp (store_rows_coalesced)
constexpr int kSmemBytes = STAGES * (kStageBytesA + kStageBytesB) + 1024 /*alignment slack*/ + 256 /*barriers*/ + kEpilogueStageBytes;

// EPI_ADD: out = round(round(acc) + aux); EPI_MASK: out = aux > 0 ? round(acc) : 0 - each exactly the two primitives
// of the traced program (a rounded product followed by an add / a select), with `aux` a tensor shaped like the output
enum Epilogue : int { EPI_NONE = 0, EPI_RELU = 1, EPI_ADD = 2, EPI_MASK = 3 };

struct GemmArgs {
    int M, N, K, batch;
    int a_mn_major, b_mn_major;
    void* d;
    int d_bf16;           // output rounded once to bf16 (else fp32)
    int d_f16;
    int in_bf16;          // operands bfloat16 (else float16): the MMA's operand format
    long long ldd, d_batch_stride;
    int epilogue;
    const void* aux;      // EPI_ADD / EPI_MASK operand: same dtype as the output, row-major [batch, M, N] view
    long long ld_aux, aux_batch_stride;
    int* status;          // device word: set to LB_ERR_TIMEOUT when a bounded wait gave up
    int tiles_m, tiles_n, group_m;
    // split-K: the K loop of every tile is cut into `splits` ranges of `kb_per_split` 64-wide blocks; each (tile, range)
    // unit writes a float32 partial tile to `partial` [splits][batch][M][N] and splitk_reduce adds them in order
    int splits, kb_per_split;
    float* partial;
};

__device__ __forceinline__ void tile_coords(const GemmArgs& p, int tile, int& b, int& m_blk, int& n_blk) {
    int per_batch = p.tiles_m * p.tiles_n;
    b = tile / per_batch;
    int t = tile - b * per_batch;
    // grouped raster: GROUP_M row-blocks share each column-block while they are resident together in L2
    int group_size = p.group_m * p.tiles_n;
    int g = t / group_size;
    int first_m = g * p.group_m;
    int rows = min(p.tiles_m - first_m, p.group_m);
    int in_group = t - g * group_size;
    m_blk = first_m + in_group % rows;
    n_blk = in_group / rows;
}

// Drains 128 accumulator columns (this warp's half of a 256-wide tile) of the thread's row from tensor memory and
// stores them: float32 partial sums when K is split, otherwise the epilogue and one rounding to the output dtype.
__device__ __forceinline__ void drain_tile(const GemmArgs& p, uint32_t tbase, int row, long long row_off, int col_base, int b, int split,
                                           bool vec_ok, uint4* stage, int lane) {
#pragma unroll 1
    for (int c2 = 0; c2 < BN / 2 / 64; c2++) {
        // warp-uniform: 16-bit rows of 64 whole columns leave through the staging area, 128 contiguous bytes per row
        const bool coalesced = vec_ok && p.splits == 1 && (p.d_bf16 || p.d_f16) && col_base + c2 * 64 + 64 <= p.N;
        uint4 packed[8];
        uint32_t vv[64];
        tmem_ld_32x32(tbase + c2 * 64, vv);  // two loads in flight, one wait
        tmem_ld_32x32(tbase + c2 * 64 + 32, vv + 32);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t* v = vv + h * 32;
            const int col0 = col_base + c2 * 64 + h * 32;
            // warp-uniform: a float32 row piece of 32 whole columns is one 128-byte line and leaves through the staging area too
            const bool staged32 = vec_ok && p.splits == 1 && !(p.d_bf16 || p.d_f16) && col0 + 32 <= p.N;
            if (p.splits > 1) {
                // a partial sum: float32, dense [split][batch][M][N]; the epilogue and rounding happen in splitk_reduce
                if (row < p.M && col0 < p.N) {
                    float* out = p.partial + ((long long)(split * p.batch + b) * p.M + row) * p.N + col0;
                    if (col0 + 32 <= p.N && p.N % 4 == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *(uint4*)(out + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < p.N) out[j] = __uint_as_float(v[j]);
                    }
                }
            } else if (row < p.M && col0 < p.N) {
                if (p.epilogue == EPI_RELU) {
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.0f));
                }
                const bool full_chunk = col0 + 32 <= p.N;
                if (p.epilogue >= EPI_ADD) {
                    // 16-bit outputs only (checked by the host). The product is rounded first, as its own primitive.
                    const uint16_t* ax = (const uint16_t*)p.aux + (long long)b * p.aux_batch_stride + (long long)row * p.ld_aux + col0;
                    uint32_t aw[16];
                    if (full_chunk && p.ld_aux % 8 == 0 && p.aux_batch_stride % 8 == 0 && ((uintptr_t)p.aux & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint4 t = *(const uint4*)(ax + 8 * j);
                            aw[4 * j] = t.x, aw[4 * j + 1] = t.y, aw[4 * j + 2] = t.z, aw[4 * j + 3] = t.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const uint32_t lo = col0 + 2 * j < p.N ? ax[2 * j] : 0u, hi = col0 + 2 * j + 1 < p.N ? ax[2 * j + 1] : 0u;
                            aw[j] = lo | (hi << 16);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const uint16_t a16 = (uint16_t)(j & 1 ? aw[j / 2] >> 16 : aw[j / 2] & 0xffffu);
                        const float acc = __uint_as_float(v[j]);
                        float prod, other;
                        if (p.d_bf16) prod = __bfloat162float(__float2bfloat16_rn(acc)), other = __uint_as_float((uint32_t)a16 << 16);
                        else prod = __half2float(__float2half_rn(acc)), other = __half2float(__ushort_as_half(a16));
                        v[j] = __float_as_uint(p.epilogue == EPI_ADD ? __fadd_rn(other, prod) : (other > 0.0f ? prod : 0.0f));
                    }
                }
                if (p.d_bf16 || p.d_f16) {
                    uint16_t* out = (uint16_t*)p.d + row_off + col0;
                    if (full_chunk && vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                float lo = __uint_as_float(v[j + 2 * q]), hi = __uint_as_float(v[j + 2 * q + 1]);
                                if (p.d_bf16) {
                                    __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi);
                                    w[q] = *(uint32_t*)&hh;
                                } else {
                                    __half2 hh = __floats2half2_rn(lo, hi);
                                    w[q] = *(uint32_t*)&hh;
                                }
                            }
                            if (coalesced) packed[h * 4 + j / 8] = make_uint4(w[0], w[1], w[2], w[3]);
                            else *(uint4*)(out + j) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) {  // unrolled with a predicate: keeps the fragment in registers
                            float x = __uint_as_float(v[j]);
                            if (col0 + j < p.N)
                                out[j] = p.d_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
                        }
                    }
                } else {
                    float* out = (float*)p.d + row_off + col0;
                    if (staged32) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) packed[j / 4] = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else if (full_chunk && vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *(uint4*)(out + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (col0 + j < p.N) out[j] = __uint_as_float(v[j]);
                    }
                }
            }
            if (staged32)
                store_rows_coalesced<8>(stage, packed, (uint8_t*)((float*)p.d + (row_off - (long long)lane * p.ldd) + col0), p.ldd * 4,
                                        p.M - (row - lane), lane);
        }
        if (coalesced)  // rows past M hold nothing and are not written
            store_rows_coalesced<8>(stage, packed, (uint8_t*)((uint16_t*)p.d + (row_off - (long long)lane * p.ldd) + col_base + c2 * 64),
                                    p.ldd * 2, p.M - (row - lane), lane);
    }
}

// The add / mask epilogues on the fast path (unsplit K, a full 128-column span inside N, 16-byte aligned rows of the
// operand and the output): the operand's 32-column chunks are loaded one chunk ahead - the first one before the
// warp waits for the tile's MMAs - so that their global-memory latency never sits between the accumulator load
// and the store.
__device__ __forceinline__ bool aux_fast_path(const GemmArgs& p, int row, int col_base, bool vec_ok) {
    return p.epilogue >= EPI_ADD && p.splits == 1 && vec_ok && row < p.M && col_base + BN / 2 <= p.N && p.ld_aux % 8 == 0 &&
           p.aux_batch_stride % 8 == 0 && ((uintptr_t)p.aux & 15) == 0;
}
// Loads a 32-row x 32-column chunk of the operand with whole 64-byte row pieces per four lanes (eight rows per load
// instruction): lane l gets the 16-byte segment l % 4 of rows l / 4, 8 + l / 4, 16 + l / 4 and 24 + l / 4.
// `ax_warp` points at the warp's first row.
__device__ __forceinline__ void aux_load(const uint16_t* ax_warp, long long ld_aux, int lane, uint4* raw) {
#pragma unroll
    for (int t = 0; t < 4; t++) raw[t] = *(const uint4*)(ax_warp + (long long)(t * 8 + (lane >> 2)) * ld_aux + (lane & 3) * 8);
}
// Turns what aux_load fetched into each lane's own row (16 packed pairs) through 2 KB of the warp's staging area.
__device__ __forceinline__ void aux_to_rows(uint4* stage_aux, const uint4* raw, uint32_t* aw, int lane) {
    __syncwarp();
#pragma unroll
    for (int t = 0; t < 4; t++) {
        const int r = t * 8 + (lane >> 2), q = lane & 3;
        stage_aux[r * 4 + (q ^ ((r >> 1) & 3))] = raw[t];
    }
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const uint4 x = stage_aux[lane * 4 + (q ^ ((lane >> 1) & 3))];
        aw[4 * q] = x.x, aw[4 * q + 1] = x.y, aw[4 * q + 2] = x.z, aw[4 * q + 3] = x.w;
    }
}
__device__ __forceinline__ void drain_tile_aux(const GemmArgs& p, uint32_t tbase, long long row_off, const uint16_t* ax_warp, uint4* raw,
                                               uint4* stage, int lane) {
    uint8_t* out0 = (uint8_t*)((uint16_t*)p.d + (row_off - (long long)lane * p.ldd));  // the warp's first row (all 32 are inside M)
#pragma unroll 1
    for (int c = 0; c < BN / 2 / 32; c++) {
        uint32_t v[32], aw[16];
        tmem_ld_32x32(tbase + c * 32, v);
        aux_to_rows(stage + 128, raw, aw, lane);
        if (c + 1 < BN / 2 / 32) aux_load(ax_warp + (c + 1) * 32, p.ld_aux, lane, raw);
        tmem_ld_wait();
        uint4 packed[4];
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float r[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const uint32_t pair = aw[(j + 2 * q) / 2];
                    const uint16_t a16 = (uint16_t)(u ? pair >> 16 : pair & 0xffffu);
                    const float acc = __uint_as_float(v[j + 2 * q + u]);
                    float prod, other;
                    if (p.d_bf16) prod = __bfloat162float(__float2bfloat16_rn(acc)), other = __uint_as_float((uint32_t)a16 << 16);
                    else prod = __half2float(__float2half_rn(acc)), other = __half2float(__ushort_as_half(a16));
                    r[u] = p.epilogue == EPI_ADD ? __fadd_rn(other, prod) : (other > 0.0f ? prod : 0.0f);
                }
                if (p.d_bf16) {
                    __nv_bfloat162 hh = __floats2bfloat162_rn(r[0], r[1]);
                    w[q] = *(uint32_t*)&hh;
                } else {
                    __half2 hh = __floats2half2_rn(r[0], r[1]);
                    w[q] = *(uint32_t*)&hh;
                }
            }
            packed[j / 8] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        store_rows_coalesced<4>(stage, packed, out0 + c * 64, p.ldd * 2, 32, lane);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * kStageBytesA;
    uint64_t* full = (uint64_t*)(smem + STAGES * (kStageBytesA + kStageBytesB));
    uint64_t* empty = full + STAGES;
    uint64_t* tmem_full = empty + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_slot = (uint32_t*)(tmem_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n * p.batch;
    const int total_kb = (p.K + BK - 1) / BK;
    const int num_units = num_tiles * p.splits;  // unit = split * num_tiles + tile: neighbours share a K range

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], kEpilogueWarps);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
                int b, m_blk, n_blk;
                tile_coords(p, unit % num_tiles, b, m_blk, n_blk);
                const int kb0 = (unit / num_tiles) * p.kb_per_split, kb1 = min(total_kb, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag))) break;
                    mbar_expect_tx(&full[stage], kStageBytesA + kStageBytesB);
                    uint8_t* sa = smem_a + stage * kStageBytesA;
                    uint8_t* sb = smem_b + stage * kStageBytesB;
                    if (!p.a_mn_major) {
                        tma_load_3d(sa, &map_a, &full[stage], kb * BK, m_blk * BM, b);  // box {64 k, 128 m}
                    } else {
                        for (int j = 0; j < BM / 64; j++)  // boxes {64 m, 64 k}
                            tma_load_3d(sa + j * (64 * BK * 2), &map_a, &full[stage], m_blk * BM + j * 64, kb * BK, b);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d(sb, &map_b, &full[stage], kb * BK, n_blk * BN, b);  // box {64 k, 256 n}
                    } else {
                        for (int j = 0; j < BN / 64; j++)  // boxes {64 n, 64 k}
                            tma_load_3d(sb + j * (64 * BK * 2), &map_b, &full[stage], n_blk * BN + j * 64, kb * BK, b);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN, p.in_bf16 != 0, p.a_mn_major, p.b_mn_major);
            // descriptors of stage 0; a stage and a 16-wide k step only move the address field.
            // K-major: 16 k-elements = 32 bytes further inside the swizzled 128-byte row.
            // MN-major: 16 k-rows of 128 bytes = 2048 bytes further; 64-element blocks 8 KB apart.
            const uint64_t da0 = p.a_mn_major ? make_smem_desc(smem_u32(smem_a), 64 * BK * 2, 1024) : make_smem_desc(smem_u32(smem_a), 16, 1024);
            const uint64_t db0 = p.b_mn_major ? make_smem_desc(smem_u32(smem_b), 64 * BK * 2, 1024) : make_smem_desc(smem_u32(smem_b), 16, 1024);
            const uint32_t a_step = p.a_mn_major ? 2048u : 32u, b_step = p.b_mn_major ? 2048u : 32u;
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, local++) {
                const int buf = local & 1;
                const uint32_t use = (uint32_t)(local >> 1);
                if (!(ok = mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const int kb0 = (unit / num_tiles) * p.kb_per_split;
                const int num_kb = min(total_kb, kb0 + p.kb_per_split) - kb0;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!(ok = mbar_wait(&full[stage], phase, abort_flag))) break;
                    tc_fence_after();
                    uint64_t da = desc_advance(da0, (uint32_t)(stage * kStageBytesA)), db = desc_advance(db0, (uint32_t)(stage * kStageBytesB));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        mma_f16(tmem_d, da, db, idesc, (kb | k) != 0);
                        da = desc_advance(da, a_step), db = desc_advance(db, b_step);
                    }
                    mma_commit(&empty[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) mma_commit(&tmem_full[buf]);
            }
        }
    } else {
        // ---- epilogue: warps 2..9. A warp may only read TMEM lanes 32*(warp%4) .. +31; the two warps sharing a lane
        // quarter split the tile's 256 columns between them. ----
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        uint4* stage = (uint4*)(smem + STAGES * (kStageBytesA + kStageBytesB) + 256) + (warp - 2) * (kStageBytesPerWarp / 16);
        int local = 0;
        bool ok = true;
        const bool vec_ok = p.d_bf16 || p.d_f16 ? (p.ldd % 8 == 0 && p.d_batch_stride % 8 == 0 && ((uintptr_t)p.d & 15) == 0)
                                                : (p.ldd % 4 == 0 && p.d_batch_stride % 4 == 0 && ((uintptr_t)p.d & 15) == 0);
        for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, local++) {
            const int buf = local & 1;
            const uint32_t use = (uint32_t)(local >> 1);
            int b, m_blk, n_blk;
            tile_coords(p, unit % num_tiles, b, m_blk, n_blk);
            const int split = unit / num_tiles;
            const int row = m_blk * BM + quarter * 32 + lane;
            const int col_base = n_blk * BN + col_half * (BN / 2);
            const long long row_off = (long long)b * p.d_batch_stride + (long long)row * p.ldd;
            const bool fast = __all_sync(0xffffffffu, aux_fast_path(p, row, col_base, vec_ok));  // warp-uniform: both drains load tensor memory warp-wide
            const uint16_t* ax_warp = (const uint16_t*)p.aux + (long long)b * p.aux_batch_stride + (long long)(row - lane) * p.ld_aux + col_base;
            uint4 raw[4];
            if (fast) aux_load(ax_warp, p.ld_aux, lane, raw);
            if (!(ok = mbar_wait(&tmem_full[buf], use & 1, abort_flag))) break;
            __syncwarp();
            tc_fence_after();
            const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + col_half * (BN / 2));
            if (fast) drain_tile_aux(p, tbase, row_off + col_base, ax_warp, raw, stage, lane);
            else drain_tile(p, tbase, row, row_off, col_base, b, split, vec_ok, stage, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    }

    // ---- teardown: every role leaves its loop (normally, or because the abort flag was raised) ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, LB_ERR_TIMEOUT);
        // give copies and MMAs still in flight a bounded time to land before shared/tensor memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- the same GEMM on CTA pairs ---------------------------------------------------------------------------------
// A cluster of two CTAs computes a 256 x 256 tile with tcgen05.mma.cta_group::2: CTA `rank` holds rows
// [128 rank, 128 rank + 128) of the A tile and columns [128 rank, 128 rank + 128) of the B tile, so every SM fetches
// only half of B from shared memory per instruction (8 KB instead of 12 KB), which lifts the one-CTA kernel's
// operand-fetch ceiling. The leader (rank 0) issues all MMAs; its commits arrive on the barriers of both CTAs. Both
// CTAs load their own tiles with TMA, counting bytes on the leader's `full` barrier. Each CTA drains its own 128
// accumulator rows; "accumulator drained" arrivals from both CTAs go to the leader's `tmem_empty` barrier.
constexpr int PSTAGES = 6;
constexpr int kPairStageBytesA = BM * BK * 2, kPairStageBytesB = (BN / 2) * BK * 2;
constexpr int kPairSmemBytes = PSTAGES * (kPairStageBytesA + kPairStageBytesB) + 1024 + 256 + kEpilogueStageBytes;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + PSTAGES * kPairStageBytesA;
    uint64_t* full = (uint64_t*)(smem + PSTAGES * (kPairStageBytesA + kPairStageBytesB));
    uint64_t* empty = full + PSTAGES;
    uint64_t* tmem_full = empty + PSTAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_base_slot = (uint32_t*)(tmem_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_tiles = p.tiles_m * p.tiles_n * p.batch;  // tiles_m counts 256-row pair tiles here
    const int total_kb = (p.K + BK - 1) / BK;
    const int num_units = num_tiles * p.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; s++) {
            mbar_init(&full[s], 1);   // the leader's expect_tx arrival; bytes of both CTAs
            mbar_init(&empty[s], 1);  // one commit from the leader's MMA thread
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_empty[s], 2 * kEpilogueWarps);  // used in the leader only: every epilogue warp of the pair
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // barriers of both CTAs are initialised and both allocations are done before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer (both CTAs) ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = pair; unit < num_units && ok; unit += num_pairs) {
                int b, m_blk, n_blk;
                tile_coords(p, unit % num_tiles, b, m_blk, n_blk);
                const int row0 = m_blk * 2 * BM + (int)rank * BM, col0 = n_blk * BN + (int)rank * (BN / 2);
                const int kb0 = (unit / num_tiles) * p.kb_per_split, kb1 = min(total_kb, kb0 + p.kb_per_split);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!(ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag))) break;
                    if (rank == 0) mbar_expect_tx(&full[stage], 2 * (kPairStageBytesA + kPairStageBytesB));
                    uint8_t* sa = smem_a + stage * kPairStageBytesA;
                    uint8_t* sb = smem_b + stage * kPairStageBytesB;
                    if (!p.a_mn_major) {
                        tma_load_3d_pair(sa, &map_a, &full[stage], kb * BK, row0, b);  // box {64 k, 128 m}
                    } else {
                        for (int j = 0; j < BM / 64; j++)  // boxes {64 m, 64 k}
                            tma_load_3d_pair(sa + j * (64 * BK * 2), &map_a, &full[stage], row0 + j * 64, kb * BK, b);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d_pair(sb, &map_b, &full[stage], kb * BK, col0, b);  // box {64 k, 128 n}
                    } else {
                        for (int j = 0; j < BN / 2 / 64; j++)  // boxes {64 n, 64 k}
                            tma_load_3d_pair(sb + j * (64 * BK * 2), &map_b, &full[stage], col0 + j * 64, kb * BK, b);
                    }
                    if (++stage == PSTAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
            // every commit aimed at this CTA's `empty` barriers has to land before the CTA may exit
            for (int s = 0; s < PSTAGES && ok; s++) {
                ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag);
                if (++stage == PSTAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (leader only) ----
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(2 * BM, BN, p.in_bf16 != 0, p.a_mn_major, p.b_mn_major);
            const uint64_t da0 = p.a_mn_major ? make_smem_desc(smem_u32(smem_a), 64 * BK * 2, 1024) : make_smem_desc(smem_u32(smem_a), 16, 1024);
            const uint64_t db0 = p.b_mn_major ? make_smem_desc(smem_u32(smem_b), 64 * BK * 2, 1024) : make_smem_desc(smem_u32(smem_b), 16, 1024);
            const uint32_t a_step = p.a_mn_major ? 2048u : 32u, b_step = p.b_mn_major ? 2048u : 32u;
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = true;
            for (int unit = pair; unit < num_units && ok; unit += num_pairs, local++) {
                const int buf = local & 1;
                const uint32_t use = (uint32_t)(local >> 1);
                if (!(ok = mbar_wait_cluster(&tmem_empty[buf], (use & 1) ^ 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
                const int kb0 = (unit / num_tiles) * p.kb_per_split;
                const int num_kb = min(total_kb, kb0 + p.kb_per_split) - kb0;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!(ok = mbar_wait(&full[stage], phase, abort_flag))) break;
                    tc_fence_after();
                    uint64_t da = desc_advance(da0, (uint32_t)(stage * kPairStageBytesA)), db = desc_advance(db0, (uint32_t)(stage * kPairStageBytesB));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        mma_f16_pair(tmem_d, da, db, idesc, (kb | k) != 0);
                        da = desc_advance(da, a_step), db = desc_advance(db, b_step);
                    }
                    mma_commit_pair(&empty[stage], 3);  // frees the stage in both CTAs
                    if (++stage == PSTAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) mma_commit_pair(&tmem_full[buf], 3);
            }
        }
    } else {
        // ---- epilogue: warps 2..9 of both CTAs, each CTA on its own 128 rows ----
        const int quarter = warp & 3;
        const int col_half = (warp - 2) >> 2;
        uint4* stage = (uint4*)(smem + PSTAGES * (kPairStageBytesA + kPairStageBytesB) + 256) + (warp - 2) * (kStageBytesPerWarp / 16);
        int local = 0;
        bool ok = true;
        const bool vec_ok = p.d_bf16 || p.d_f16 ? (p.ldd % 8 == 0 && p.d_batch_stride % 8 == 0 && ((uintptr_t)p.d & 15) == 0)
                                                : (p.ldd % 4 == 0 && p.d_batch_stride % 4 == 0 && ((uintptr_t)p.d & 15) == 0);
        for (int unit = pair; unit < num_units && ok; unit += num_pairs, local++) {
            const int buf = local & 1;
            const uint32_t use = (uint32_t)(local >> 1);
            int b, m_blk, n_blk;
            tile_coords(p, unit % num_tiles, b, m_blk, n_blk);
            const int split = unit / num_tiles;
            const int row = m_blk * 2 * BM + (int)rank * BM + quarter * 32 + lane;
            const int col_base = n_blk * BN + col_half * (BN / 2);
            const long long row_off = (long long)b * p.d_batch_stride + (long long)row * p.ldd;
            const bool fast = __all_sync(0xffffffffu, aux_fast_path(p, row, col_base, vec_ok));  // warp-uniform: both drains load tensor memory warp-wide
            const uint16_t* ax_warp = (const uint16_t*)p.aux + (long long)b * p.aux_batch_stride + (long long)(row - lane) * p.ld_aux + col_base;
            uint4 raw[4];
            if (fast) aux_load(ax_warp, p.ld_aux, lane, raw);
            if (!(ok = mbar_wait(&tmem_full[buf], use & 1, abort_flag))) break;
            __syncwarp();
            tc_fence_after();
            const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + col_half * (BN / 2));
            if (fast) drain_tile_aux(p, tbase, row_off + col_base, ax_warp, raw, stage, lane);
            else drain_tile(p, tbase, row, row_off, col_base, b, split, vec_ok, stage, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&tmem_empty[buf], 0);
        }
    }

    // ---- teardown: every role of both CTAs leaves its loop (normally, or because an abort flag was raised) ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, LB_ERR_TIMEOUT);
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
        __syncthreads();
    }
    cluster_sync();  // neither CTA releases shared or tensor memory while the other may still signal or compute into it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// Adds the split-K partial tiles in split order (fixed, so results are reproducible), applies the epilogue and rounds once.
__global__ void splitk_reduce(const float* __restrict__ partial, GemmArgs p) {
    const long long per = (long long)p.batch * p.M * p.N;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < per; i += (long long)gridDim.x * blockDim.x * 4) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const bool vec = p.N % 4 == 0;  // then a group of 4 never crosses a row
        for (int s = 0; s < p.splits; s++) {
            if (vec) {
                const float4 v = *(const float4*)(partial + s * per + i);
                acc[0] += v.x, acc[1] += v.y, acc[2] += v.z, acc[3] += v.w;
            } else {
                for (int j = 0; j < 4 && i + j < per; j++) acc[j] += partial[s * per + i + j];
            }
        }
        for (int j = 0; j < 4 && i + j < per; j++) {
            const long long e = i + j;
            const long long b = e / ((long long)p.M * p.N), r = (e / p.N) % p.M, c = e % p.N;
            float x = acc[j];
            if (p.epilogue == EPI_RELU) x = fmaxf(x, 0.0f);
            if (p.epilogue >= EPI_ADD) {
                const uint16_t a16 = ((const uint16_t*)p.aux)[b * p.aux_batch_stride + r * p.ld_aux + c];
                float prod, other;
                if (p.d_bf16) prod = __bfloat162float(__float2bfloat16_rn(x)), other = __uint_as_float((uint32_t)a16 << 16);
                else prod = __half2float(__float2half_rn(x)), other = __half2float(__ushort_as_half(a16));
                x = p.epilogue == EPI_ADD ? __fadd_rn(other, prod) : (other > 0.0f ? prod : 0.0f);
            }
            const long long at = b * p.d_batch_stride + r * p.ldd + c;
            if (p.d_bf16) ((__nv_bfloat16*)p.d)[at] = __float2bfloat16_rn(x);
            else if (p.d_f16) ((__half*)p.d)[at] = __float2half_rn(x);
            else ((float*)p.d)[at] = x;
        }
    }
}

// ---- SIMT GEMM: exact fp32 accumulation in contracting order -------------------------------------------------
template <class T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }

struct SimtArgs {
    int M, N, K, batch;
    long long a_sm, a_sk, a_sb, b_sk, b_sn, b_sb, ldd, d_sb;
    void* d;
    int d_dtype;
    int epilogue;
    const void* aux;  // EPI_ADD / EPI_MASK operand (16-bit, the output's dtype), rows ld_aux apart, batches aux_sb apart
    long long ld_aux, aux_sb;
};

constexpr int ST = 64, SK = 16;  // 64x64 output tile per 256 threads (4x4 each), 16-deep k slices

template <class T>
__global__ void __launch_bounds__(256) gemm_simt(const T* __restrict__ a, const T* __restrict__ b, const SimtArgs p) {
    __shared__ float sa[SK][ST + 1], sb[SK][ST + 1];
    const int bz = blockIdx.z, m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const T* ab = a + (long long)bz * p.a_sb;
    const T* bb = b + (long long)bz * p.b_sb;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += SK) {
        for (int i = threadIdx.x; i < ST * SK; i += 256) {
            // read along whichever of (row, k) is contiguous in memory
            int r, k;
            if (p.a_sk == 1) { k = i % SK; r = i / SK; } else { r = i % ST; k = i / ST; }
            int gm = m0 + r, gk = k0 + k;
            sa[k][r] = (gm < p.M && gk < p.K) ? load_as_float(ab + gm * p.a_sm + gk * p.a_sk) : 0.0f;
            int c;
            if (p.b_sn == 1) { c = i % ST; k = i / ST; } else { k = i % SK; c = i / SK; }
            int gn = n0 + c;
            gk = k0 + k;
            sb[k][c] = (gn < p.N && gk < p.K) ? load_as_float(bb + gk * p.b_sk + gn * p.b_sn) : 0.0f;
        }
        __syncthreads();
        const int kmax = min(SK, p.K - k0);
        for (int k = 0; k < kmax; k++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = sa[k][ty * 4 + i], bv[i] = sb[k][tx * 4 + i];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
            if (gm >= p.M || gn >= p.N) continue;
            float x = acc[i][j];
            if (p.epilogue == EPI_RELU) x = fmaxf(x, 0.0f);
            if (p.epilogue >= EPI_ADD) {  // the rounded product, then the second primitive on it (as the tensor-core kernels do)
                const uint16_t a16 = ((const uint16_t*)p.aux)[(long long)bz * p.aux_sb + (long long)gm * p.ld_aux + gn];
                float prod, other;
                if (p.d_dtype == LB_BF16) prod = __bfloat162float(__float2bfloat16_rn(x)), other = __uint_as_float((uint32_t)a16 << 16);
                else prod = __half2float(__float2half_rn(x)), other = __half2float(__ushort_as_half(a16));
                x = p.epilogue == EPI_ADD ? __fadd_rn(other, prod) : (other > 0.0f ? prod : 0.0f);
            }
            long long at = (long long)bz * p.d_sb + (long long)gm * p.ldd + gn;
            if (p.d_dtype == LB_F32) ((float*)p.d)[at] = x;
            else if (p.d_dtype == LB_BF16) ((__nv_bfloat16*)p.d)[at] = __float2bfloat16_rn(x);
            else ((__half*)p.d)[at] = __float2half_rn(x);
        }
}

// [batch, rows, cols] view of a rank-2/3 tensor
struct View3 {
    void* ptr;
    int dtype;
    long long batch, rows, cols, sb, sr, sc;
};
View3 view3(const lb_tensor& t, const char* what) {
    if (t.rank != 2 && t.rank != 3) fail(LB_ERR_INVALID, format("gemm: %s must have rank 2 or 3, got %d", what, t.rank));
    View3 v;
    v.ptr = t.ptr;
    v.dtype = t.dtype;
    int o = t.rank - 2;
    v.batch = o ? t.shape[0] : 1;
    v.sb = o ? t.stride[0] : 0;
    v.rows = t.shape[o];
    v.cols = t.shape[o + 1];
    v.sr = t.stride[o];
    v.sc = t.stride[o + 1];
    return v;
}

CUtensorMap make_map(const View3& v, bool contiguous_is_cols, int box_inner, int box_outer) {
    // dims innermost first: {contiguous, strided, batch}
    long long inner = contiguous_is_cols ? v.cols : v.rows, outer = contiguous_is_cols ? v.rows : v.cols;
    long long outer_stride = contiguous_is_cols ? v.sr : v.sc;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)v.batch};
    if (outer == 1) outer_stride = inner;
    cuuint64_t strides[2] = {(cuuint64_t)outer_stride * 2, (cuuint64_t)(v.batch > 1 ? v.sb : outer_stride * outer) * 2};
    cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
    cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap map;
    check_cu(driver().cuTensorMapEncodeTiled(&map, v.dtype == LB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                             3, v.ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
             "cuTensorMapEncodeTiled");
    return map;
}

}  // namespace

// Number of K ranges for a GEMM with few output tiles and a long K (weight gradients). 1 = no split. A cost model
// picks it: waves of (tile, range) units times the k-blocks of a range, at the measured 4 x 171 cycles per k-block of
// a 128 x 256 tile, plus the float32 partial tiles written by the GEMM and re-read by the reduction kernel at HBM
// speed and that kernel's launch. A split has to win by a tenth to be taken; each range keeps at least 16 k-blocks.
int gemm_splits(long long M, long long N, long long K, long long batch, int sms) {
    const long long tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch, total_kb = (K + BK - 1) / BK;
    if (tiles >= 4LL * sms || total_kb < 32) return 1;
    const double us_per_kb = 0.36, bytes_per_us = 5.0e6, launch_us = 6.0;
    auto cost = [&](int s) {
        const long long waves = (tiles * s + sms - 1) / sms, kb = (total_kb + s - 1) / s;
        double us = (double)waves * (double)kb * us_per_kb;
        if (s > 1) us += ((2.0 * s * 4 + 2) * (double)(batch * M * N)) / bytes_per_us + launch_us;
        return us;
    };
    int best = 1;
    double best_us = cost(1) * 0.9;
    for (int s = 2; s <= 32 && total_kb / s >= 16; s++)
        if (cost(s) < best_us) best = s, best_us = cost(s);
    return best;
}

// CTA pairs of gemm_tcgen05_pair that can be resident on `dev` at once (asked of the runtime once per device).
static int resident_pairs(const DeviceInfo& dev) {
    static std::mutex mutex;
    static std::map<int, int> cache;
    std::lock_guard<std::mutex> lock(mutex);
    auto it = cache.find(dev.device);
    if (it != cache.end()) return it->second;
    int pairs = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (dev.sms / 2), 1, 1), cfg.blockDim = dim3(kThreads, 1, 1), cfg.dynamicSmemBytes = kPairSmemBytes;
    if (cudaOccupancyMaxActiveClusters(&pairs, gemm_tcgen05_pair, &cfg) != cudaSuccess || pairs <= 0) {
        cudaGetLastError();
        pairs = 0;
    }
    return cache[dev.device] = pairs;
}

int gemm_model_splits(long long M, long long N, long long K, long long batch) { return gemm_splits(M, N, K, batch, sm_count_hint()); }

size_t gemm_scratch_bytes(long long M, long long N, long long K, long long batch) {
    const int s = gemm_splits(M, N, K, batch, sm_count_hint());
    return s > 1 ? (size_t)s * batch * M * N * 4 : 0;
}

void gemm(const lb_tensor& a_t, const lb_tensor& b_t, const lb_tensor& d_t, int epilogue, int kernel_choice, void* stream,
          void* scratch, size_t scratch_bytes, const lb_tensor* aux_t, const GemmTuning* tuning) {
    View3 a = view3(a_t, "a"), b = view3(b_t, "b"), d = view3(d_t, "output");
    if (epilogue < EPI_NONE || epilogue > EPI_MASK) fail(LB_ERR_INVALID, "gemm: unknown epilogue");
    View3 aux{};
    if (epilogue >= EPI_ADD) {
        if (!aux_t || !aux_t->ptr) fail(LB_ERR_INVALID, "gemm: the add / mask epilogue needs its operand tensor");
        aux = view3(*aux_t, "epilogue operand");
        if (aux.dtype != d.dtype || aux.rows != d.rows || aux.cols != d.cols || aux.batch != d.batch || (aux.sc != 1 && aux.cols > 1))
            fail(LB_ERR_INVALID, "gemm: the epilogue operand must be a row-major tensor of the output's shape and dtype");
        if (d.dtype != LB_BF16 && d.dtype != LB_F16)
            fail(LB_ERR_UNSUPPORTED, "gemm: the add / mask epilogue is built for 16-bit outputs of the tensor-core kernels");
    }
    if (a.dtype != b.dtype) fail(LB_ERR_INVALID, "gemm: operands must share a dtype (no hidden casts)");
    if (a.cols != b.rows || a.batch != b.batch || d.rows != a.rows || d.cols != b.cols || d.batch != a.batch)
        fail(LB_ERR_INVALID, format("gemm: shapes [%lld,%lld,%lld] x [%lld,%lld,%lld] -> [%lld,%lld,%lld] do not match",
                                    a.batch, a.rows, a.cols, b.batch, b.rows, b.cols, d.batch, d.rows, d.cols));
    if (d.sc != 1 && d.cols > 1) fail(LB_ERR_UNSUPPORTED, "gemm: the output must be row-major");
    if (a.dtype != LB_F32 && a.dtype != LB_BF16 && a.dtype != LB_F16) fail(LB_ERR_UNSUPPORTED, "gemm: float16, bfloat16 or float32 operands");
    if (d.dtype != LB_F32 && d.dtype != a.dtype) fail(LB_ERR_INVALID, "gemm: the output is float32 (the accumulator) or the operands' dtype");
    const long long M = a.rows, N = b.cols, K = a.cols, batch = a.batch;
    if (M == 0 || N == 0 || batch == 0) return;
    driver();
    cudaStream_t s = (cudaStream_t)stream;

    auto major = [](const View3& v, bool& cols_contig) {
        if (v.sc == 1 || v.cols == 1) { cols_contig = true; return true; }
        if (v.sr == 1 || v.rows == 1) { cols_contig = false; return true; }
        return false;
    };
    bool a_cols, b_cols;
    bool tc_ok = (a.dtype == LB_BF16 || a.dtype == LB_F16) && K > 0 && major(a, a_cols) && major(b, b_cols) && kernel_choice != 2;
    if (tc_ok) {
        // TMA: 16-byte aligned base, strides multiples of 16 bytes
        auto aligned = [](const View3& v, bool cols_contig) {
            long long inner = cols_contig ? v.cols : v.rows, outer = cols_contig ? v.rows : v.cols;
            long long ld = outer == 1 ? inner : (cols_contig ? v.sr : v.sc);
            return ((uintptr_t)v.ptr & 15) == 0 && ld % 8 == 0 && ld >= inner && (v.batch == 1 || v.sb % 8 == 0);
        };
        tc_ok = aligned(a, a_cols) && aligned(b, b_cols) && M <= INT32_MAX && N <= INT32_MAX && K <= INT32_MAX;
    }
    if (kernel_choice == 1 && !tc_ok) fail(LB_ERR_UNSUPPORTED, "gemm: the tcgen05 kernels need bfloat16 or float16 operands with a unit stride and 16-byte aligned rows");

    if (tc_ok) {
        GemmArgs p{};
        p.M = (int)M, p.N = (int)N, p.K = (int)K, p.batch = (int)batch;
        p.a_mn_major = !a_cols;  // A [M, K]: contiguous columns = K-major
        p.b_mn_major = b_cols;   // B [K, N]: contiguous columns = N-major
        p.d = d.ptr;
        p.d_bf16 = d.dtype == LB_BF16;
        p.d_f16 = d.dtype == LB_F16;
        p.in_bf16 = a.dtype == LB_BF16;
        p.ldd = d.sr;
        p.d_batch_stride = d.batch > 1 ? d.sb : 0;
        p.epilogue = epilogue;
        p.aux = aux.ptr, p.ld_aux = aux.sr, p.aux_batch_stride = aux.batch > 1 ? aux.sb : 0;
        p.status = status_word();
        // CTA pairs (256 x 256 tiles over two SMs) whenever there is more than one 128-row block; kernel_choice 3 keeps
        // the one-CTA kernel
        const bool pairs = M > BM && kernel_choice != 3;
        const int tile_rows = pairs ? 2 * BM : BM;
        p.tiles_m = (int)((M + tile_rows - 1) / tile_rows);
        p.tiles_n = (int)((N + BN - 1) / BN);
        p.group_m = tuning && tuning->group_m > 0 ? tuning->group_m : (pairs ? 8 : 16);
        // K-major operands: box {64 k, rows}; MN-major: box {64 mn, 64 k}
        CUtensorMap map_a = p.a_mn_major ? make_map(a, false, 64, BK) : make_map(a, true, BK, BM);
        // B as the N x K operand: "rows" of the operand are B's columns
        View3 bt = b;  // transposed view: rows = N, cols = K
        bt.rows = b.cols, bt.cols = b.rows, bt.sr = b.sc, bt.sc = b.sr;
        CUtensorMap map_b = p.b_mn_major ? make_map(bt, false, 64, BK) : make_map(bt, true, BK, pairs ? BN / 2 : BN);
        const DeviceInfo& dev = device_info();
        if (first_use_on_device((const void*)gemm_tcgen05_pair)) {
            LB_CUDA(cudaFuncSetAttribute(gemm_tcgen05, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            LB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
        }
        const int max_pairs = resident_pairs(dev);
        long long tiles = (long long)p.tiles_m * p.tiles_n * batch;
        const int sms = dev.sms;
        p.splits = 1;
        p.kb_per_split = (int)((K + BK - 1) / BK);
        p.partial = (float*)scratch;
        int want = scratch ? gemm_splits(M, N, K, batch, sms) : 1;
        if (tuning && tuning->splits > 0) want = scratch ? tuning->splits : 1;  // a tuned split count, if the scratch holds it
        if (want > 1 && scratch_bytes >= (size_t)want * batch * M * N * 4 && ((uintptr_t)scratch & 15) == 0) {
            const int total_kb = p.kb_per_split;
            p.kb_per_split = (total_kb + want - 1) / want;
            p.splits = (total_kb + p.kb_per_split - 1) / p.kb_per_split;
        }
        if (pairs) {
            const int resident = max_pairs > 0 ? max_pairs : sms / 2;
            int grid = 2 * (int)std::min<long long>(tiles * p.splits, resident);
            gemm_tcgen05_pair<<<grid, kThreads, kPairSmemBytes, s>>>(map_a, map_b, p);
        } else {
            int grid = (int)std::min<long long>(tiles * p.splits, sms);
            gemm_tcgen05<<<grid, kThreads, kSmemBytes, s>>>(map_a, map_b, p);
        }
        LB_CUDA(cudaGetLastError());
        if (p.splits > 1) {
            long long groups = ((long long)batch * M * N + 3) / 4;
            splitk_reduce<<<(unsigned)std::min<long long>((groups + 255) / 256, sms * 8), 256, 0, s>>>(p.partial, p);
            LB_CUDA(cudaGetLastError());
        }
        return;
    }

    SimtArgs p{};
    if (epilogue >= EPI_ADD) p.aux = aux.ptr, p.ld_aux = aux.sr, p.aux_sb = aux.batch > 1 ? aux.sb : 0;
    p.M = (int)M, p.N = (int)N, p.K = (int)K, p.batch = (int)batch;
    p.a_sm = a.sr, p.a_sk = a.sc, p.a_sb = a.batch > 1 ? a.sb : 0;
    p.b_sk = b.sr, p.b_sn = b.sc, p.b_sb = b.batch > 1 ? b.sb : 0;
    p.ldd = d.sr, p.d_sb = d.batch > 1 ? d.sb : 0;
    p.d = d.ptr, p.d_dtype = d.dtype, p.epilogue = epilogue;
    dim3 grid((unsigned)((N + ST - 1) / ST), (unsigned)((M + ST - 1) / ST), (unsigned)batch);
    if (a.dtype == LB_F32) gemm_simt<float><<<grid, 256, 0, s>>>((const float*)a.ptr, (const float*)b.ptr, p);
    else if (a.dtype == LB_BF16) gemm_simt<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)a.ptr, (const __nv_bfloat16*)b.ptr, p);
    else gemm_simt<__half><<<grid, 256, 0, s>>>((const __half*)a.ptr, (const __half*)b.ptr, p);
    LB_CUDA(cudaGetLastError());
}

}  // namespace lb

extern "C" {

int lb_gemm(const lb_tensor* a, const lb_tensor* b, const lb_gemm_out* out, const lb_gemm_cfg* cfg, void* stream) {
    return lb::guarded([&] {
        if (!a || !b || !out) lb::fail(LB_ERR_INVALID, "lb_gemm: null argument");
        lb::GemmTuning tuning{cfg ? cfg->splits : 0, cfg ? cfg->group_m : 0};
        lb::gemm(*a, *b, out->product, out->epilogue, cfg ? cfg->kernel : 0, stream, cfg ? cfg->scratch : nullptr,
                 cfg ? cfg->scratch_bytes : 0, out->epilogue >= 2 ? &out->aux : nullptr, &tuning);
    });
}

size_t lb_gemm_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t batch) { return lb::gemm_scratch_bytes(m, n, k, batch); }

int lb_device_status(void) {
    int status = 0;
    int rc = lb::guarded([&] { status = lb::read_status(); });
    if (rc != LB_OK) return rc;
    if (status != 0) lb::set_last_error("a device-side wait ran out of its poll budget (kernel wound down early)");
    return status;
}
}
