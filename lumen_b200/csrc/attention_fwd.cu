// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [causal]) V with online softmax and an optional
// float32 log-sum-exp, the counterpart of the reference's Ampere FA-2 forward kernel behind its ATTENTION hook
// (lumen/codegen/attention/cuda/ampere/forward.py:810-1157, lumen/codegen/attention/cuda/mod.rs:261-294) and of the
// traced program it replaces (lumen/functional/attention/flash.py:30-49).
//
// One CTA per (128-query tile, head, batch), two CTAs per SM. Q, K, V are read in place from their [B, S, N, H] views
// by TMA (4-d tensor maps, 128-byte swizzle). Per 128-key tile:
//   S = Q K^T            tcgen05.mma, both operands K-major in shared memory, fp32 scores in tensor memory
//   P = exp2(S*c - m)    four softmax warps, one query row per thread holding the whole row of 128 scores in registers
//                        (one tensor-memory round trip per tile); P is rounded to bf16 and written back over S
//                        (head dim 128) or into 64 columns of its own (head dim 64: S 128 + O 64 + P 64 = 256)
//   O += P V             tcgen05.mma with P as the TMEM operand and V as an MN-major shared-memory operand; O stays
//                        in tensor memory for the whole CTA
// m is a reference maximum that is raised lazily (softmax_rows). At head dim 128 the tensor core, the softmax warps
// and the TMA producer of ONE CTA work in turn (S and O are single-buffered: 256 columns) and the other CTA on the
// SM fills the gaps. At head dim 64 S is free as soon as the softmax threads hold it in registers, so S(j + 1) is
// computed during softmax(j) and only P(j) V(j) sits between two softmax passes. Probabilities are rounded to bf16 before the PV product as the traced program does (flash.py:38-45); sums
// and the output accumulate in fp32. Every barrier wait is bounded.
#include <mutex>
#include <type_traits>

#include "device.h"
#include "sm100.cuh"

namespace lb {
namespace {

using namespace sm100;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int BQ = 128, BKV = 128;
// warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: softmax (thread = query row). 256 tensor-memory columns (S 128,
// O up to 128) and at most 96 KB of shared memory per CTA, so that TWO CTAs share an SM: one CTA's prologue, epilogue
// and softmax are covered by the other CTA's MMAs.
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;

struct FwdArgs {
    int B, N, Nkv, Sq, Sk;
    int causal;
    long long causal_offset;  // key j is visible to query i iff j <= i + causal_offset
    float scale_log2;         // scale * log2(e)
    void* o;                  // bf16 [B, Sq, N, D] view
    long long o_sb, o_ss, o_sn;
    float* lse;               // [B, N, Sq] or null
    int* status;
};

template <int D, int NS>
struct FwdSmem {
    static constexpr int kTile = BKV * D * 2;  // one Q, K or V tile
    static constexpr int kBytes = (1 + 2 * NS) * kTile + 1024 + 256;  // Q, NS stages of K and of V, alignment, barriers
};

// The softmax warpgroup of the one-warpgroup kernel (thread = query row). The output accumulates in tensor memory
// (O += P V by the tensor core), so the thread's registers hold a whole row of scores: ONE tensor-memory round trip
// per key tile instead of one per 32 columns and pass. Probabilities are taken against a reference maximum that is
// only raised when the row's maximum outgrows it by more than 2^8 (then O and the running sum are rescaled, after
// the previous tile's product has landed); a stale reference changes no result beyond rounding, since it cancels
// in O / l and in the log-sum-exp.
template <int D>
__device__ __forceinline__ void softmax_rows(const FwdArgs& p, int n_kv, long long q_row, uint32_t lane_addr, uint32_t tmem_s,
                                               uint32_t tmem_o, uint64_t* s_full, uint64_t* p_ready, uint64_t* pv_full,
                                               volatile int* abort_flag, int head, int batch, uint32_t tmem_p, uint64_t* s_empty) {
    constexpr float kRaise = 8.0f;  // log2 of the largest probability tolerated before the reference is raised
    const uint32_t s_addr = tmem_s + lane_addr, o_addr = tmem_o + lane_addr, p_addr = tmem_p + lane_addr;
    const bool separate_p = tmem_p != tmem_s;  // P has columns of its own (head dim 64)
    const long long row_last = p.causal ? min((long long)p.Sk - 1, q_row + p.causal_offset) : (long long)p.Sk - 1;
    float m_ref = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; j++) {
        if (!(ok = mbar_wait(s_full, (uint32_t)j & 1, abort_flag))) break;
        __syncwarp();
        tc_fence_after();
        uint32_t x[BKV];
#pragma unroll
        for (int c = 0; c < BKV / 32; c++) tmem_ld_32x32(s_addr + c * 32, x + c * 32);
        tmem_ld_wait();
        if (separate_p) {  // S may be overwritten by the next tile's product
            tc_fence_before();
            mbar_arrive(s_empty);
        }
        const int limit = (int)min(row_last - (long long)j * BKV, (long long)BKV);  // tile-relative index of the last visible key
        const bool masked_tile = __any_sync(0xffffffffu, limit < BKV - 1);
        if (masked_tile) {
#pragma unroll
            for (int i = 0; i < BKV; i++)
                if (i > limit) x[i] = 0xff800000u;  // -inf: drops out of the maximum, exp2 gives 0
        }
        // eight independent chains: with one or two warps per scheduler a single chain of 128 dependent maxima (or sums,
        // below) would run at the instruction latency, not the issue rate
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; i++) mx[i] = __uint_as_float(x[i]);
#pragma unroll
        for (int i = 8; i < BKV; i++) mx[i & 7] = fmaxf(mx[i & 7], __uint_as_float(x[i]));
        const float tile_max = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        const float m_new = tile_max * p.scale_log2;
        const bool raise = m_new > m_ref + kRaise;  // also the first finite maximum (m_ref = -inf)
        if (__any_sync(0xffffffffu, raise)) {
            const float alpha = raise ? fast_exp2(m_ref - m_new) : 1.0f;  // 0 when nothing was accumulated yet
            if (raise) m_ref = m_new, l *= alpha;
            if (j > 0) {
                // O *= alpha, once the previous tile's product has landed (tensor-memory accesses are warp-wide)
                if (!(ok = mbar_wait(pv_full, (uint32_t)(j - 1) & 1, abort_flag))) break;
                __syncwarp();
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 32; c++) {
                    uint32_t v[32];
                    tmem_ld_32x32(o_addr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 r = __fmul2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), make_float2(alpha, alpha));
                        v[i] = __float_as_uint(r.x), v[i + 1] = __float_as_uint(r.y);
                    }
                    tmem_st_32x16(o_addr + c * 32, v);
                    tmem_st_32x16(o_addr + c * 32 + 16, v + 16);
                }
            }
        }
        const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
        // two keys per instruction (packed float32 FMA / ADD of sm_100), four independent pairs of partial sums
        float2 sums[4] = {{0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}};
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-m_use, -m_use);
        if (separate_p && j > 0) {
            // P(j) goes where P(j - 1) was: the product that read it has to have completed (it has, unless this row's
            // softmax overtook the tensor pipe)
            if (!(ok = mbar_wait(pv_full, (uint32_t)(j - 1) & 1, abort_flag))) break;
            __syncwarp();
            tc_fence_after();
        }
#pragma unroll
        for (int c = 0; c < BKV / 32; c++) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                const float2 arg = __ffma2_rn(make_float2(__uint_as_float(x[c * 32 + i]), __uint_as_float(x[c * 32 + i + 1])), scale2, shift2);
                const float2 pr = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                __nv_bfloat162 h = __floats2bfloat162_rn(pr.x, pr.y);  // low half = the even key
                packed[i / 2] = *(uint32_t*)&h;
                sums[(i / 2) & 3] = __fadd2_rn(sums[(i / 2) & 3], pr);  // the normaliser sums the float32 probabilities
            }
            tmem_st_32x16(p_addr + c * 16, packed);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(p_ready);
        const float2 s01 = __fadd2_rn(sums[0], sums[1]), s23 = __fadd2_rn(sums[2], sums[3]);
        l += (s01.x + s01.y) + (s23.x + s23.y);
    }
    if (n_kv > 0) ok = ok && mbar_wait(pv_full, (uint32_t)(n_kv - 1) & 1, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return;
    tc_fence_after();
    const bool live = q_row < p.Sq;
    const float inv = 1.0f / l;  // a row that sees no key is 0 / 0 in the traced program: NaN
    uint16_t* out = (uint16_t*)p.o + (long long)batch * p.o_sb + q_row * p.o_ss + (long long)head * p.o_sn;
    const bool vec = (p.o_sb % 8 == 0) && (p.o_ss % 8 == 0) && (p.o_sn % 8 == 0) && (((uintptr_t)p.o & 15) == 0);
#pragma unroll
    for (int c = 0; c < D / 32; c++) {
        uint32_t v[32];
        if (n_kv > 0) {
            tmem_ld_32x32(o_addr + c * 32, v);
            tmem_ld_wait();
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = 0u;
        }
        if (live) {
#pragma unroll
            for (int d = 0; d < 32; d += 8) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[d + 2 * q]) * inv, __uint_as_float(v[d + 2 * q + 1]) * inv);
                    w[q] = *(uint32_t*)&h;
                }
                if (vec) {
                    *(uint4*)(out + c * 32 + d) = make_uint4(w[0], w[1], w[2], w[3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        out[c * 32 + d + 2 * q] = (uint16_t)(w[q] & 0xffff);
                        out[c * 32 + d + 2 * q + 1] = (uint16_t)(w[q] >> 16);
                    }
                }
            }
        }
    }
    if (live && p.lse) p.lse[((long long)batch * p.N + head) * p.Sq + q_row] = (m_ref + log2f(l)) * 0.6931471805599453f;
}

template <int D, int NS>
__global__ void __launch_bounds__(kThreads, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const FwdArgs p) {
    constexpr int kTile = FwdSmem<D, NS>::kTile;
    static_assert(NS == 1 || NS == 2, "one or two K/V stages");
    static_assert(128 + D <= kTmemCols, "S and O have to fit the CTA's tensor-memory columns");
    constexpr int kHalf = 128 * 128;  // bytes of one 64-wide (128-byte) column block of a 128-row tile
    constexpr int DB = D / 64;        // 64-element blocks along the head dimension
    // key tile j uses K/V stage j % NS (barrier parity (j / NS) & 1); the S/P buffer and O are single (parity j & 1)
    auto kst = [](int j) { return j % NS; };
    auto kph = [](int j) { return (uint32_t)(j / NS) & 1u; };
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sq = smem;
    uint8_t* sk = smem + kTile;             // NS stages
    uint8_t* sv = smem + (1 + NS) * kTile;  // NS stages
    uint64_t* bars = (uint64_t*)(smem + (1 + 2 * NS) * kTile);
    uint64_t* q_full = bars;         // 1
    uint64_t* k_full = bars + 1;     // NS
    uint64_t* k_empty = bars + 3;    // NS
    uint64_t* v_full = bars + 5;     // NS
    uint64_t* v_empty = bars + 7;    // NS
    uint64_t* s_full = bars + 9;     // S(j) is in tensor memory
    uint64_t* p_ready = bars + 10;   // the softmax warps wrote P(j) (128 arrivals)
    uint64_t* pv_full = bars + 11;   // O += P(j) V(j) has completed
    uint64_t* s_empty = bars + 12;   // head dim 64: every softmax thread has loaded S(j) (128 arrivals)
    uint32_t* tmem_slot = (uint32_t*)(bars + 13);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_tile = gridDim.x - 1 - blockIdx.x;  // longest (most keys under a causal mask) first
    const int head = blockIdx.y, batch = blockIdx.z;
    const int kv_head = head / (p.N / p.Nkv);
    const int q0 = q_tile * BQ;
    // keys this tile can see
    long long last_key = p.causal ? min((long long)p.Sk - 1, (long long)q0 + BQ - 1 + p.causal_offset) : (long long)p.Sk - 1;
    const int n_kv = last_key < 0 ? 0 : (int)(last_key / BKV) + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < NS; s++) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_ready, 128);
        mbar_init(pv_full, 1);
        mbar_init(s_empty, 128);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // At head dim 64 the CTA's 256 columns hold S (128), O (64) and P (64) side by side: S is free as soon as the
    // softmax threads have loaded it, so S(j + 1) is computed during softmax(j) instead of behind P(j) V(j).
    // At head dim 128 P overwrites the first 64 columns of S.
    constexpr bool kSeparateP = 128 + D + 64 <= kTmemCols;
    const uint32_t tmem_s = tmem_base;        // S
    const uint32_t tmem_o = tmem_base + 128;  // O: D columns
    const uint32_t tmem_p = kSeparateP ? tmem_base + 128 + D : tmem_s;

    if (warp == 0) {
        if (lane == 0 && n_kv > 0) {
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            mbar_expect_tx(q_full, kTile);
            for (int d = 0; d < DB; d++) tma_load_4d(sq + d * kHalf, &map_q, q_full, d * 64, head, q0, batch);
            bool ok = true;
            for (int j = 0; j < n_kv && ok; j++) {
                const int st = kst(j);
                const uint32_t ph = kph(j);
                if (!(ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag))) break;
                mbar_expect_tx(&k_full[st], kTile);
                for (int d = 0; d < DB; d++) tma_load_4d(sk + st * kTile + d * kHalf, &map_k, &k_full[st], d * 64, kv_head, j * BKV, batch);
                if (!(ok = mbar_wait(&v_empty[st], ph ^ 1, abort_flag))) break;
                mbar_expect_tx(&v_full[st], kTile);
                for (int d = 0; d < DB; d++) tma_load_4d(sv + st * kTile + d * kHalf, &map_v, &v_full[st], d * 64, kv_head, j * BKV, batch);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_kv > 0) {
            const uint32_t idesc_s = make_idesc(BQ, BKV, true, false, false);
            const uint32_t idesc_pv = make_idesc(BQ, D, true, false, true);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            // Descriptors are built once and advanced by adds: the one issuing thread is otherwise bound by its own
            // integer instructions, not by the tensor pipe.
            const uint64_t dq0 = make_smem_desc(smem_u32(sq), 16, 1024), dk0 = make_smem_desc(smem_u32(sk), 16, 1024);
            const uint64_t dv0 = make_smem_desc(smem_u32(sv), kHalf, 1024);
            auto issue_s = [&](int j) -> bool {
                const int st = kst(j);
                if (!mbar_wait(&k_full[st], kph(j), abort_flag)) return false;
                tc_fence_after();
                const uint64_t kd = desc_advance(dk0, (uint32_t)(st * kTile));
#pragma unroll
                for (int k = 0; k < D / 16; k++) {
                    const uint32_t off = (uint32_t)((k / 4) * kHalf + (k % 4) * 32);
                    mma_f16(tmem_s, desc_advance(dq0, off), desc_advance(kd, off), idesc_s, k != 0);
                }
                mma_commit(&k_empty[st]);
                mma_commit(s_full);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_kv && ok; j++) {
                const int vs = kst(j);
                if (kSeparateP && j + 1 < n_kv) {
                    if (!(ok = mbar_wait(s_empty, (uint32_t)j & 1, abort_flag))) break;
                    tc_fence_after();
                    if (!(ok = issue_s(j + 1))) break;
                }
                if (!(ok = mbar_wait(p_ready, (uint32_t)j & 1, abort_flag))) break;
                if (!(ok = mbar_wait(&v_full[vs], kph(j), abort_flag))) break;
                tc_fence_after();
                const uint64_t vd = desc_advance(dv0, (uint32_t)(vs * kTile));
#pragma unroll
                for (int k = 0; k < BKV / 16; k++) {
                    // O += P V. P: 16 keys = 8 packed columns per step. V (MN-major): 16 key rows of 128 bytes = 2048 bytes
                    // per step, 64-wide head-dimension blocks kHalf apart.
                    mma_f16_ts(tmem_o, tmem_p + k * 8, desc_advance(vd, k * 2048), idesc_pv, (j | k) != 0);
                }
                mma_commit(&v_empty[vs]);
                mma_commit(pv_full);
                if (!kSeparateP && j + 1 < n_kv) ok = issue_s(j + 1);  // behind PV(j), which reads P from the S buffer: the tensor pipe runs in order
            }
        }
    } else {
        // ---- softmax warps: thread = query row ----
        const int quarter = warp & 3;
        const long long q_row = (long long)q0 + quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        softmax_rows<D>(p, n_kv, q_row, lane_addr, tmem_s, tmem_o, s_full, p_ready, pv_full, abort_flag, head, batch, tmem_p, s_empty);
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, LB_ERR_TIMEOUT);
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// 4-d tensor map over a [B, S, N, H] view: dims innermost first {H, N, S, B}; box = 64 head-dim elements x `box_rows` rows.
CUtensorMap make_bsnh_map(const lb_tensor& t, const char* what, int box_rows = 128) {
    if (t.rank != 4) fail(LB_ERR_INVALID, format("attention: %s must be a [B, S, N, H] tensor", what));
    if (t.dtype != LB_BF16) fail(LB_ERR_UNSUPPORTED, format("attention: %s must be bfloat16", what));
    if (t.stride[3] != 1 || ((uintptr_t)t.ptr & 15) || t.stride[0] % 8 || t.stride[1] % 8 || t.stride[2] % 8)
        fail(LB_ERR_UNSUPPORTED, format("attention: %s needs a unit head-dim stride and 16-byte aligned rows", what));
    cuuint64_t dims[4] = {(cuuint64_t)t.shape[3], (cuuint64_t)t.shape[2], (cuuint64_t)t.shape[1], (cuuint64_t)t.shape[0]};
    cuuint64_t strides[3] = {(cuuint64_t)t.stride[2] * 2, (cuuint64_t)t.stride[1] * 2, (cuuint64_t)t.stride[0] * 2};
    // size-1 dimensions may carry any stride: give TMA one it accepts
    if (t.shape[2] == 1) strides[0] = (cuuint64_t)t.shape[3] * 2;
    if (t.shape[1] == 1) strides[1] = strides[0] * t.shape[2];
    if (t.shape[0] == 1) strides[2] = strides[1] * t.shape[1];
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap map;
    check_cu(driver().cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, elem,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
             "cuTensorMapEncodeTiled(attention)");
    return map;
}

}  // namespace

CUtensorMap attention_map_rows(const lb_tensor& t, const char* what, int box_rows) { return make_bsnh_map(t, what, box_rows); }

void attention_fwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                   const lb_tensor* lse, void* stream) {
    if (q.rank != 4 || k.rank != 4 || v.rank != 4) fail(LB_ERR_INVALID, "attention: operands must be [B, S, N, H] tensors");
    if (q.shape[0] == 0 || q.shape[1] == 0 || q.shape[2] == 0) return;  // nothing to compute: no launch (and no tensor map over nothing)
    CUtensorMap mq = make_bsnh_map(q, "query"), mk = make_bsnh_map(k, "key"), mv = make_bsnh_map(v, "value");
    const long long B = q.shape[0], Sq = q.shape[1], N = q.shape[2], D = q.shape[3];
    const long long Sk = k.shape[1], Nkv = k.shape[2];
    if (k.shape[0] != B || v.shape[0] != B || k.shape[3] != D || v.shape[1] != Sk || v.shape[2] != Nkv || Nkv == 0 || N % Nkv)
        fail(LB_ERR_INVALID, "attention: shapes are not [B,Sq,N,H], [B,Sk,Nkv,H], [B,Sk,Nkv,Hv] with N a multiple of Nkv");
    if (v.shape[3] != D) fail(LB_ERR_UNSUPPORTED, "attention: value head dim must equal the query head dim");
    if (D != 64 && D != 128) fail(LB_ERR_UNSUPPORTED, "attention: head dims 64 and 128 have a tcgen05 kernel");
    if (o.rank != 4 || o.dtype != LB_BF16 || o.shape[0] != B || o.shape[1] != Sq || o.shape[2] != N || o.shape[3] != D || o.stride[3] != 1)
        fail(LB_ERR_INVALID, "attention: the output must be a bfloat16 [B, Sq, N, H] view with a unit head-dim stride");
    if (lse) check_dense(*lse, LB_F32, {B, N, Sq}, "attention log-sum-exp");
    if (!(desc.scale > 0.0f)) fail(LB_ERR_UNSUPPORTED, "attention: the softmax scale must be positive");
    if (B == 0 || Sq == 0 || N == 0) return;
    FwdArgs p{};
    p.B = (int)B, p.N = (int)N, p.Nkv = (int)Nkv, p.Sq = (int)Sq, p.Sk = (int)Sk;
    p.causal = desc.causal;
    p.causal_offset = desc.causal_offset;
    p.scale_log2 = desc.scale * 1.4426950408889634f;
    p.o = o.ptr, p.o_sb = o.stride[0], p.o_ss = o.stride[1], p.o_sn = o.stride[2];
    p.lse = lse ? (float*)lse->ptr : nullptr;
    p.status = status_word();
    dim3 grid((unsigned)((Sq + BQ - 1) / BQ), (unsigned)N, (unsigned)B);
    cudaStream_t s = (cudaStream_t)stream;
    // One warpgroup, O in tensor memory, two CTAs per SM: two K/V stages at head dim 64, one at head dim 128 (96 KB per CTA)
    if (D == 128) {
        if (first_use_on_device((const void*)attention_fwd_kernel<128, 1>))
            LB_CUDA(cudaFuncSetAttribute(attention_fwd_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<128, 1>::kBytes));
        attention_fwd_kernel<128, 1><<<grid, kThreads, FwdSmem<128, 1>::kBytes, s>>>(mq, mk, mv, p);
    } else {
        if (first_use_on_device((const void*)attention_fwd_kernel<64, 2>))
            LB_CUDA(cudaFuncSetAttribute(attention_fwd_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<64, 2>::kBytes));
        attention_fwd_kernel<64, 2><<<grid, kThreads, FwdSmem<64, 2>::kBytes, s>>>(mq, mk, mv, p);
    }
    LB_CUDA(cudaGetLastError());
}

}  // namespace lb

namespace lb {
void attention_simt_fwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                        const lb_tensor* lse, void* stream);

// bfloat16 with head dim 64/128 and TMA-addressable views runs on tensor cores; everything else on CUDA cores
bool attention_on_tensor_cores(const lb_tensor& q, const lb_tensor& k, const lb_tensor& v) {
    auto ok = [](const lb_tensor& t) {
        return t.rank == 4 && t.dtype == LB_BF16 && t.stride[3] == 1 && ((uintptr_t)t.ptr & 15) == 0 && t.stride[0] % 8 == 0 &&
               t.stride[1] % 8 == 0 && t.stride[2] % 8 == 0;
    };
    return ok(q) && ok(k) && ok(v) && (q.shape[3] == 64 || q.shape[3] == 128) && v.shape[3] == q.shape[3];
}

void attention_forward(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                       const lb_tensor* lse, void* stream) {
    if (attention_on_tensor_cores(q, k, v)) attention_fwd(desc, q, k, v, o, lse, stream);
    else attention_simt_fwd(desc, q, k, v, o, lse, stream);
}
}  // namespace lb

extern "C" int lb_attention_fwd(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                                const lb_tensor* o, const lb_tensor* lse, void* stream) {
    return lb::guarded([&] {
        if (!desc || !q || !k || !v || !o) lb::fail(LB_ERR_INVALID, "lb_attention_fwd: null argument");
        lb::attention_forward(*desc, *q, *k, *v, *o, lse, stream);
    });
}
