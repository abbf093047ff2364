// Flash-attention backward for sm_100a: FlashAttention-2's recompute-from-log-sum-exp backward as the reference
// traces it (lumen/functional/attention/flash.py:51-85) and as its Triton backend runs it in deterministic mode
// (dkdv_kernel + dq_kernel, lumen/codegen/attention/triton/kernel.py:108-264); the reference's CUDA backend has a
// backward kernel that is never launched (lumen/codegen/attention/README.md:27-28).
//
//   delta = rowsum(dO * O)                                    attention_delta (CUDA cores, HBM bound)
//   P^T   = exp(scale * K Q^T - lse),  dP^T = V dO^T           per (key tile, query tile)
//   dS^T  = P^T * (dP^T - delta) * scale   (rounded to bf16),  P^T rounded to bf16
//   dV   += P^T dO,  dK += dS^T Q,  dQ += dS K
//
// One kernel template runs in two modes. Both keep a 128-row pair of tiles resident in shared memory, stream
// 64-row tile pairs through a 3-stage TMA ring, compute X = R1 T1^T and Y = R2 T2^T with tcgen05.mma into
// double-buffered tensor memory, turn them into bf16 P and Z = dS (one row per thread, written back over X and Y
// as TMEM operands) and accumulate in tensor memory:
//   dK/dV mode: CTA = (key tile, kv head, batch); R = (K, V), T = (Q, dO) over every query head of the group and
//               every query tile that sees the keys; acc_a = dK += Z Q, acc_b = dV += P dO.
//   dQ mode:    CTA = (query tile, head, batch); R = (Q, dO), T = (K, V) over the visible key tiles; acc_a = dQ += Z K.
// No atomics and no scratch: every output element is produced by one CTA in a fixed order (bit-reproducible run to
// run, as the reference's deterministic mode requires, tests/functional/test_attention.py:403-407).
#include <mutex>
#include <type_traits>

#include "device.h"
#include "sm100.cuh"

namespace lb {
CUtensorMap attention_map_rows(const lb_tensor& t, const char* what, int box_rows);
// attention_bwd_atomic.cu: the single-kernel form (head dim 64) that adds dQ into a zeroed float32 accumulator
bool attention_bwd_atomic_supported(const lb_tensor& q, const lb_tensor& dq);
size_t attention_bwd_atomic_scratch_bytes(const lb_tensor& q);
void attention_bwd_atomic_launch(const lb_attn_desc& desc, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mq,
                                 const CUtensorMap& mdo, const lb_tensor& q, const lb_tensor& k, const float* lse, const float* delta,
                                 float* dq_acc, const lb_tensor& dq, const lb_tensor& dk, const lb_tensor& dv, cudaStream_t s);
namespace {

using namespace sm100;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int BR = 128;  // resident rows (thread = row)
constexpr int BT = 64;   // streamed rows per step
// warp 0: TMA, warp 1: MMA + TMEM owner, then WGS compute warpgroups of four warps, over BUFS X/Y buffers.
//  BUFS = WGS = 2 (head dim 128): warpgroup w takes iterations w, w + WGS, ... on its own X/Y buffer;
//  one CTA per SM. An iteration is a chain MMA -> commit -> wake -> tensor-memory load -> element-wise -> store ->
//  arrive -> wake -> MMA of about 2000 cycles, most of it signalling and load latency (a commit-to-wake takes about
//  350 cycles, an arrive-to-wake 280, a tensor-memory load 170), so throughput is set by how many chains are in
//  flight.
//  BUFS = 1 (head dim 64): single X/Y buffers, 256 tensor-memory columns and half the shared memory, so that TWO CTAs
//  share an SM and one CTA's prologue, epilogue and element-wise latency are covered by the other's MMAs. With
//  WGS = 2 both warpgroups work on EVERY iteration, each on 32 of the 64 streamed columns (the kernels are bound by
//  latency, not by a pipe: 16 compute warps per SM hide twice as much of it as 8).
//  In that mode P and Z are written over Y's columns only, so X is free as soon as every thread has loaded it: the
//  next tile's X product is issued while this tile's element-wise phase runs, and the exponentials (which need X
//  alone) start before the next Y - which has to wait for the accumulation products that read P and Z - has landed.
//  The serial chain per tile shrinks from math + accumulate + X/Y + signalling to roughly accumulate + Y + the Z half
//  of the math. The two-buffer configuration of head dim 128 already overlaps two chains, so it keeps one load round
//  trip for X and Y together.
constexpr int threads_of(int wgs) { return 64 + 128 * wgs; }

struct BwdArgs {
    int B, N, Nkv, Sq, Sk;
    int causal;
    long long causal_offset;
    float scale, scale_log2;
    const float* lse;    // [B, N, Sq]
    const float* delta;  // [B, N, Sq]
    void* out_a;         // dK (dkdv mode) or dQ (dq mode): bf16 [B, S, heads, D] view
    long long a_sb, a_ss, a_sn;
    void* out_b;         // dV (dkdv mode)
    long long b_sb, b_ss, b_sn;
    int* status;
};

template <int D, int BUFS>
struct BwdSmem {
    static constexpr int kResident = BR * D * 2;
    static constexpr int kStream = BT * D * 2;
    // ring of streamed tile pairs: deep enough to hide a tile's TMA latency behind several iterations
    static constexpr int STAGES = BUFS == 1 ? 4 : (D == 64 ? 8 : 4);
    static constexpr int kBytes = 2 * kResident + STAGES * 2 * kStream + 1024 + 256 + 8192;  // tiles, alignment, barriers, column statistics
};

template <int D, bool DKDV, int BUFS, int WGS>
__global__ void __launch_bounds__(threads_of(WGS), BUFS == 1 ? 2 : 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap map_r1, const __grid_constant__ CUtensorMap map_r2,
                     const __grid_constant__ CUtensorMap map_t1, const __grid_constant__ CUtensorMap map_t2, const BwdArgs p) {
    constexpr int kResident = BwdSmem<D, BUFS>::kResident, kStream = BwdSmem<D, BUFS>::kStream, STAGES = BwdSmem<D, BUFS>::STAGES;
    constexpr int kTmemCols = BUFS == 1 ? 256 : 512;
    constexpr bool SPLIT = BUFS == 1 && WGS == 2;  // both warpgroups on every iteration, half of the streamed columns each
    static_assert(BUFS == 1 || BUFS == 2, "one X/Y buffer (two CTAs per SM) or two");
    static_assert(BUFS == 2 || D == 64, "single X/Y buffers with 256 columns only fit the accumulators of head dim 64");
    static_assert(BUFS == 1 || WGS == BUFS, "several X/Y buffers are worked by one warpgroup each");
    static_assert(2 * BUFS * 64 + 2 * D <= kTmemCols && (1 + 2 * STAGES + 4 * BUFS + 2) * 8 + 8 <= 256, "tensor memory / barrier space");
    constexpr int kRBlock = BR * 128, kTBlock = BT * 128;  // bytes of one 64-wide head-dim block of a tile
    constexpr int DB = D / 64;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sr1 = smem;
    uint8_t* sr2 = smem + kResident;
    uint8_t* st1 = smem + 2 * kResident;
    uint8_t* st2 = st1 + STAGES * kStream;
    uint64_t* bars = (uint64_t*)(st2 + STAGES * kStream);
    uint64_t* r_full = bars;             // 1
    uint64_t* t_full = bars + 1;             // STAGES
    uint64_t* t_empty = t_full + STAGES;     // STAGES
    uint64_t* xy_full = t_empty + STAGES;    // BUFS
    uint64_t* pz_ready = xy_full + BUFS;     // BUFS (one arrival per compute thread)
    uint64_t* acc_full = pz_ready + BUFS;    // 1
    uint64_t* y_full = acc_full + 1;         // BUFS, split columns only: Y lands on its own (xy_full then means X)
    uint64_t* x_empty = y_full + BUFS;       // BUFS, split columns only: every compute thread has loaded its X values
    uint64_t* z_free = x_empty + BUFS;       // 1, split columns in dQ mode: the accumulation that read Z has completed
    uint32_t* tmem_slot = (uint32_t*)(z_free + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    // dkdv mode: log-sum-exp (in log2 units) and delta of the streamed query tile, one private copy per compute warp
    // ([warp][lse|delta][BT]) so that staging needs no barrier across warps
    float* col_stats = (float*)((uint8_t*)bars + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = DKDV ? (int)blockIdx.x : (int)(gridDim.x - 1 - blockIdx.x);
    const int head = blockIdx.y, batch = blockIdx.z;  // kv head in dkdv mode, query head in dq mode
    const int group = p.N / p.Nkv;
    const int r0 = tile * BR;

    // streamed range: [t_begin, t_end) in units of BT rows, per head; heads_here heads are walked in dkdv mode
    int t_begin, t_end, heads_here;
    if (DKDV) {
        // queries that see at least the first key of this tile: i >= r0 - offset
        long long first_q = p.causal ? max(0LL, (long long)r0 - p.causal_offset) : 0LL;
        t_begin = (int)(first_q / BT);
        t_end = (p.Sq + BT - 1) / BT;
        heads_here = group;
    } else {
        long long last_key = p.causal ? min((long long)p.Sk - 1, (long long)r0 + BR - 1 + p.causal_offset) : (long long)p.Sk - 1;
        t_begin = 0;
        t_end = last_key < 0 ? 0 : (int)(last_key / BT) + 1;
        heads_here = 1;
    }
    const int per_head = max(t_end - t_begin, 0);
    const int n_iter = per_head * heads_here;
    const int r_head = head;                          // resident tiles: kv head (dkdv) / query head (dq)
    const int kv_head_of_q = DKDV ? head : head / group;

    if (threadIdx.x == 0) {
        mbar_init(r_full, 1);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&t_full[s], 1);
            mbar_init(&t_empty[s], 1);
        }
        for (int s = 0; s < BUFS; s++) {
            mbar_init(&xy_full[s], 1);
            mbar_init(&pz_ready[s], SPLIT ? 256 : 128);
            mbar_init(&y_full[s], 1);
            mbar_init(&x_empty[s], 256);
        }
        mbar_init(acc_full, 1);
        mbar_init(z_free, 1);
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
    const uint32_t tmem_x = tmem_base;                    // BUFS X buffers of 64 columns (P written over their first 32)
    const uint32_t tmem_y = tmem_base + BUFS * 64;        // BUFS Y buffers (Z over their first 32 columns)
    const uint32_t tmem_a = tmem_base + 2 * BUFS * 64;    // acc_a: D columns
    const uint32_t tmem_b = tmem_a + D;                   // acc_b: D columns
    // iteration `it` uses X/Y buffer it % BUFS; its barriers complete once per BUFS iterations
    // bf16 P / Z of 16 streamed rows take 8 columns. A thread writes them over the START of the columns it read, so
    // with split columns the second warpgroup's halves sit at columns 32.. (never over columns the first still reads)
    auto pz_col = [](int k) { return SPLIT ? (k >> 1) * 32 + (k & 1) * 8 : k * 8; };  // k-th group of 16 streamed rows
    // dK/dV mode with split columns: P and Z share the X buffer (P in the first, Z in the second 16 of a thread's 32
    // columns), written with ONE tensor-memory store per iteration - a store's issue cost is paid once
    // With split columns P and Z live in the Y buffer (dK/dV mode: P in the first, Z in the second 16 of a thread's 32
    // columns, written with ONE tensor-memory store; dQ mode: Z alone), so that X is free as soon as every thread has
    // loaded it: the next tile's X product is issued during this tile's element-wise phase, and its exponentials start
    // before the next Y - which has to wait for the accumulation products that read P and Z - has landed.
    // In dQ mode with split columns the second accumulator's columns are unused: Z goes there, so Y is free once it is
    // loaded as well, and BOTH products of the next tile run under this tile's element-wise phase.
    constexpr bool PZ_TOGETHER = SPLIT && DKDV;
    constexpr bool DQ_EARLY = SPLIT && !DKDV;
    const uint32_t tmem_p = SPLIT ? tmem_y : tmem_x;
    const uint32_t tmem_z = PZ_TOGETHER ? tmem_y + 16 : (DQ_EARLY ? tmem_b : tmem_y);
    auto buf_of = [](int it) { return it % BUFS; };
    auto par_of = [](int it) { return (uint32_t)(it / BUFS) & 1u; };

    if (warp == 0) {
        if (lane == 0 && n_iter > 0) {
            tma_prefetch_desc(&map_r1);
            tma_prefetch_desc(&map_r2);
            tma_prefetch_desc(&map_t1);
            tma_prefetch_desc(&map_t2);
            mbar_expect_tx(r_full, 2 * kResident);
            for (int d = 0; d < DB; d++) {
                tma_load_4d(sr1 + d * kRBlock, &map_r1, r_full, d * 64, r_head, r0, batch);
                tma_load_4d(sr2 + d * kRBlock, &map_r2, r_full, d * 64, r_head, r0, batch);
            }
            bool ok = true;
            for (int it = 0; it < n_iter && ok; it++) {
                const int stage = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1;
                const int hh = it / per_head;
                const int t = t_begin + it - hh * per_head;
                const int t_head = DKDV ? head * group + hh : kv_head_of_q;
                if (!(ok = mbar_wait(&t_empty[stage], ph ^ 1, abort_flag))) break;
                mbar_expect_tx(&t_full[stage], 2 * kStream);
                for (int d = 0; d < DB; d++) {
                    tma_load_4d(st1 + stage * kStream + d * kTBlock, &map_t1, &t_full[stage], d * 64, t_head, t * BT, batch);
                    tma_load_4d(st2 + stage * kStream + d * kTBlock, &map_t2, &t_full[stage], d * 64, t_head, t * BT, batch);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_iter > 0) {
            const uint32_t idesc_xy = make_idesc(BR, BT, true, false, false);
            const uint32_t idesc_acc = make_idesc(BR, D, true, false, true);
            bool ok = mbar_wait(r_full, 0, abort_flag);
            // Descriptors are built once and advanced by adds: the one issuing thread is otherwise bound by its own
            // integer instructions, not by the tensor pipe (47 cycles per N = 64 MMA against 94 with rebuilt descriptors).
            const uint64_t dr1 = make_smem_desc(smem_u32(sr1), 16, 1024), dr2 = make_smem_desc(smem_u32(sr2), 16, 1024);
            const uint64_t dt1 = make_smem_desc(smem_u32(st1), 16, 1024), dt2 = make_smem_desc(smem_u32(st2), 16, 1024);
            const uint64_t dt1_mn = make_smem_desc(smem_u32(st1), kTBlock, 1024), dt2_mn = make_smem_desc(smem_u32(st2), kTBlock, 1024);
            auto issue_x = [&](int it) -> bool {
                const int stage = it % STAGES;
                if (!mbar_wait(&t_full[stage], (uint32_t)(it / STAGES) & 1, abort_flag)) return false;
                tc_fence_after();
                const int buf = buf_of(it);
                const uint64_t t1 = desc_advance(dt1, (uint32_t)(stage * kStream));
#pragma unroll
                for (int k = 0; k < D / 16; k++) {
                    const uint32_t roff = (uint32_t)((k / 4) * kRBlock + (k % 4) * 32), toff = (uint32_t)((k / 4) * kTBlock + (k % 4) * 32);
                    mma_f16(tmem_x + buf * 64, desc_advance(dr1, roff), desc_advance(t1, toff), idesc_xy, k != 0);
                }
                if (SPLIT) mma_commit(&xy_full[buf]);
                return true;
            };
            auto issue_y = [&](int it) {  // after issue_x(it): the tile has landed
                const int stage = it % STAGES, buf = buf_of(it);
                const uint64_t t2 = desc_advance(dt2, (uint32_t)(stage * kStream));
#pragma unroll
                for (int k = 0; k < D / 16; k++) {
                    const uint32_t roff = (uint32_t)((k / 4) * kRBlock + (k % 4) * 32), toff = (uint32_t)((k / 4) * kTBlock + (k % 4) * 32);
                    mma_f16(tmem_y + buf * 64, desc_advance(dr2, roff), desc_advance(t2, toff), idesc_xy, k != 0);
                }
                mma_commit(SPLIT ? &y_full[buf] : &xy_full[buf]);
            };
            auto issue_xy = [&](int it) -> bool {
                if (!issue_x(it)) return false;
                issue_y(it);
                return true;
            };
            if (ok) ok = issue_xy(0);
            for (int pre = 1; pre < BUFS && pre < n_iter && ok; pre++) ok = issue_xy(pre);
            for (int it = 0; it < n_iter && ok; it++) {
                const int buf = buf_of(it), stage = it % STAGES;
                if (SPLIT && it + 1 < n_iter) {  // X is free once it is loaded: the next one runs under this tile's element-wise phase
                    if (!(ok = mbar_wait(&x_empty[buf], par_of(it), abort_flag))) break;
                    tc_fence_after();
                    if (!(ok = issue_x(it + 1))) break;
                    if (DQ_EARLY) issue_y(it + 1);  // x_empty then says that X and Y are both in registers
                }
                if (!(ok = mbar_wait(&pz_ready[buf], par_of(it), abort_flag))) break;
                tc_fence_after();
                const uint64_t t1 = desc_advance(dt1_mn, (uint32_t)(stage * kStream)), t2 = desc_advance(dt2_mn, (uint32_t)(stage * kStream));
#pragma unroll
                for (int k = 0; k < BT / 16; k++)  // acc_a += Z . T1   (T1 as an MN-major operand: 16 rows = 2048 bytes per step)
                    mma_f16_ts(tmem_a, tmem_z + buf * 64 + pz_col(k), desc_advance(t1, k * 2048), idesc_acc, (it | k) != 0);
                if (DKDV) {
#pragma unroll
                    for (int k = 0; k < BT / 16; k++)  // acc_b += P . T2
                        mma_f16_ts(tmem_b, tmem_p + buf * 64 + pz_col(k), desc_advance(t2, k * 2048), idesc_acc, (it | k) != 0);
                }
                mma_commit(&t_empty[stage]);
                if (DQ_EARLY) {
                    mma_commit(z_free);
                } else if (SPLIT) {
                    if (it + 1 < n_iter) issue_y(it + 1);  // behind the products that read P and Z in Y's columns: the tensor pipe runs in order
                } else if (it + BUFS < n_iter) {
                    ok = issue_xy(it + BUFS);  // behind the products that read P and Z
                }
            }
            if (ok) mma_commit(acc_full);
        }
    } else {
        // ---- compute warps: thread = resident row. Two warpgroups (warps 2..5 and 6..9) take alternate iterations, each
        // owning one X/Y buffer, so that two rows of exponentials and conversions are in flight per scheduler. ----
        const int wg = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const long long row = (long long)r0 + row_in_tile;  // key index (dkdv) or query index (dq)
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        float row_lse = 0.0f, row_delta = 0.0f;
        if (!DKDV && row < p.Sq) {
            const long long at = ((long long)batch * p.N + head) * p.Sq + row;
            row_lse = p.lse[at] * LOG2E;
            row_delta = p.delta[at] * p.scale;
        }
        bool ok = true;
        constexpr int NC = SPLIT ? 1 : BT / 32;  // 32-column chunks of the streamed tile this thread works on ...
        const int c_first = SPLIT ? wg : 0;      // ... starting at this one
        for (int it = SPLIT ? 0 : wg; it < n_iter && ok; it += SPLIT ? 1 : WGS) {
            const int buf = buf_of(it);
            const int hh = it / per_head;
            const int t = t_begin + it - hh * per_head;
            const long long c0 = (long long)t * BT;  // first streamed index: query (dkdv) or key (dq)
            float* stat_lse = col_stats + (warp - 2) * 2 * BT;
            float* stat_delta = stat_lse + BT;
            if (DKDV) {
                // each warp stages the tile's 64 log-sum-exps and 64 deltas once; its lanes then read them as shared-memory
                // broadcasts instead of two global loads per score
                const long long at = ((long long)batch * p.N + (head * group + hh)) * p.Sq;
                __syncwarp();  // every lane is done with the previous tile's values
#pragma unroll
                for (int u = 0; u < BT / 32; u++) {
                    const long long cc = min(c0 + lane + 32 * u, (long long)p.Sq - 1);
                    stat_lse[lane + 32 * u] = __ldg(p.lse + at + cc) * LOG2E;
                    stat_delta[lane + 32 * u] = __ldg(p.delta + at + cc) * p.scale;
                }
                __syncwarp();
            }
            if (!(ok = mbar_wait(&xy_full[buf], par_of(it), abort_flag))) break;
            __syncwarp();
            tc_fence_after();
            // columns visible to this row: dkdv: query i sees key `row` iff row <= i + off  <=>  i >= row - off, and i < Sq
            //                              dq:   key j visible iff j <= row + off and j < Sk
            long long col_lo, col_hi;  // visible columns are [col_lo, col_hi)
            if (DKDV) {
                col_lo = p.causal ? row - p.causal_offset : 0;
                col_hi = p.Sq;
            } else {
                col_lo = 0;
                col_hi = p.causal ? min((long long)p.Sk, row + p.causal_offset + 1) : (long long)p.Sk;
            }
            // tile-relative visible range [lo, hi) in 32-bit; the unmasked version runs unless some row of the warp is cut
            const int lo = (int)max(0LL, min(col_lo - c0, (long long)BT)), hi = (int)max(0LL, min(col_hi - c0, (long long)BT));
            const bool masked_tile = __any_sync(0xffffffffu, lo > 0 || hi < BT);
            // two-buffer form (head dim 128): X and Y in one load round trip, P over X and Z over Y
            bool early_ok = true;
            auto compute = [&](auto masked) {
                // P and Z = dS of one 32-column chunk from its scores and dP values, written back as bf16 TMEM operands
                auto chunk = [&](int c, const uint32_t* x, const uint32_t* y) {
                    uint32_t pp[16], zz[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float lse4[4], dsc4[4];  // log-sum-exp (log2 units) and delta * scale of the four columns
                        if (DKDV) {
                            const float4 l4 = *(const float4*)(stat_lse + c * 32 + i), d4 = *(const float4*)(stat_delta + c * 32 + i);
                            lse4[0] = l4.x, lse4[1] = l4.y, lse4[2] = l4.z, lse4[3] = l4.w;
                            dsc4[0] = d4.x, dsc4[1] = d4.y, dsc4[2] = d4.z, dsc4[3] = d4.w;
                        } else {
#pragma unroll
                            for (int u = 0; u < 4; u++) lse4[u] = row_lse, dsc4[u] = row_delta;
                        }
                        // two columns per instruction (packed float32 FMA / MUL of sm_100): the element-wise phase is bound by
                        // instruction issue while it runs, and each lane's roundings are those of the scalar form
                        float pv[4], zv[4];
#pragma unroll
                        for (int u = 0; u < 4; u += 2) {
                            const int e = c * 32 + i + u;  // column within the streamed tile
                            const float2 arg = __ffma2_rn(make_float2(__uint_as_float(x[i + u]), __uint_as_float(x[i + u + 1])),
                                                          make_float2(p.scale_log2, p.scale_log2), make_float2(-lse4[u], -lse4[u + 1]));
                            float2 pr = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                            if (decltype(masked)::value) {
                                if (e < lo || e >= hi) pr.x = 0.0f;
                                if (e + 1 < lo || e + 1 >= hi) pr.y = 0.0f;
                            }
                            const float2 t = __ffma2_rn(make_float2(__uint_as_float(y[i + u]), __uint_as_float(y[i + u + 1])),
                                                        make_float2(p.scale, p.scale), make_float2(-dsc4[u], -dsc4[u + 1]));
                            const float2 z = __fmul2_rn(pr, t);  // P * (dP - delta) * scale
                            pv[u] = pr.x, pv[u + 1] = pr.y, zv[u] = z.x, zv[u + 1] = z.y;
                        }
#pragma unroll
                        for (int u = 0; u < 4; u += 2) {
                            __nv_bfloat162 ph2 = __floats2bfloat162_rn(pv[u], pv[u + 1]);
                            __nv_bfloat162 zh2 = __floats2bfloat162_rn(zv[u], zv[u + 1]);
                            pp[(i + u) / 2] = *(uint32_t*)&ph2;
                            zz[(i + u) / 2] = *(uint32_t*)&zh2;
                        }
                    }
                    if (DKDV) tmem_st_32x16(tmem_x + lane_addr + buf * 64 + pz_col(2 * c), pp);
                    tmem_st_32x16(tmem_z + lane_addr + buf * 64 + pz_col(2 * c), zz);
                };
                // all of the thread's scores and dP values in one round trip to tensor memory
                uint32_t x[NC * 32], y[NC * 32];
#pragma unroll
                for (int cc = 0; cc < NC; cc++) {
                    tmem_ld_32x32(tmem_x + lane_addr + buf * 64 + (c_first + cc) * 32, x + cc * 32);
                    tmem_ld_32x32(tmem_y + lane_addr + buf * 64 + (c_first + cc) * 32, y + cc * 32);
                }
                tmem_ld_wait();
                if (DQ_EARLY) {
                    // X and Y are in registers: both products of the next tile may run now. Z(it) goes where Z(it - 1) was:
                    // the accumulation that read it has completed, unless this warp overtook the tensor pipe.
                    tc_fence_before();
                    mbar_arrive(&x_empty[buf]);
                    if (it > 0) {
                        early_ok = __all_sync(0xffffffffu, mbar_wait(z_free, (uint32_t)(it - 1) & 1, abort_flag));  // warp-uniform
                        if (!early_ok) return;
                        tc_fence_after();
                    }
                }
#pragma unroll
                for (int cc = 0; cc < NC; cc++) chunk(c_first + cc, x + cc * 32, y + cc * 32);
            };
            // Split columns: the exponentials run on X alone while the tensor pipe is still busy with the previous tile's
            // accumulation and this tile's Y; X is handed back for the next tile's product as soon as it is in registers.
            auto compute_split = [&](auto masked) -> bool {
                const int c = c_first;  // this warpgroup's 32 of the 64 streamed columns
                uint32_t x[32];
                tmem_ld_32x32(tmem_x + lane_addr + buf * 64 + c * 32, x);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(&x_empty[buf]);
                float pr[32];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float lse4[4];
                    if (DKDV) {
                        const float4 l4 = *(const float4*)(stat_lse + c * 32 + i);
                        lse4[0] = l4.x, lse4[1] = l4.y, lse4[2] = l4.z, lse4[3] = l4.w;
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; u++) lse4[u] = row_lse;
                    }
#pragma unroll
                    for (int u = 0; u < 4; u += 2) {
                        const int e = c * 32 + i + u;  // column within the streamed tile
                        const float2 arg = __ffma2_rn(make_float2(__uint_as_float(x[i + u]), __uint_as_float(x[i + u + 1])),
                                                      make_float2(p.scale_log2, p.scale_log2), make_float2(-lse4[u], -lse4[u + 1]));
                        float2 q = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                        if (decltype(masked)::value) {
                            if (e < lo || e >= hi) q.x = 0.0f;
                            if (e + 1 < lo || e + 1 >= hi) q.y = 0.0f;
                        }
                        pr[i + u] = q.x, pr[i + u + 1] = q.y;
                    }
                }
                if (!mbar_wait(&y_full[buf], par_of(it), abort_flag)) return false;
                __syncwarp();
                tc_fence_after();
                uint32_t y[32], both[32];
                tmem_ld_32x32(tmem_y + lane_addr + buf * 64 + c * 32, y);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float dsc4[4];  // delta * scale of the four columns
                    if (DKDV) {
                        const float4 d4 = *(const float4*)(stat_delta + c * 32 + i);
                        dsc4[0] = d4.x, dsc4[1] = d4.y, dsc4[2] = d4.z, dsc4[3] = d4.w;
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; u++) dsc4[u] = row_delta;
                    }
#pragma unroll
                    for (int u = 0; u < 4; u += 2) {
                        const float2 t = __ffma2_rn(make_float2(__uint_as_float(y[i + u]), __uint_as_float(y[i + u + 1])),
                                                    make_float2(p.scale, p.scale), make_float2(-dsc4[u], -dsc4[u + 1]));
                        const float2 z = __fmul2_rn(make_float2(pr[i + u], pr[i + u + 1]), t);  // P * (dP - delta) * scale
                        __nv_bfloat162 ph2 = __floats2bfloat162_rn(pr[i + u], pr[i + u + 1]);
                        __nv_bfloat162 zh2 = __floats2bfloat162_rn(z.x, z.y);
                        both[(i + u) / 2] = *(uint32_t*)&ph2;
                        both[16 + (i + u) / 2] = *(uint32_t*)&zh2;
                    }
                }
                tmem_st_32x32(tmem_y + lane_addr + buf * 64 + c * 32, both);  // P in the first, Z in the second 16 columns
                return true;
            };
            if (PZ_TOGETHER) {
                if (!(ok = masked_tile ? compute_split(std::true_type{}) : compute_split(std::false_type{}))) break;
            } else {
                if (DQ_EARLY) {  // Y was issued with X: it has landed or is about to
                    if (!(ok = mbar_wait(&y_full[buf], par_of(it), abort_flag))) break;
                    __syncwarp();
                    tc_fence_after();
                }
                if (masked_tile) compute(std::true_type{});
                else compute(std::false_type{});
                if (!(ok = early_ok)) break;
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&pz_ready[buf]);
        }
        // ---- epilogue: accumulators -> bf16 rows ----
        if (n_iter > 0) ok = ok && mbar_wait(acc_full, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const long long limit = DKDV ? p.Sk : p.Sq;
#pragma unroll 1
            // dkdv: with several warpgroups, 0 writes dK and 1 writes dV; a single warpgroup writes both
            for (int which = (DKDV && WGS >= 2) ? wg : 0; which < (DKDV ? (WGS >= 2 ? min(wg + 1, 2) : 2) : 1); which++) {
                uint16_t* base = (uint16_t*)(which == 0 ? p.out_a : p.out_b);
                const long long sb = which == 0 ? p.a_sb : p.b_sb, ss = which == 0 ? p.a_ss : p.b_ss, sn = which == 0 ? p.a_sn : p.b_sn;
                uint16_t* out = base + (long long)batch * sb + row * ss + (long long)head * sn;
                const bool vec = (sb % 8 == 0) && (ss % 8 == 0) && (sn % 8 == 0) && (((uintptr_t)base & 15) == 0);
#pragma unroll 1
                for (int c = (DKDV || WGS == 1) ? 0 : wg; c < D / 32; c += (DKDV || WGS == 1) ? 1 : WGS) {  // dq: the warpgroups take 32-column chunks in turn
                    uint32_t v[32];
                    if (n_iter > 0) {
                        tmem_ld_32x32((which == 0 ? tmem_a : tmem_b) + lane_addr + c * 32, v);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i++) v[i] = 0u;
                    }
                    if (vec && n_iter > 0) {
                        // The warp's 32 rows leave through 2 KB of the first resident tile's shared memory (every product
                        // that read it has completed): whole 64-byte row pieces, eight rows per store instruction.
                        uint4 packed[4];
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * q]), __uint_as_float(v[i + 2 * q + 1]));
                                w[q] = *(uint32_t*)&h;
                            }
                            packed[i / 8] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                        store_rows_coalesced<4>((uint4*)(sr1 + (warp - 2) * 2048), packed, (uint8_t*)(out - (long long)lane * ss + c * 32), ss * 2,
                                                (int)max(0LL, min(32LL, limit - (row - lane))), lane);
                    } else if (row < limit) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * q]), __uint_as_float(v[i + 2 * q + 1]));
                                w[q] = *(uint32_t*)&h;
                            }
                            if (vec) {
                                *(uint4*)(out + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
                            } else {
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    out[c * 32 + i + 2 * q] = (uint16_t)(w[q] & 0xffff);
                                    out[c * 32 + i + 2 * q + 1] = (uint16_t)(w[q] >> 16);
                                }
                            }
                        }
                    }
                }
            }
        }
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

// delta[b, n, s] = sum_d dO[b, s, n, d] * O[b, s, n, d] in fp32. D / 8 lanes per (s, n) row, 16 bytes per lane and
// tensor, several rows per warp; heads of one token are adjacent so a warp reads contiguous memory. One grid row
// (blockIdx.y) per batch entry and 32-bit index arithmetic: the kernel is a pure stream of 2 x 16 bytes per thread,
// and 64-bit divisions per thread used to cost more than the loads.
__global__ void __launch_bounds__(256) attention_delta(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                        float* __restrict__ delta, int S, int N, int D, int n_shift, long long o_sb,
                                                        long long o_ss, long long o_sn, long long g_sb, long long g_ss, long long g_sn) {
    const int lanes = D >> 3;  // 8 (D = 64) or 16 (D = 128)
    const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned row = t / (unsigned)lanes;  // (s, n) of this batch entry; lanes is a power of two
    const int part = (int)(t & (unsigned)(lanes - 1));
    const int b = blockIdx.y;
    const bool live = row < (unsigned)S * (unsigned)N;
    float acc = 0.0f;
    unsigned sq = 0, n = 0;
    if (live) {
        if (n_shift >= 0) sq = row >> n_shift, n = row & ((1u << n_shift) - 1u);
        else sq = row / (unsigned)N, n = row - sq * (unsigned)N;
        const uint4 x = __ldg((const uint4*)(o + b * o_sb + (long long)sq * o_ss + (long long)n * o_sn + part * 8));
        const uint4 y = __ldg((const uint4*)(d_o + b * g_sb + (long long)sq * g_ss + (long long)n * g_sn + part * 8));
        const __nv_bfloat162* xp = (const __nv_bfloat162*)&x;
        const __nv_bfloat162* yp = (const __nv_bfloat162*)&y;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            acc = fmaf(__low2float(xp[k]), __low2float(yp[k]), acc);
            acc = fmaf(__high2float(xp[k]), __high2float(yp[k]), acc);
        }
    }
    for (int m = lanes / 2; m >= 1; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (live && part == 0) delta[((long long)b * N + n) * S + sq] = acc;
}

// Launches attention_delta over [B, S, N, D] views of o and dO.
void launch_delta(const lb_tensor& o, const lb_tensor& d_o, float* delta, cudaStream_t s) {
    const long long B = o.shape[0], S = o.shape[1], N = o.shape[2], D = o.shape[3];
    if (S * N * (D / 8) >= (1LL << 31) || B > 65535) fail(LB_ERR_UNSUPPORTED, "attention backward: sequence x heads or batch too large for the delta kernel's grid");
    int n_shift = -1;
    for (int k = 0; k < 31; k++)
        if ((1LL << k) == N) n_shift = k;
    const unsigned blocks = (unsigned)((S * N * (D / 8) + 255) / 256);
    attention_delta<<<dim3(blocks, (unsigned)B), 256, 0, s>>>((const __nv_bfloat16*)o.ptr, (const __nv_bfloat16*)d_o.ptr, delta, (int)S, (int)N,
                                                              (int)D, n_shift, o.stride[0], o.stride[1], o.stride[2], d_o.stride[0],
                                                              d_o.stride[1], d_o.stride[2]);
    LB_CUDA(cudaGetLastError());
}

template <int D>
void launch_bwd(const CUtensorMap& mq128, const CUtensorMap& mdo128, const CUtensorMap& mk128, const CUtensorMap& mv128,
                const CUtensorMap& mq64, const CUtensorMap& mdo64, const CUtensorMap& mk64, const CUtensorMap& mv64, BwdArgs dkdv,
                BwdArgs dq, cudaStream_t s) {
    constexpr int BUFS = D == 64 ? 1 : 2, WGS = 2;  // head dim 64: two CTAs per SM, both warpgroups on every iteration
    constexpr int kBytes = BwdSmem<D, BUFS>::kBytes, kThreads = threads_of(WGS);
    if (first_use_on_device((const void*)attention_bwd_kernel<D, true, BUFS, WGS>)) {
        LB_CUDA(cudaFuncSetAttribute(attention_bwd_kernel<D, true, BUFS, WGS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
        LB_CUDA(cudaFuncSetAttribute(attention_bwd_kernel<D, false, BUFS, WGS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    }
    dim3 grid_kv((unsigned)((dkdv.Sk + BR - 1) / BR), (unsigned)dkdv.Nkv, (unsigned)dkdv.B);
    attention_bwd_kernel<D, true, BUFS, WGS><<<grid_kv, kThreads, kBytes, s>>>(mk128, mv128, mq64, mdo64, dkdv);
    dim3 grid_q((unsigned)((dq.Sq + BR - 1) / BR), (unsigned)dq.N, (unsigned)dq.B);
    attention_bwd_kernel<D, false, BUFS, WGS><<<grid_q, kThreads, kBytes, s>>>(mq128, mdo128, mk64, mv64, dq);
}

}  // namespace

// `dq_acc` (optional): a dense float32 [B, Sq, N, H] accumulator. With it, and where the single-kernel form applies
// (head dim 64), dQ is summed there atomically over the key blocks - in no fixed order, as the reference's backend does
// unless `deterministic` (lumen/codegen/attention/triton/mod.rs:458-466) - and rounded to dq afterwards.
void attention_bwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                   const lb_tensor& d_o, const lb_tensor& lse, const lb_tensor& delta, const lb_tensor& dq, const lb_tensor& dk,
                   const lb_tensor& dv, void* stream, const lb_tensor* dq_acc = nullptr) {
    const long long B = q.shape[0], Sq = q.shape[1], N = q.shape[2], D = q.shape[3];
    if (q.rank != 4 || k.rank != 4 || v.rank != 4) fail(LB_ERR_INVALID, "attention backward: operands must be [B, S, N, H] tensors");
    const long long Sk = k.shape[1], Nkv = k.shape[2];
    if (k.shape[0] != B || v.shape[0] != B || k.shape[3] != D || v.shape[1] != Sk || v.shape[2] != Nkv || v.shape[3] != D || Nkv == 0 || N % Nkv)
        fail(LB_ERR_INVALID, "attention backward: shapes are not [B,Sq,N,H], [B,Sk,Nkv,H], [B,Sk,Nkv,H] with N a multiple of Nkv");
    if (D != 64 && D != 128) fail(LB_ERR_UNSUPPORTED, "attention backward: head dims 64 and 128 have a tcgen05 kernel (the reference supports up to 128)");
    if (!(desc.scale > 0.0f)) fail(LB_ERR_UNSUPPORTED, "attention: the softmax scale must be positive");
    auto same = [&](const lb_tensor& t, const lb_tensor& like, const char* what) {
        if (t.rank != 4 || t.dtype != LB_BF16 || t.stride[3] != 1)
            fail(LB_ERR_INVALID, format("attention backward: %s must be a bfloat16 [B, S, N, H] view with a unit head-dim stride", what));
        for (int d = 0; d < 4; d++)
            if (t.shape[d] != like.shape[d]) fail(LB_ERR_INVALID, format("attention backward: %s has the wrong shape", what));
    };
    same(o, q, "o"), same(d_o, q, "dO"), same(dq, q, "dQ"), same(dk, k, "dK"), same(dv, v, "dV");
    if (B == 0 || N == 0) return;  // nothing to compute: no launch
    check_dense(lse, LB_F32, {B, N, Sq}, "attention log-sum-exp");
    check_dense(delta, LB_F32, {B, N, Sq}, "attention delta");
    driver();
    cudaStream_t s = (cudaStream_t)stream;
    if (Sq > 0) {
        if (o.stride[0] % 8 || o.stride[1] % 8 || o.stride[2] % 8 || d_o.stride[0] % 8 || d_o.stride[1] % 8 || d_o.stride[2] % 8 ||
            ((uintptr_t)o.ptr & 15) || ((uintptr_t)d_o.ptr & 15))
            fail(LB_ERR_UNSUPPORTED, "attention backward: o and dO rows must be 16-byte aligned");
        launch_delta(o, d_o, (float*)delta.ptr, s);
    }
    BwdArgs a{};
    a.B = (int)B, a.N = (int)N, a.Nkv = (int)Nkv, a.Sq = (int)Sq, a.Sk = (int)Sk;
    a.causal = desc.causal, a.causal_offset = desc.causal_offset;
    a.scale = desc.scale, a.scale_log2 = desc.scale * 1.4426950408889634f;
    a.lse = (const float*)lse.ptr, a.delta = (const float*)delta.ptr;
    a.status = status_word();
    BwdArgs kv = a, qq = a;
    kv.out_a = dk.ptr, kv.a_sb = dk.stride[0], kv.a_ss = dk.stride[1], kv.a_sn = dk.stride[2];
    kv.out_b = dv.ptr, kv.b_sb = dv.stride[0], kv.b_ss = dv.stride[1], kv.b_sn = dv.stride[2];
    qq.out_a = dq.ptr, qq.a_sb = dq.stride[0], qq.a_ss = dq.stride[1], qq.a_sn = dq.stride[2];
    if (Sk == 0 || Sq == 0) fail(LB_ERR_UNSUPPORTED, "attention backward: empty sequences");
    CUtensorMap mq128 = attention_map_rows(q, "query", 128), mdo128 = attention_map_rows(d_o, "dO", 128);
    CUtensorMap mk128 = attention_map_rows(k, "key", 128), mv128 = attention_map_rows(v, "value", 128);
    if (dq_acc && attention_bwd_atomic_supported(q, dq)) {
        check_dense(*dq_acc, LB_F32, {B, Sq, N, D}, "attention dQ accumulator");
        attention_bwd_atomic_launch(desc, mk128, mv128, mq128, mdo128, q, k, a.lse, a.delta, (float*)dq_acc->ptr, dq, dk, dv, s);
        return;
    }
    CUtensorMap mq64 = attention_map_rows(q, "query", 64), mdo64 = attention_map_rows(d_o, "dO", 64);
    CUtensorMap mk64 = attention_map_rows(k, "key", 64), mv64 = attention_map_rows(v, "value", 64);
    if (D == 128) launch_bwd<128>(mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64, kv, qq, s);
    else launch_bwd<64>(mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64, kv, qq, s);
    LB_CUDA(cudaGetLastError());
}

}  // namespace lb

namespace lb {
bool attention_on_tensor_cores(const lb_tensor& q, const lb_tensor& k, const lb_tensor& v);
void attention_simt_bwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                        const lb_tensor& g, const lb_tensor& lse, const lb_tensor& delta, const lb_tensor& dq, const lb_tensor& dk,
                        const lb_tensor& dv, void* stream);
void attention_backward(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                        const lb_tensor& d_o, const lb_tensor& lse, const lb_tensor& delta, const lb_tensor& dq, const lb_tensor& dk,
                        const lb_tensor& dv, void* stream, const lb_tensor* dq_acc) {
    if (attention_on_tensor_cores(q, k, v) && attention_on_tensor_cores(d_o, k, v) && attention_on_tensor_cores(o, k, v) && q.shape[1] > 0 &&
        k.shape[1] > 0)
        attention_bwd(desc, q, k, v, o, d_o, lse, delta, dq, dk, dv, stream, dq_acc);
    else
        attention_simt_bwd(desc, q, k, v, o, d_o, lse, delta, dq, dk, dv, stream);
}
}  // namespace lb

extern "C" int lb_attention_bwd(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                                const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* delta,
                                const lb_tensor* dq, const lb_tensor* dk, const lb_tensor* dv, void* stream) {
    return lb::guarded([&] {
        if (!desc || !q || !k || !v || !o || !d_o || !lse || !delta || !dq || !dk || !dv)
            lb::fail(LB_ERR_INVALID, "lb_attention_bwd: null argument");
        lb::attention_backward(*desc, *q, *k, *v, *o, *d_o, *lse, *delta, *dq, *dk, *dv, stream, nullptr);
    });
}

// lb_attention_bwd in the reference backend's default (non-deterministic) mode: with bfloat16 operands of head dim 64
// the backward runs as ONE kernel that adds each key block's dS K into `dq_accum` (dense float32 [B, Sq, N, H], zeroed
// by the call) in no fixed order and rounds it to dq at the end; other operands run exactly as lb_attention_bwd does.
extern "C" int lb_attention_bwd_atomic(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                                       const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* delta,
                                       const lb_tensor* dq_accum, const lb_tensor* dq, const lb_tensor* dk, const lb_tensor* dv, void* stream) {
    return lb::guarded([&] {
        if (!desc || !q || !k || !v || !o || !d_o || !lse || !delta || !dq_accum || !dq || !dk || !dv)
            lb::fail(LB_ERR_INVALID, "lb_attention_bwd_atomic: null argument");
        lb::attention_backward(*desc, *q, *k, *v, *o, *d_o, *lse, *delta, *dq, *dk, *dv, stream, dq_accum);
    });
}

// ---- allocation-free variant ---------------------------------------------------------------------------------
// For callers that must not allocate device memory when they call in: code running inside a memory pool that
// forbids cudaMalloc after start-up, inside a region where the allocator is locked, or under a real-time budget
// where an allocation's latency and possible failure are unacceptable. The backward's one piece of scratch, the
// per-row delta = rowsum(dO * O), lives in a fixed array in the library's device image instead of caller memory.
namespace lb {
namespace {

constexpr long long kStaticDeltaFloats = 1LL << 20;  // 4 MiB per GPU that loads the library, held until exit
static __device__ __align__(256) float g_static_delta[kStaticDeltaFloats];
static __device__ __align__(256) int g_static_status[64];

struct StaticSetup {
    bool ready = false;
    float* delta = nullptr;  // DEVICE address of g_static_delta (the symbol's name is only a host-side stand-in)
    int* status = nullptr;
    decltype(Driver::cuTensorMapEncodeTiled) encode = nullptr;
};
StaticSetup g_static[64];
std::mutex g_static_mutex;

// Once per device, with that device current: resolve the device addresses of the static arrays and the tensor-map
// encoder. Nothing here allocates.
const StaticSetup& static_setup() {
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) fail(LB_ERR_UNSUPPORTED, "lb_attention_bwd_static: device index beyond 63");
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSetup& s = g_static[dev];
    if (s.ready) return s;
    cudaError_t err = cudaGetSymbolAddress((void**)&s.delta, g_static_delta);
    if (err != cudaSuccess) fail(LB_ERR_CUDA, format("cudaGetSymbolAddress(delta scratch): %s", cudaGetErrorString(err)));
    err = cudaGetSymbolAddress((void**)&s.status, g_static_status);
    if (err != cudaSuccess) fail(LB_ERR_CUDA, format("cudaGetSymbolAddress(status word): %s", cudaGetErrorString(err)));
    cudaDriverEntryPointQueryResult found;
    void* fn = nullptr;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found);
    if (err != cudaSuccess || found != cudaDriverEntryPointSuccess || !fn)
        fail(LB_ERR_CUDA, "lb_attention_bwd_static: cuTensorMapEncodeTiled is unavailable");
    s.encode = (decltype(s.encode))fn;
    LB_CUDA(cudaMemset(s.status, 0, sizeof(int)));  // the status word must start at zero
    register_status_word(s.status);                 // lb_device_status() reads (and clears) it with the library's other words
    s.ready = true;
    return s;
}

CUtensorMap static_map(const StaticSetup& s, const lb_tensor& t, const char* what, int box_rows) {
    if (t.rank != 4 || t.dtype != LB_BF16 || t.stride[3] != 1 || ((uintptr_t)t.ptr & 15) || t.stride[0] % 8 || t.stride[1] % 8 || t.stride[2] % 8)
        fail(LB_ERR_UNSUPPORTED, format("lb_attention_bwd_static: %s must be a bfloat16 [B, S, N, H] view with a unit head-dim stride and 16-byte aligned rows", what));
    cuuint64_t dims[4] = {(cuuint64_t)t.shape[3], (cuuint64_t)t.shape[2], (cuuint64_t)t.shape[1], (cuuint64_t)t.shape[0]};
    cuuint64_t strides[3] = {(cuuint64_t)t.stride[2] * 2, (cuuint64_t)t.stride[1] * 2, (cuuint64_t)t.stride[0] * 2};
    if (t.shape[2] == 1) strides[0] = (cuuint64_t)t.shape[3] * 2;
    if (t.shape[1] == 1) strides[1] = strides[0] * t.shape[2];
    if (t.shape[0] == 1) strides[2] = strides[1] * t.shape[1];
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap map;
    CUresult rc = s.encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) fail(LB_ERR_CUDA, format("cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)rc));
    return map;
}

void attention_bwd_static(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                          const lb_tensor& d_o, const lb_tensor& lse, const lb_tensor& dq, const lb_tensor& dk, const lb_tensor& dv,
                          void* stream) {
    if (q.rank != 4 || k.rank != 4 || v.rank != 4) fail(LB_ERR_INVALID, "lb_attention_bwd_static: operands must be [B, S, N, H] tensors");
    const long long B = q.shape[0], Sq = q.shape[1], N = q.shape[2], D = q.shape[3], Sk = k.shape[1], Nkv = k.shape[2];
    if (k.shape[0] != B || v.shape[0] != B || k.shape[3] != D || v.shape[1] != Sk || v.shape[2] != Nkv || v.shape[3] != D || Nkv == 0 || N % Nkv)
        fail(LB_ERR_INVALID, "lb_attention_bwd_static: shapes are not [B,Sq,N,H], [B,Sk,Nkv,H], [B,Sk,Nkv,H] with N a multiple of Nkv");
    if (D != 64 && D != 128) fail(LB_ERR_UNSUPPORTED, "lb_attention_bwd_static: head dims 64 and 128 only");
    if (!(desc.scale > 0.0f)) fail(LB_ERR_UNSUPPORTED, "lb_attention_bwd_static: the softmax scale must be positive");
    if (B <= 0 || N <= 0 || Sq <= 0 || Sk <= 0) fail(LB_ERR_UNSUPPORTED, "lb_attention_bwd_static: empty operands");
    if (B * N * Sq > kStaticDeltaFloats)
        fail(LB_ERR_INVALID, format("lb_attention_bwd_static: batch * heads * query length = %lld exceeds the built-in scratch of %lld rows; "
                                    "use lb_attention_bwd with caller-provided scratch", B * N * Sq, kStaticDeltaFloats));
    auto same = [&](const lb_tensor& t, const lb_tensor& like, const char* what) {
        if (t.rank != 4 || t.dtype != LB_BF16 || t.stride[3] != 1) fail(LB_ERR_INVALID, format("lb_attention_bwd_static: %s must be a bfloat16 [B, S, N, H] view", what));
        for (int d = 0; d < 4; d++)
            if (t.shape[d] != like.shape[d]) fail(LB_ERR_INVALID, format("lb_attention_bwd_static: %s has the wrong shape", what));
    };
    same(o, q, "o"), same(d_o, q, "dO"), same(dq, q, "dQ"), same(dk, k, "dK"), same(dv, v, "dV");
    check_dense(lse, LB_F32, {B, N, Sq}, "attention log-sum-exp");
    if (o.stride[0] % 8 || o.stride[1] % 8 || o.stride[2] % 8 || d_o.stride[0] % 8 || d_o.stride[1] % 8 || d_o.stride[2] % 8 ||
            ((uintptr_t)o.ptr & 15) || ((uintptr_t)d_o.ptr & 15))
        fail(LB_ERR_UNSUPPORTED, "lb_attention_bwd_static: o and dO rows must be 16-byte aligned");
    const StaticSetup& st = static_setup();
    cudaStream_t s = (cudaStream_t)stream;
    launch_delta(o, d_o, st.delta, s);
    BwdArgs a{};
    a.B = (int)B, a.N = (int)N, a.Nkv = (int)Nkv, a.Sq = (int)Sq, a.Sk = (int)Sk;
    a.causal = desc.causal, a.causal_offset = desc.causal_offset;
    a.scale = desc.scale, a.scale_log2 = desc.scale * 1.4426950408889634f;
    a.lse = (const float*)lse.ptr, a.delta = st.delta, a.status = st.status;
    BwdArgs kv = a, qq = a;
    kv.out_a = dk.ptr, kv.a_sb = dk.stride[0], kv.a_ss = dk.stride[1], kv.a_sn = dk.stride[2];
    kv.out_b = dv.ptr, kv.b_sb = dv.stride[0], kv.b_ss = dv.stride[1], kv.b_sn = dv.stride[2];
    qq.out_a = dq.ptr, qq.a_sb = dq.stride[0], qq.a_ss = dq.stride[1], qq.a_sn = dq.stride[2];
    CUtensorMap mq128 = static_map(st, q, "query", 128), mdo128 = static_map(st, d_o, "dO", 128);
    CUtensorMap mk128 = static_map(st, k, "key", 128), mv128 = static_map(st, v, "value", 128);
    CUtensorMap mq64 = static_map(st, q, "query", 64), mdo64 = static_map(st, d_o, "dO", 64);
    CUtensorMap mk64 = static_map(st, k, "key", 64), mv64 = static_map(st, v, "value", 64);
    if (D == 128) launch_bwd<128>(mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64, kv, qq, s);
    else launch_bwd<64>(mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64, kv, qq, s);
    LB_CUDA(cudaGetLastError());
}

}  // namespace

// The status word of lb_attention_bwd_static on the current device (sets the entry up on first use; allocates nothing).
int* static_status_word() { return static_setup().status; }
}  // namespace lb

// lb_attention_bwd without any device allocation. The scratch the backward needs (one float per query row and
// head) is a 4 MiB array built into the library; it is shared by every call, so two calls whose kernels can overlap
// on the GPU (different streams, or different host threads) race on it: serialise them. The array keeps whatever
// the previous call left there; each call overwrites the part it reads before reading it, so nothing needs
// clearing. The first call on a device resolves the array's device address (cudaGetSymbolAddress) and the
// tensor-map encoder; make that first call before starting any stream capture. Limit: batch * heads * query
// length <= 1,048,576, bfloat16 operands, head dim 64 or 128; beyond that the call fails with a message and
// lb_attention_bwd (caller-provided scratch) is the entry to use.
extern "C" int lb_attention_bwd_static(const lb_attn_desc* desc, const lb_tensor* q, const lb_tensor* k, const lb_tensor* v,
                                       const lb_tensor* o, const lb_tensor* d_o, const lb_tensor* lse, const lb_tensor* dq,
                                       const lb_tensor* dk, const lb_tensor* dv, void* stream) {
    return lb::guarded([&] {
        if (!desc || !q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv) lb::fail(LB_ERR_INVALID, "lb_attention_bwd_static: null argument");
        lb::attention_bwd_static(*desc, *q, *k, *v, *o, *d_o, *lse, *dq, *dk, *dv, stream);
    });
}

