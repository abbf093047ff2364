// Flash-attention backward for sm_100a, head dim 64, as ONE kernel: the mode the reference's backend runs unless
// `deterministic` is set - dK and dV per key block, each key block's dS K added atomically into a zeroed float32 dQ
// (lumen/codegen/attention/triton/mod.rs:176-180,458-466, kernel.py:108-200 with ADD_DQ; the traced math is
// lumen/functional/attention/flash.py:51-85). The two-kernel form of attention_bwd.cu recomputes the scores and dP in
// its dQ kernel: seven products and two sets of exponentials per (key tile, query tile); this form needs five and one.
//
// CTA = (128-key tile, kv head, batch), one CTA per SM, all 512 tensor-memory columns:
//   X  = K Q^T   [keys x queries] fp32, 128 columns      Y  = V dO^T, 128 columns
//   P  = exp2(X c - lse) as bf16, 64 columns (the TMEM operand of dV += P dO)
//   dK, dV accumulators, 64 columns each                 dQ' = dS K of this tile pair, 64 columns
// K and V stay resident in shared memory; Q and dO tiles of 128 queries stream through a 3-stage TMA ring, over every
// query head of the kv head's group and every query tile that sees the keys. Z = dS^T = P (Y - delta) scale is
// rounded to bf16 and written by the compute threads (thread = key row) into shared memory in the 128-byte-swizzled
// tile layout; the same buffer is the K-major operand of dK += Z Q and the MN-major operand of dQ' = Z^T K. X and Y
// are free as soon as the compute threads hold them in registers, so the next tile's products run under this tile's
// element-wise phase. dQ' leaves through a warpgroup of its own: two [128 queries x 32 columns] halves staged in shared
// memory as swizzled tiles and added to the float32 accumulator by TMA tensor reduces (cp.reduce.async.bulk.tensor ...
// add), which clip the rows beyond the sequence; a separate pass rounds the accumulator to bf16.
// Roles get their own register budgets (setmaxnreg): the two compute warpgroups 160 per thread, the others 96.
// Every barrier wait is bounded; a wait that runs out raises the device status word and winds the CTA down.
// What bounds it: the tensor pipe's operand traffic, not its arithmetic. At head dim 64 a (128 x 128) tile pair is
// 10.5 MFLOP (1280 cycles of tensor-core time) but its five products read 176 KB of operands from shared memory; the
// issuing thread measured about 90 cycles per 128 x 64 x 16 product with every wait removed, 3600 per tile pair.
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

constexpr int D = 64;        // head dim
constexpr int BR = 128;      // resident key rows (thread = key row)
constexpr int BT = 128;      // streamed query rows per iteration
constexpr int STAGES = 3;    // ring of (Q, dO) tile pairs
// warp 0: TMA, warp 1: MMA + TMEM owner (warps 2, 3 idle: register budgets are set per aligned group of four warps),
// warps 4..7: the warpgroup that moves dQ' out, warps 8..15: two compute warpgroups
constexpr int kThreads = 512;
// Register budgets per role (setmaxnreg). An increase only draws on registers the CTA already owns - those it was
// launched with (kLaunchRegs per thread) minus what other warpgroups have released - and BLOCKS until they are there:
// the budgets must add up to no more than the launch allocation, or the compute warps would wait forever.
constexpr int kLaunchRegs = 128;  // what the compiler assigns under __launch_bounds__(512, 1); checked before the first launch
constexpr int kRegsLight = 96, kRegsDrain = 96, kRegsCompute = 160;
static_assert(128 * kRegsLight + 128 * kRegsDrain + 256 * kRegsCompute <= kLaunchRegs * kThreads, "register budgets exceed the launch allocation");
constexpr int kTile = BR * D * 2;   // one 128 x 64 bf16 tile (K, V, Q or dO)
constexpr int kZBlock = BR * 128;   // one 64-query block of Z: 128 key rows of 128 bytes
constexpr int kHalf = BT * 128;     // staging of one warpgroup's half of dQ': 128 query rows of 32 floats
constexpr int kOffZ = (2 + 2 * STAGES) * kTile;
constexpr int kOffStage = kOffZ + 2 * kZBlock;
constexpr int kOffStats = kOffStage + 2 * kHalf;
constexpr int kOffBars = kOffStats + 8 * 2 * 64 * 4;
constexpr int kSmemBytes = kOffBars + 256 + 1024;

struct AtomicArgs {
    int B, N, Nkv, Sq, Sk;
    int causal;
    long long causal_offset;
    float scale, scale_log2;
    const float* lse;    // [B, N, Sq]
    const float* delta;  // [B, N, Sq]
    float* dq_acc;       // dense float32 [B, Sq, N, D], zeroed
    void* dk;            // bf16 [B, Sk, Nkv, D] views
    long long k_sb, k_ss, k_sn;
    void* dv;
    long long v_sb, v_ss, v_sn;
    int* status;
};

// Adds the float32 tile at `src_smem` (the map's box, swizzled as the map says) to global memory at the coordinates.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, const void* src_smem, int c0, int c1, int c2, int c3) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
                 "r"(smem_u32(src_smem)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
// Register budget of the calling warpgroup (all four of its warps execute this): the kernel starts with 128 per thread.
template <int N>
__device__ __forceinline__ void regs_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void regs_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
// Barrier `id` over `count` threads (a warpgroup): the CTA-wide barrier 0 stays free for the other roles.
__device__ __forceinline__ void named_barrier(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
attention_bwd_atomic_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                            const __grid_constant__ CUtensorMap map_acc, const AtomicArgs p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sk = smem;
    uint8_t* sv = smem + kTile;
    uint8_t* sq = smem + 2 * kTile;             // STAGES tiles
    uint8_t* sdo = sq + STAGES * kTile;         // STAGES tiles
    uint8_t* sz = smem + kOffZ;                 // Z: two 64-query blocks of [128 keys x 128 bytes], swizzled
    uint8_t* stage = smem + kOffStage;          // dQ' rows on their way out
    float* col_stats = (float*)(smem + kOffStats);
    uint64_t* bars = (uint64_t*)(smem + kOffBars);
    uint64_t* r_full = bars;               // K and V have landed
    uint64_t* t_full = bars + 1;           // STAGES: a (Q, dO) pair has landed
    uint64_t* t_empty = t_full + STAGES;   // STAGES: the products that read it have completed
    uint64_t* xy_full = t_empty + STAGES;  // X(it) and Y(it) are in tensor memory
    uint64_t* xy_empty = xy_full + 1;      // every compute thread holds its part of X(it) and Y(it) (256 arrivals)
    uint64_t* pz_ready = xy_empty + 1;     // P(it) is in tensor memory and Z(it) in shared memory (256 arrivals)
    uint64_t* pz_free = pz_ready + 1;      // the products that read P(it) and Z(it) have completed
    uint64_t* dq_full = pz_free + 1;       // dQ'(it) is in tensor memory
    uint64_t* dq_empty = dq_full + 1;      // every compute thread has loaded its part of dQ'(it) (128 arrivals)
    uint64_t* acc_full = dq_empty + 1;     // dK and dV are complete
    uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = (int)blockIdx.x, head = (int)blockIdx.y, batch = (int)blockIdx.z;  // key tile, kv head
    const int group = p.N / p.Nkv;
    const int r0 = tile * BR;
    // query tiles that see at least the first key of this tile: i >= r0 - offset
    const long long first_q = p.causal ? max(0LL, (long long)r0 - p.causal_offset) : 0LL;
    const int t_begin = (int)(first_q / BT), t_end = (p.Sq + BT - 1) / BT;
    const int per_head = max(t_end - t_begin, 0);
    const int n_iter = per_head * group;

    if (threadIdx.x == 0) {
        mbar_init(r_full, 1);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&t_full[s], 1);
            mbar_init(&t_empty[s], 1);
        }
        mbar_init(xy_full, 1);
        mbar_init(xy_empty, 256);
        mbar_init(pz_ready, 256);
        mbar_init(pz_free, 1);
        mbar_init(dq_full, 1);
        mbar_init(dq_empty, 128);
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_x = tmem_base, tmem_y = tmem_base + 128, tmem_dk = tmem_base + 256, tmem_dv = tmem_base + 320;
    const uint32_t tmem_dq = tmem_base + 384, tmem_p = tmem_base + 448;

    // each register budget is set inside the branch it governs: code after a join is compiled for the smallest one
    if (warp < 4) {
      regs_dec<kRegsLight>();
      if (warp == 0) {
        if (lane == 0 && n_iter > 0) {
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_do);
            tma_prefetch_desc(&map_acc);
            mbar_expect_tx(r_full, 2 * kTile);
            tma_load_4d(sk, &map_k, r_full, 0, head, r0, batch);
            tma_load_4d(sv, &map_v, r_full, 0, head, r0, batch);
            bool ok = true;
            for (int it = 0; it < n_iter && ok; it++) {
                const int st = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1;
                const int hh = it / per_head;
                const int t = t_begin + it - hh * per_head;
                if (!(ok = mbar_wait(&t_empty[st], ph ^ 1, abort_flag))) break;
                mbar_expect_tx(&t_full[st], 2 * kTile);
                tma_load_4d(sq + st * kTile, &map_q, &t_full[st], 0, head * group + hh, t * BT, batch);
                tma_load_4d(sdo + st * kTile, &map_do, &t_full[st], 0, head * group + hh, t * BT, batch);
            }
        }
      } else if (warp == 1) {
        if (lane == 0 && n_iter > 0) {
            const uint32_t idesc_xy = make_idesc(BR, BT, true, false, false);  // K-major A and B
            const uint32_t idesc_acc = make_idesc(BR, D, true, false, true);   // A from tensor memory or K-major, B MN-major
            const uint32_t idesc_dq = make_idesc(BT, D, true, true, true);     // A and B MN-major
            bool ok = mbar_wait(r_full, 0, abort_flag);
            const uint64_t dk_k = make_smem_desc(smem_u32(sk), 16, 1024), dv_k = make_smem_desc(smem_u32(sv), 16, 1024);
            const uint64_t dk_mn = make_smem_desc(smem_u32(sk), kTile, 1024);
            const uint64_t dq_k = make_smem_desc(smem_u32(sq), 16, 1024), ddo_k = make_smem_desc(smem_u32(sdo), 16, 1024);
            const uint64_t dq_mn = make_smem_desc(smem_u32(sq), kTile, 1024), ddo_mn = make_smem_desc(smem_u32(sdo), kTile, 1024);
            const uint64_t dz_k = make_smem_desc(smem_u32(sz), 16, 1024), dz_mn = make_smem_desc(smem_u32(sz), kZBlock, 1024);
            auto issue_xy = [&](int it) -> bool {
                const int st = it % STAGES;
                if (!mbar_wait(&t_full[st], (uint32_t)(it / STAGES) & 1, abort_flag)) return false;
                tc_fence_after();
                const uint64_t tq = desc_advance(dq_k, (uint32_t)(st * kTile)), tdo = desc_advance(ddo_k, (uint32_t)(st * kTile));
#pragma unroll
                for (int k = 0; k < D / 16; k++) mma_f16(tmem_x, desc_advance(dk_k, k * 32), desc_advance(tq, k * 32), idesc_xy, k != 0);
#pragma unroll
                for (int k = 0; k < D / 16; k++) mma_f16(tmem_y, desc_advance(dv_k, k * 32), desc_advance(tdo, k * 32), idesc_xy, k != 0);
                mma_commit(xy_full);
                return true;
            };
            if (ok) ok = issue_xy(0);
            for (int it = 0; it < n_iter && ok; it++) {
                const int st = it % STAGES;
                const uint32_t par = (uint32_t)it & 1;
                if (it + 1 < n_iter) {  // X and Y are in registers: the next tile's products run under this tile's element-wise phase
                    if (!(ok = mbar_wait(xy_empty, par, abort_flag))) break;
                    tc_fence_after();
                    if (!(ok = issue_xy(it + 1))) break;
                }
                if (!(ok = mbar_wait(pz_ready, par, abort_flag))) break;
                tc_fence_after();
                const uint64_t tq = desc_advance(dq_mn, (uint32_t)(st * kTile)), tdo = desc_advance(ddo_mn, (uint32_t)(st * kTile));
#pragma unroll
                for (int k = 0; k < BT / 16; k++)  // dV += P dO: 16 queries = 8 packed columns of P, 16 rows (2048 bytes) of dO
                    mma_f16_ts(tmem_dv, tmem_p + k * 8, desc_advance(tdo, k * 2048), idesc_acc, (it | k) != 0);
#pragma unroll
                for (int k = 0; k < BT / 16; k++)  // dK += Z Q: Z K-major, 16 queries = 32 bytes of a row, 64-query blocks kZBlock apart
                    mma_f16(tmem_dk, desc_advance(dz_k, (uint32_t)((k / 4) * kZBlock + (k % 4) * 32)), desc_advance(tq, k * 2048), idesc_acc, (it | k) != 0);
                if (it > 0) {
                    if (!(ok = mbar_wait(dq_empty, par ^ 1, abort_flag))) break;
                    tc_fence_after();
                }
#pragma unroll
                for (int k = 0; k < BR / 16; k++)  // dQ' = Z^T K: Z MN-major (16 key rows = 2048 bytes per step), K MN-major
                    mma_f16(tmem_dq, desc_advance(dz_mn, k * 2048), desc_advance(dk_mn, k * 2048), idesc_dq, k != 0);
                mma_commit(&t_empty[st]);
                mma_commit(pz_free);
                mma_commit(dq_full);
            }
            if (ok) mma_commit(acc_full);
        }
      }
    } else if (warp < 8) {
        regs_dec<kRegsDrain>();
        // ---- dQ' out of tensor memory (lane = query row of the tile) and into the accumulator ----
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int swz = row_in_tile & 7;
        const bool issuer = warp == 4 && lane == 0;
        bool ok = true;
        for (int j = 0; j < n_iter && ok; j++) {
            const int hh = j / per_head;
            const int q0 = (t_begin + j - hh * per_head) * BT;
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(dq_full, (uint32_t)j & 1, abort_flag)))) break;
            tc_fence_after();
            if (issuer) bulk_wait_read();  // the previous reduces have read the staging tiles
            named_barrier(1, 128);
#pragma unroll
            for (int h = 0; h < 2; h++) {  // two halves of 32 columns: [128 rows x 128 bytes], swizzled as the tensor map expects
                uint32_t v[32];
                tmem_ld_32x32(tmem_dq + lane_addr + h * 32, v);
                tmem_ld_wait();
                if (h == 1) {
                    tc_fence_before();
                    mbar_arrive(dq_empty);
                }
#pragma unroll
                for (int i = 0; i < 8; i++)
                    *(uint4*)(stage + h * kHalf + row_in_tile * 128 + ((i ^ swz) * 16)) = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
            fence_proxy_async();
            named_barrier(1, 128);
            if (issuer) {
                tma_reduce_add_4d(&map_acc, stage, 0, head * group + hh, q0, batch);
                tma_reduce_add_4d(&map_acc, stage + kHalf, 32, head * group + hh, q0, batch);
                bulk_commit();
            }
        }
        bulk_wait_all();
    } else {
        regs_inc<kRegsCompute>();
        // ---- compute warps: thread = key row; warpgroup w works on 64 of the tile's 128 query columns ----
        const int wg = (warp - 8) >> 2, quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const long long row = (long long)r0 + row_in_tile;  // key index
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float LOG2E = 1.4426950408889634f;
        float* stat_lse = col_stats + (warp - 8) * 128;
        float* stat_delta = stat_lse + 64;
        uint8_t* z_row = sz + wg * kZBlock + row_in_tile * 128;  // this thread's 128 bytes of Z: its key row in the 64-query block wg
        const int z_swz = row_in_tile & 7;
        bool ok = true;

        // log-sum-exp and delta of an iteration's 64 columns, two of each per lane: loaded one iteration ahead, so that
        // their latency is not part of an iteration's chain
        float nl[2] = {0.0f, 0.0f}, nd[2] = {0.0f, 0.0f};
        auto load_stats = [&](int j) {
            const int hj = j / per_head;
            const long long cj = (long long)(t_begin + j - hj * per_head) * BT + wg * 64;
            const long long at = ((long long)batch * p.N + (head * group + hj)) * p.Sq;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const long long cc = min(cj + lane + 32 * u, (long long)p.Sq - 1);
                nl[u] = __ldg(p.lse + at + cc);  // scaled when they are staged: a use here would wait for the load
                nd[u] = __ldg(p.delta + at + cc);
            }
        };
        if (n_iter > 0) load_stats(0);
        for (int it = 0; it < n_iter && ok; it++) {
            const uint32_t par = (uint32_t)it & 1;
            const int hh = it / per_head;
            const long long c0 = (long long)(t_begin + it - hh * per_head) * BT + wg * 64;  // first query column of this warpgroup
            // each warp stages its 64 columns' statistics once (log2 units, times the scale): its lanes then read them as
            // shared-memory broadcasts
            __syncwarp();
#pragma unroll
            for (int u = 0; u < 2; u++) stat_lse[lane + 32 * u] = nl[u] * LOG2E, stat_delta[lane + 32 * u] = nd[u] * p.scale;
            __syncwarp();
            if (it + 1 < n_iter) load_stats(it + 1);
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(xy_full, par, abort_flag)))) break;
            tc_fence_after();
            // query i sees key `row` iff row <= i + offset, and i < Sq: visible columns [lo, hi) relative to c0
            const long long col_lo = p.causal ? row - p.causal_offset : 0;
            const int lo = (int)max(0LL, min(col_lo - c0, 64LL)), hi = (int)max(0LL, min((long long)p.Sq - c0, 64LL));
            const bool masked_tile = __any_sync(0xffffffffu, lo > 0 || hi < 64);
            auto compute = [&](auto masked) -> bool {
#pragma unroll
                for (int c = 0; c < 2; c++) {  // 32 columns at a time: bf16 pairs of the probabilities and of dS
                    uint32_t x[32], y[32], pp[16], zz[16];
                    tmem_ld_32x32(tmem_x + lane_addr + wg * 64 + c * 32, x);
                    tmem_ld_32x32(tmem_y + lane_addr + wg * 64 + c * 32, y);
                    tmem_ld_wait();
                    if (c == 1) {  // X and Y are in registers: the next tile's products may overwrite them
                        tc_fence_before();
                        mbar_arrive(xy_empty);
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 l4 = *(const float4*)(stat_lse + c * 32 + i), d4 = *(const float4*)(stat_delta + c * 32 + i);
                        const float lse4[4] = {l4.x, l4.y, l4.z, l4.w}, dsc4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                        for (int u = 0; u < 4; u += 2) {
                            const int e = c * 32 + i + u, f = i + u;
                            const float2 arg = __ffma2_rn(make_float2(__uint_as_float(x[f]), __uint_as_float(x[f + 1])),
                                                          make_float2(p.scale_log2, p.scale_log2), make_float2(-lse4[u], -lse4[u + 1]));
                            float2 pr = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                            if (decltype(masked)::value) {
                                if (e < lo || e >= hi) pr.x = 0.0f;
                                if (e + 1 < lo || e + 1 >= hi) pr.y = 0.0f;
                            }
                            const float2 t = __ffma2_rn(make_float2(__uint_as_float(y[f]), __uint_as_float(y[f + 1])),
                                                        make_float2(p.scale, p.scale), make_float2(-dsc4[u], -dsc4[u + 1]));
                            const float2 z = __fmul2_rn(pr, t);  // P * (dP - delta) * scale
                            __nv_bfloat162 ph2 = __floats2bfloat162_rn(pr.x, pr.y);
                            __nv_bfloat162 zh2 = __floats2bfloat162_rn(z.x, z.y);
                            pp[(i + u) / 2] = *(uint32_t*)&ph2;
                            zz[(i + u) / 2] = *(uint32_t*)&zh2;
                        }
                    }
                    if (c == 0) {
                        if (it > 0) {
                            // P and Z go where the previous tile's were: the products that read them have to have completed
                            if (!__all_sync(0xffffffffu, mbar_wait(pz_free, par ^ 1, abort_flag))) return false;
                            tc_fence_after();
                        }
                    }
                    tmem_st_32x16(tmem_p + lane_addr + wg * 32 + c * 16, pp);
#pragma unroll
                    for (int j = 0; j < 4; j++)  // 16-byte chunk c * 4 + j of this key row's 128 bytes, swizzled as TMA would write it
                        *(uint4*)(z_row + (((c * 4 + j) ^ z_swz) * 16)) = make_uint4(zz[4 * j], zz[4 * j + 1], zz[4 * j + 2], zz[4 * j + 3]);
                }
                return true;
            };
            if (!(ok = masked_tile ? compute(std::true_type{}) : compute(std::false_type{}))) break;
            tmem_st_wait();
            tc_fence_before();
            fence_proxy_async();  // Z was written through the generic proxy and is read by the tensor core
            mbar_arrive(pz_ready);
        }
        // ---- epilogue: dK (first warpgroup) and dV (second) -> bf16 rows ----
        if (n_iter > 0) ok = ok && mbar_wait(acc_full, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            uint16_t* base = (uint16_t*)(wg == 0 ? p.dk : p.dv);
            const long long sb = wg == 0 ? p.k_sb : p.v_sb, ss = wg == 0 ? p.k_ss : p.v_ss, sn = wg == 0 ? p.k_sn : p.v_sn;
            uint16_t* out = base + (long long)batch * sb + row * ss + (long long)head * sn;
            const bool vec = (sb % 8 == 0) && (ss % 8 == 0) && (sn % 8 == 0) && (((uintptr_t)base & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < D / 32; c++) {
                uint32_t v[32];
                if (n_iter > 0) {
                    tmem_ld_32x32((wg == 0 ? tmem_dk : tmem_dv) + lane_addr + c * 32, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = 0u;
                }
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
                if (vec && n_iter > 0) {
                    // the warp's 32 rows leave through 2 KB of the resident K tile (every product that read it has completed)
                    store_rows_coalesced<4>((uint4*)(sk + (warp - 8) * 2048), packed, (uint8_t*)(out - (long long)lane * ss + c * 32), ss * 2,
                                            (int)max(0LL, min(32LL, (long long)p.Sk - (row - lane))), lane);
                } else if (row < p.Sk) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (vec) {
                            *(uint4*)(out + c * 32 + i * 8) = packed[i];
                        } else {
                            const uint32_t w[4] = {packed[i].x, packed[i].y, packed[i].z, packed[i].w};
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                out[c * 32 + i * 8 + 2 * q] = (uint16_t)(w[q] & 0xffff);
                                out[c * 32 + i * 8 + 2 * q + 1] = (uint16_t)(w[q] >> 16);
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
        tmem_dealloc(tmem_base, 512);
    }
}

// dq[b, s, n, :] = bf16(acc[b, s, n, :]): 8 values (32 bytes in, 16 out) per thread; the accumulator is dense, dq a view.
__global__ void __launch_bounds__(256) attention_dq_round(const float* __restrict__ acc, uint16_t* __restrict__ dq, long long rows, int N,
                                                           long long sb_rows, long long q_sb, long long q_ss, long long q_sn) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long r = t >> 3;  // (b, s, n) row of 64 values
    const int part = (int)(t & 7);
    if (r >= rows) return;
    const float4 a = __ldg((const float4*)(acc + r * D + part * 8)), b = __ldg((const float4*)(acc + r * D + part * 8 + 4));
    const long long bs = r / N;
    const int n = (int)(r - bs * N);
    const long long bi = bs / sb_rows, s = bs - bi * sb_rows;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
    uint16_t* out = dq + bi * q_sb + s * q_ss + (long long)n * q_sn + part * 8;
    *(uint4*)out = make_uint4(*(uint32_t*)&h0, *(uint32_t*)&h1, *(uint32_t*)&h2, *(uint32_t*)&h3);
}

}  // namespace

bool attention_bwd_atomic_supported(const lb_tensor& q, const lb_tensor& dq) {
    return q.shape[3] == D && dq.stride[0] % 8 == 0 && dq.stride[1] % 8 == 0 && dq.stride[2] % 8 == 0 && ((uintptr_t)dq.ptr & 15) == 0;
}

size_t attention_bwd_atomic_scratch_bytes(const lb_tensor& q) { return (size_t)q.shape[0] * q.shape[1] * q.shape[2] * q.shape[3] * 4; }

// The single-kernel backward over operands already validated by attention_bwd's caller; `delta` has been computed.
namespace {
// 4-d map over the dense float32 accumulator [B, Sq, N, 64]: boxes of 32 columns x 128 query rows, 128-byte swizzle
CUtensorMap make_acc_map(float* acc, long long B, long long Sq, long long N) {
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)Sq, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)D * 4, (cuuint64_t)N * D * 4, (cuuint64_t)Sq * N * D * 4};
    cuuint32_t box[4] = {32, 1, (cuuint32_t)BT, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap map;
    check_cu(driver().cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, acc, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
             "cuTensorMapEncodeTiled(attention dQ accumulator)");
    return map;
}
}  // namespace

void attention_bwd_atomic_launch(const lb_attn_desc& desc, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mq,
                                 const CUtensorMap& mdo, const lb_tensor& q, const lb_tensor& k, const float* lse, const float* delta,
                                 float* dq_acc, const lb_tensor& dq, const lb_tensor& dk, const lb_tensor& dv, cudaStream_t s) {
    const long long B = q.shape[0], Sq = q.shape[1], N = q.shape[2], Sk = k.shape[1], Nkv = k.shape[2];
    AtomicArgs a{};
    a.B = (int)B, a.N = (int)N, a.Nkv = (int)Nkv, a.Sq = (int)Sq, a.Sk = (int)Sk;
    a.causal = desc.causal, a.causal_offset = desc.causal_offset;
    a.scale = desc.scale, a.scale_log2 = desc.scale * 1.4426950408889634f;
    a.lse = lse, a.delta = delta, a.dq_acc = dq_acc;
    a.dk = dk.ptr, a.k_sb = dk.stride[0], a.k_ss = dk.stride[1], a.k_sn = dk.stride[2];
    a.dv = dv.ptr, a.v_sb = dv.stride[0], a.v_ss = dv.stride[1], a.v_sn = dv.stride[2];
    a.status = status_word();
    if (first_use_on_device((const void*)attention_bwd_atomic_kernel)) {
        cudaFuncAttributes attr;
        LB_CUDA(cudaFuncGetAttributes(&attr, attention_bwd_atomic_kernel));
        if (attr.numRegs != kLaunchRegs)
            fail(LB_ERR_UNSUPPORTED, format("attention backward: the single-kernel form was built with %d registers per thread, its register "
                                            "budgets assume %d", attr.numRegs, kLaunchRegs));
        LB_CUDA(cudaFuncSetAttribute(attention_bwd_atomic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    }
    LB_CUDA(cudaMemsetAsync(dq_acc, 0, (size_t)B * Sq * N * D * 4, s));
    dim3 grid((unsigned)((Sk + BR - 1) / BR), (unsigned)Nkv, (unsigned)B);
    if (((uintptr_t)dq_acc & 15) != 0) fail(LB_ERR_UNSUPPORTED, "attention backward: the dQ accumulator must be 16-byte aligned");
    attention_bwd_atomic_kernel<<<grid, kThreads, kSmemBytes, s>>>(mk, mv, mq, mdo, make_acc_map(dq_acc, B, Sq, N), a);
    LB_CUDA(cudaGetLastError());
    const long long rows = B * Sq * N;
    attention_dq_round<<<(unsigned)((rows * 8 + 255) / 256), 256, 0, s>>>(dq_acc, (uint16_t*)dq.ptr, rows, (int)N, Sq, dq.stride[0], dq.stride[1],
                                                                           dq.stride[2]);
    LB_CUDA(cudaGetLastError());
}

}  // namespace lb
