// Row gather/scatter and a CUDA-core attention for the shapes the tensor-core kernels do not take.
//
//  * scatter_add_rows: out[clamp(ids[t]), :] += updates[t, :] (the embedding gradient; lumen/reference/mod.rs:765-808),
//    in the two forms of the reference's backends (lumen/codegen/scatter_add/README.md:23-39). The DETERMINISTIC form
//    (count, starts, place, sort, rows) adds a row's updates in update order, rounding to the operand's dtype after
//    every add exactly like the interpreter: bit-identical to it and from run to run. The ATOMIC form adds in float32
//    atomics in arrival order and rounds once: results vary in the last bits when a row is hit more than once.
//  * attention_simt_fwd / attention_simt_bwd: float32 or bfloat16, any head dim up to 256, one warp per query row,
//    scores and sums in float32 in key order. Used for float32 graphs (no hidden narrowing to bf16 tensor cores)
//    and head dims other than 64/128.
#include "device.h"

#include <cuda_bf16.h>

#include <algorithm>

namespace lb {
namespace {

template <class T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <class T, class I>
__global__ void scatter_add_rows_kernel(float* __restrict__ acc, const I* __restrict__ ids, const T* __restrict__ updates,
                                        long long tokens, long long rows, int width) {
    const long long t = blockIdx.x;
    if (t >= tokens) return;
    long long r = (long long)ids[t];
    r = r < 0 ? 0 : (r > rows - 1 ? rows - 1 : r);
    for (int d = threadIdx.x; d < width; d += blockDim.x) atomicAdd(acc + r * width + d, to_f(updates[t * width + d]));
}

template <class T>
__global__ void add_convert_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ acc, long long n, int has_x) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // out = x + sum(updates): one rounding of the float32 sum into the operand dtype
    out[i] = from_f<T>(has_x ? __fadd_rn(to_f(x[i]), acc[i]) : acc[i]);
}

// ---- deterministic scatter-add: a counting sort of the picks by destination row, then one block per row -----------
template <class I>
__device__ __forceinline__ int clamped_row(const I* ids, long long t, long long rows) {
    long long r = (long long)ids[t];
    return (int)(r < 0 ? 0 : (r > rows - 1 ? rows - 1 : r));
}

template <class I>
__global__ void scatter_count_kernel(int* __restrict__ counts, const I* __restrict__ ids, long long tokens, long long rows) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < tokens) atomicAdd(counts + clamped_row(ids, t, rows), 1);  // integer atomics: the counts do not depend on order
}

// starts[r] = sum of counts[0 .. r), starts[rows] = tokens; one block walks the rows in chunks of its size.
__global__ void scatter_starts_kernel(int* __restrict__ starts, const int* __restrict__ counts, long long rows) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long base = 0; base < rows; base += blockDim.x) {
        const long long r = base + threadIdx.x;
        const int c = r < rows ? counts[r] : 0;
        int incl = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int up = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += up;
            }
            warp_sums[lane] = w;  // inclusive over warps
        }
        __syncthreads();
        const int before = carry + (warp ? warp_sums[warp - 1] : 0) + incl - c;
        if (r < rows) starts[r] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry = before + c;
        __syncthreads();
    }
    if (threadIdx.x == 0) starts[rows] = carry;
}

template <class I>
__global__ void scatter_place_kernel(int* __restrict__ order, int* __restrict__ cursor, const int* __restrict__ starts,
                                     const I* __restrict__ ids, long long tokens, long long rows) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const int r = clamped_row(ids, t, rows);
    order[starts[r] + atomicAdd(cursor + r, 1)] = (int)t;  // arrival order within the row's segment; sorted next
}

// One block per destination row: sorts the row's picks into update order (ascending update number), then every thread
// owns columns and adds the row's updates one after the other, rounding to T after each add as the interpreter does.
// Short segments are sorted in shared memory (bitonic); longer ones by rank (every pick counts the smaller ones) into
// `sorted`, a second array of `tokens` ints.
constexpr int kSortSmem = 2048;
template <class T>
__global__ void scatter_rows_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ updates, const int* __restrict__ starts,
                                    const int* __restrict__ order, int* __restrict__ sorted, int width, int has_x) {
    __shared__ int picks[kSortSmem];
    const long long r = blockIdx.x;
    const int begin = starts[r], n = starts[r + 1] - begin;
    const int* list = picks;
    if (n <= kSortSmem) {
        int padded = 1;
        while (padded < n) padded <<= 1;
        for (int i = threadIdx.x; i < padded; i += blockDim.x) picks[i] = i < n ? order[begin + i] : 0x7fffffff;
        __syncthreads();
        for (int k = 2; k <= padded; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = threadIdx.x; i < padded; i += blockDim.x) {
                    const int partner = i ^ j;
                    if (partner > i) {
                        const int a = picks[i], b = picks[partner];
                        const bool up = (i & k) == 0;
                        if ((a > b) == up) picks[i] = b, picks[partner] = a;
                    }
                }
                __syncthreads();
            }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int mine = order[begin + i];
            int rank = 0;
            for (int j = 0; j < n; j++) rank += order[begin + j] < mine;
            sorted[begin + rank] = mine;  // update numbers are distinct: ranks are a permutation
        }
        __syncthreads();
        list = sorted + begin;
    }
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float acc = has_x ? to_f(x[r * width + d]) : 0.0f;
        for (int i = 0; i < n; i++) acc = to_f(from_f<T>(__fadd_rn(acc, to_f(updates[(long long)list[i] * width + d]))));
        out[r * width + d] = from_f<T>(acc);
    }
}

struct AttnShape {
    int B, Sq, Sk, N, Nkv, D;
    long long q_s[3], k_s[3], v_s[3], o_s[3], g_s[3], dq_s[3], dk_s[3], dv_s[3];  // strides of dims B, S, N (head dim is dense)
    int causal;
    long long offset;
    float scale;
};

// one warp per (b, n, i): online softmax over the visible keys; lane l owns head-dim elements l, l+32, ...
template <class T>
__global__ void attention_simt_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
                                          float* __restrict__ lse, AttnShape s) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)s.B * s.N * s.Sq) return;
    const int i = (int)(w % s.Sq), n = (int)((w / s.Sq) % s.N), b = (int)(w / ((long long)s.Sq * s.N));
    const int nk = n / (s.N / s.Nkv);
    const T* qp = q + b * s.q_s[0] + (long long)i * s.q_s[1] + n * s.q_s[2];
    float qv[8], acc[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        qv[u] = d < s.D ? to_f(qp[d]) : 0.0f;
        acc[u] = 0.0f;
    }
    long long last = s.causal ? min((long long)s.Sk - 1, (long long)i + s.offset) : (long long)s.Sk - 1;
    float m = -INFINITY, l = 0.0f;
    for (long long j = 0; j <= last; j++) {
        const T* kp = k + b * s.k_s[0] + j * s.k_s[1] + nk * s.k_s[2];
        float dot = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int d = lane + 32 * u;
            if (d < s.D) dot = fmaf(qv[u], to_f(kp[d]), dot);
        }
#pragma unroll
        for (int x = 16; x >= 1; x >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, x);
        const float sc = dot * s.scale;
        const float m_new = fmaxf(m, sc);
        const float alpha = __expf(m - m_new), p = __expf(sc - m_new);
        // the value product sees the probability in the operands' dtype; the normaliser is applied at the end
        l = l * alpha + p;
        const T* vp = v + b * s.v_s[0] + j * s.v_s[1] + nk * s.v_s[2];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int d = lane + 32 * u;
            if (d < s.D) acc[u] = fmaf(acc[u], alpha, p * to_f(vp[d]));
        }
        m = m_new;
    }
    T* op = o + b * s.o_s[0] + (long long)i * s.o_s[1] + n * s.o_s[2];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        if (d < s.D) op[d] = from_f<T>(acc[u] / l);
    }
    if (lse && lane == 0) lse[((long long)b * s.N + n) * s.Sq + i] = m + logf(l);
}

// dQ: one warp per query row. dK/dV: one warp per (b, kv head, key j), looping over the group's heads and the queries that see j.
template <class T>
__global__ void attention_simt_dq_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                                         const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq, AttnShape s) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)s.B * s.N * s.Sq) return;
    const int i = (int)(w % s.Sq), n = (int)((w / s.Sq) % s.N), b = (int)(w / ((long long)s.Sq * s.N));
    const int nk = n / (s.N / s.Nkv);
    const T* qp = q + b * s.q_s[0] + (long long)i * s.q_s[1] + n * s.q_s[2];
    const T* gp = g + b * s.g_s[0] + (long long)i * s.g_s[1] + n * s.g_s[2];
    float qv[8], gv[8], acc[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        qv[u] = d < s.D ? to_f(qp[d]) : 0.0f;
        gv[u] = d < s.D ? to_f(gp[d]) : 0.0f;
        acc[u] = 0.0f;
    }
    const long long at = ((long long)b * s.N + n) * s.Sq + i;
    const float L = lse[at], dl = delta[at];
    long long last = s.causal ? min((long long)s.Sk - 1, (long long)i + s.offset) : (long long)s.Sk - 1;
    for (long long j = 0; j <= last; j++) {
        const T* kp = k + b * s.k_s[0] + j * s.k_s[1] + nk * s.k_s[2];
        const T* vp = v + b * s.v_s[0] + j * s.v_s[1] + nk * s.v_s[2];
        float dot = 0.0f, dp = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int d = lane + 32 * u;
            if (d < s.D) {
                dot = fmaf(qv[u], to_f(kp[d]), dot);
                dp = fmaf(gv[u], to_f(vp[d]), dp);
            }
        }
#pragma unroll
        for (int x = 16; x >= 1; x >>= 1) {
            dot += __shfl_xor_sync(0xffffffffu, dot, x);
            dp += __shfl_xor_sync(0xffffffffu, dp, x);
        }
        const float p = __expf(dot * s.scale - L);
        const float ds = to_f(from_f<T>(p * (dp - dl) * s.scale));  // dS is rounded to the operands' dtype (flash.py:71)
#pragma unroll
        for (int u = 0; u < 8; u++) {
            int d = lane + 32 * u;
            if (d < s.D) acc[u] = fmaf(ds, to_f(kp[d]), acc[u]);
        }
    }
    T* out = dq + b * s.dq_s[0] + (long long)i * s.dq_s[1] + n * s.dq_s[2];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        if (d < s.D) out[d] = from_f<T>(acc[u]);
    }
}

template <class T>
__global__ void attention_simt_dkdv_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                                           const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dk,
                                           T* __restrict__ dv, AttnShape s) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)s.B * s.Nkv * s.Sk) return;
    const int j = (int)(w % s.Sk), nk = (int)((w / s.Sk) % s.Nkv), b = (int)(w / ((long long)s.Sk * s.Nkv));
    const int group = s.N / s.Nkv;
    const T* kp = k + b * s.k_s[0] + (long long)j * s.k_s[1] + nk * s.k_s[2];
    const T* vp = v + b * s.v_s[0] + (long long)j * s.v_s[1] + nk * s.v_s[2];
    float kv[8], vv[8], ak[8], av[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        kv[u] = d < s.D ? to_f(kp[d]) : 0.0f;
        vv[u] = d < s.D ? to_f(vp[d]) : 0.0f;
        ak[u] = av[u] = 0.0f;
    }
    long long first = s.causal ? max(0LL, (long long)j - s.offset) : 0LL;
    for (int h = 0; h < group; h++) {
        const int n = nk * group + h;
        for (long long i = first; i < s.Sq; i++) {
            const T* qp = q + b * s.q_s[0] + i * s.q_s[1] + n * s.q_s[2];
            const T* gp = g + b * s.g_s[0] + i * s.g_s[1] + n * s.g_s[2];
            float dot = 0.0f, dp = 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                int d = lane + 32 * u;
                if (d < s.D) {
                    dot = fmaf(kv[u], to_f(qp[d]), dot);
                    dp = fmaf(vv[u], to_f(gp[d]), dp);
                }
            }
#pragma unroll
            for (int x = 16; x >= 1; x >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, x);
                dp += __shfl_xor_sync(0xffffffffu, dp, x);
            }
            const long long at = ((long long)b * s.N + n) * s.Sq + i;
            const float p = __expf(dot * s.scale - lse[at]);
            const float ds = to_f(from_f<T>(p * (dp - delta[at]) * s.scale));
            const float pr = to_f(from_f<T>(p));
#pragma unroll
            for (int u = 0; u < 8; u++) {
                int d = lane + 32 * u;
                if (d < s.D) {
                    ak[u] = fmaf(ds, to_f(qp[d]), ak[u]);
                    av[u] = fmaf(pr, to_f(gp[d]), av[u]);
                }
            }
        }
    }
    T* ok = dk + b * s.dk_s[0] + (long long)j * s.dk_s[1] + nk * s.dk_s[2];
    T* ov = dv + b * s.dv_s[0] + (long long)j * s.dv_s[1] + nk * s.dv_s[2];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        int d = lane + 32 * u;
        if (d < s.D) ok[d] = from_f<T>(ak[u]), ov[d] = from_f<T>(av[u]);
    }
}

template <class T>
__global__ void attention_delta_simt(const T* __restrict__ o, const T* __restrict__ g, float* __restrict__ delta, AttnShape s) {
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)s.B * s.N * s.Sq) return;
    const int i = (int)(w % s.Sq), n = (int)((w / s.Sq) % s.N), b = (int)(w / ((long long)s.Sq * s.N));
    const T* op = o + b * s.o_s[0] + (long long)i * s.o_s[1] + n * s.o_s[2];
    const T* gp = g + b * s.g_s[0] + (long long)i * s.g_s[1] + n * s.g_s[2];
    float acc = 0.0f;
    for (int d = lane; d < s.D; d += 32) acc = fmaf(to_f(op[d]), to_f(gp[d]), acc);
#pragma unroll
    for (int x = 16; x >= 1; x >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
    if (lane == 0) delta[((long long)b * s.N + n) * s.Sq + i] = acc;
}

// out[c, r] = in[r, c] for dense row-major 2-byte or 4-byte elements: 32 x 32 tiles through shared memory, both sides
// coalesced. Used by plans to give a GEMM a K-major copy of a weight whose rows are 8 KB or more apart.
template <class T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols) {
    __shared__ T tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int r = r0 + ty + k, c = c0 + tx;
        if (r < rows && c < cols) tile[ty + k][tx] = in[(long long)r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int c = c0 + ty + k, r = r0 + tx;
        if (r < rows && c < cols) out[(long long)c * rows + r] = tile[tx][ty + k];
    }
}

void fill_strides(long long* dst, const lb_tensor& t) {
    for (int d = 0; d < 3; d++) dst[d] = t.stride[d];
    if (t.stride[3] != 1 && t.shape[3] > 1) fail(LB_ERR_UNSUPPORTED, "attention: the head dimension must be dense");
}

}  // namespace

// bfloat16 noise in [-1, 1) from a linear congruential generator, over a whole buffer: what an autotuner times its
// candidates on (a GPU's clocks under all-zero operands differ from those under real data).
__global__ void fill_noise_kernel(uint16_t* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t x = (uint32_t)i * 1664525u + 1013904223u;
        x = x * 1664525u + 1013904223u;
        const float f = (float)(x >> 8) * (2.0f / 16777216.0f) - 1.0f;
        out[i] = __bfloat16_as_ushort(__float2bfloat16_rn(f));
    }
}

void fill_noise(void* ptr, size_t bytes, void* stream) {
    const size_t n = bytes / 2;
    if (n == 0) return;
    driver();
    fill_noise_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 148 * 16), 256, 0, (cudaStream_t)stream>>>((uint16_t*)ptr, n);
    LB_CUDA(cudaGetLastError());
}

size_t scatter_add_scratch_bytes(long long rows, long long width, long long tokens, bool deterministic) {
    // deterministic: counts[rows], cursor[rows], starts[rows + 1], order[tokens], sorted[tokens]; atomic: float32 rows
    return deterministic ? (size_t)(3 * rows + 1 + 2 * tokens) * 4 : (size_t)rows * width * 4;
}

void scatter_add_rows(const lb_tensor& x, const lb_tensor& ids, const lb_tensor& updates, const lb_tensor& out, void* scratch,
                      bool x_is_zero, bool deterministic, void* stream) {
    if (x.rank != 2) fail(LB_ERR_UNSUPPORTED, "scatter_add: a [rows, width] operand scattered along axis 0");
    const long long rows = x.shape[0], width = x.shape[1];
    long long tokens = 1;
    for (int d = 0; d < ids.rank; d++) tokens *= ids.shape[d];
    check_dense(x, x.dtype, {rows, width}, "scatter_add operand");
    check_dense(out, x.dtype, {rows, width}, "scatter_add result");
    if (updates.dtype != x.dtype) fail(LB_ERR_INVALID, "scatter_add: updates must have the operand's dtype");
    if (x.dtype != LB_F32 && x.dtype != LB_BF16) fail(LB_ERR_UNSUPPORTED, "scatter_add: float32 or bfloat16 rows");
    if (ids.dtype != LB_I64 && ids.dtype != LB_I32) fail(LB_ERR_INVALID, "scatter_add: int32 or int64 indices");
    if (!scratch || ((uintptr_t)scratch & 3)) fail(LB_ERR_INVALID, "scatter_add: needs scratch memory (scatter_add_scratch_bytes), 4-byte aligned");
    if (rows > INT32_MAX || tokens > INT32_MAX || width > INT32_MAX) fail(LB_ERR_UNSUPPORTED, "scatter_add: more than 2^31 rows, updates or columns");
    driver();
    cudaStream_t s = (cudaStream_t)stream;
    if (rows == 0 || width == 0) return;
    if (deterministic) {
        int* counts = (int*)scratch;
        int* cursor = counts + rows;
        int* starts = cursor + rows;
        int* order = starts + rows + 1;
        int* sorted = order + tokens;
        LB_CUDA(cudaMemsetAsync(counts, 0, (size_t)rows * 2 * 4, s));  // counts and cursor start at zero
        if (tokens > 0) {
            const unsigned blocks = (unsigned)((tokens + 255) / 256);
            if (ids.dtype == LB_I64) scatter_count_kernel<long long><<<blocks, 256, 0, s>>>(counts, (const long long*)ids.ptr, tokens, rows);
            else scatter_count_kernel<int><<<blocks, 256, 0, s>>>(counts, (const int*)ids.ptr, tokens, rows);
        }
        scatter_starts_kernel<<<1, 1024, 0, s>>>(starts, counts, rows);
        if (tokens > 0) {
            const unsigned blocks = (unsigned)((tokens + 255) / 256);
            if (ids.dtype == LB_I64) scatter_place_kernel<long long><<<blocks, 256, 0, s>>>(order, cursor, starts, (const long long*)ids.ptr, tokens, rows);
            else scatter_place_kernel<int><<<blocks, 256, 0, s>>>(order, cursor, starts, (const int*)ids.ptr, tokens, rows);
        }
        const int threads = (int)std::min<long long>(256, ((width + 31) / 32) * 32);
        if (x.dtype == LB_F32)
            scatter_rows_kernel<float><<<(unsigned)rows, threads, 0, s>>>((float*)out.ptr, (const float*)x.ptr, (const float*)updates.ptr, starts, order, sorted, (int)width, !x_is_zero);
        else
            scatter_rows_kernel<__nv_bfloat16><<<(unsigned)rows, threads, 0, s>>>((__nv_bfloat16*)out.ptr, (const __nv_bfloat16*)x.ptr, (const __nv_bfloat16*)updates.ptr, starts, order, sorted, (int)width, !x_is_zero);
        LB_CUDA(cudaGetLastError());
        return;
    }
    float* acc = (float*)scratch;
    LB_CUDA(cudaMemsetAsync(acc, 0, (size_t)rows * width * 4, s));
    if (tokens > 0 && width > 0) {
        int threads = (int)std::min<long long>(256, ((width + 31) / 32) * 32);
        if (x.dtype == LB_F32) {
            if (ids.dtype == LB_I64) scatter_add_rows_kernel<float, long long><<<(unsigned)tokens, threads, 0, s>>>(acc, (const long long*)ids.ptr, (const float*)updates.ptr, tokens, rows, (int)width);
            else scatter_add_rows_kernel<float, int><<<(unsigned)tokens, threads, 0, s>>>(acc, (const int*)ids.ptr, (const float*)updates.ptr, tokens, rows, (int)width);
        } else {
            if (ids.dtype == LB_I64) scatter_add_rows_kernel<__nv_bfloat16, long long><<<(unsigned)tokens, threads, 0, s>>>(acc, (const long long*)ids.ptr, (const __nv_bfloat16*)updates.ptr, tokens, rows, (int)width);
            else scatter_add_rows_kernel<__nv_bfloat16, int><<<(unsigned)tokens, threads, 0, s>>>(acc, (const int*)ids.ptr, (const __nv_bfloat16*)updates.ptr, tokens, rows, (int)width);
        }
    }
    const long long n = rows * width;
    if (n > 0) {
        if (x.dtype == LB_F32) add_convert_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((float*)out.ptr, (const float*)x.ptr, acc, n, !x_is_zero);
        else add_convert_kernel<__nv_bfloat16><<<(unsigned)((n + 255) / 256), 256, 0, s>>>((__nv_bfloat16*)out.ptr, (const __nv_bfloat16*)x.ptr, acc, n, !x_is_zero);
    }
    LB_CUDA(cudaGetLastError());
}

static AttnShape attn_shape(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v) {
    if (q.rank != 4 || k.rank != 4 || v.rank != 4) fail(LB_ERR_INVALID, "attention: operands must be [B, S, N, H] tensors");
    AttnShape s{};
    s.B = (int)q.shape[0], s.Sq = (int)q.shape[1], s.N = (int)q.shape[2], s.D = (int)q.shape[3];
    s.Sk = (int)k.shape[1], s.Nkv = (int)k.shape[2];
    if (s.D > 256 || v.shape[3] != s.D || s.Nkv == 0 || s.N % s.Nkv) fail(LB_ERR_UNSUPPORTED, "attention: head dim up to 256, equal for values, N a multiple of Nkv");
    fill_strides(s.q_s, q), fill_strides(s.k_s, k), fill_strides(s.v_s, v);
    s.causal = desc.causal, s.offset = desc.causal_offset, s.scale = desc.scale;
    return s;
}

void transpose_2d(const lb_tensor& in, const lb_tensor& out, void* stream) {
    if (in.rank != 2 || out.rank != 2 || in.dtype != out.dtype || in.shape[0] != out.shape[1] || in.shape[1] != out.shape[0] ||
        in.stride[1] != 1 || in.stride[0] != in.shape[1] || out.stride[1] != 1 || out.stride[0] != out.shape[1])
        fail(LB_ERR_INVALID, "transpose: dense row-major [R, C] in, [C, R] out of one dtype");
    const long long rows = in.shape[0], cols = in.shape[1];
    if (rows == 0 || cols == 0) return;
    if (rows > INT32_MAX || cols > INT32_MAX || (cols + 31) / 32 > INT32_MAX || (rows + 31) / 32 > 65535)
        fail(LB_ERR_UNSUPPORTED, "transpose: matrix too large for the kernel's grid");
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    const int size = dtype_size(in.dtype);
    if (size == 2) transpose_kernel<uint16_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)in.ptr, (uint16_t*)out.ptr, (int)rows, (int)cols);
    else if (size == 4) transpose_kernel<uint32_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint32_t*)in.ptr, (uint32_t*)out.ptr, (int)rows, (int)cols);
    else fail(LB_ERR_UNSUPPORTED, "transpose: 2-byte and 4-byte elements");
    LB_CUDA(cudaGetLastError());
}

// ---- a view copied element by element: any strides on either side ---------------------------------------------------
// The plan's copies of views that are neither dense nor rows of a wider matrix (a permuted or sliced tensor made dense
// for a kernel that reads dense operands, or written out as a graph output). Consecutive threads take consecutive
// elements of the destination's index order, so a dense destination is written in whole lines.
struct CopyDims {
    int rank;
    long long shape[LB_MAX_RANK], src[LB_MAX_RANK], dst[LB_MAX_RANK];
};

template <class T>
__global__ void strided_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, CopyDims d, long long total) {
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        long long rest = i, from = 0, to = 0;
        for (int k = d.rank - 1; k >= 0; k--) {
            const long long c = rest % d.shape[k];
            rest /= d.shape[k];
            from += c * d.src[k], to += c * d.dst[k];
        }
        dst[to] = src[from];
    }
}

// The same copy when the source is contiguous along one axis (a) and the destination along another (b): 32 x 32 tiles
// over those two axes go through shared memory, read along a and written along b, so both sides move whole lines. The
// other axes are enumerated by the block index.
template <class T>
__global__ void __launch_bounds__(256) tiled_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, CopyDims d, int a, int b, long long tiles_a,
                                                         long long tiles_b) {
    __shared__ T tile[32][33];
    long long block = blockIdx.x;
    const long long ta = block % tiles_a;
    block /= tiles_a;
    const long long tb = block % tiles_b;
    block /= tiles_b;
    long long from = 0, to = 0;
    for (int k = d.rank - 1; k >= 0; k--) {
        if (k == a || k == b) continue;
        const long long c = block % d.shape[k];
        block /= d.shape[k];
        from += c * d.src[k], to += c * d.dst[k];
    }
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        const long long ia = ta * 32 + tx, ib = tb * 32 + j;
        if (ia < d.shape[a] && ib < d.shape[b]) tile[j][tx] = src[from + ia * d.src[a] + ib * d.src[b]];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const long long ia = ta * 32 + j, ib = tb * 32 + tx;
        if (ia < d.shape[a] && ib < d.shape[b]) dst[to + ia * d.dst[a] + ib * d.dst[b]] = tile[tx][j];
    }
}

void strided_copy(const lb_tensor& in, const lb_tensor& out, void* stream) {
    if (in.rank != out.rank || in.dtype != out.dtype) fail(LB_ERR_INVALID, "copy: views of one rank and dtype");
    CopyDims d{};
    long long total = 1;
    for (int k = 0; k < in.rank; k++) {
        if (in.shape[k] != out.shape[k]) fail(LB_ERR_INVALID, "copy: views of one shape");
        total *= in.shape[k];
        if (in.shape[k] == 1) continue;  // contributes no offset
        // an axis that continues the one before it on both sides is merged into it
        if (d.rank > 0 && d.src[d.rank - 1] == in.stride[k] * in.shape[k] && d.dst[d.rank - 1] == out.stride[k] * out.shape[k]) {
            d.shape[d.rank - 1] *= in.shape[k], d.src[d.rank - 1] = in.stride[k], d.dst[d.rank - 1] = out.stride[k];
            continue;
        }
        d.shape[d.rank] = in.shape[k], d.src[d.rank] = in.stride[k], d.dst[d.rank] = out.stride[k];
        d.rank++;
    }
    if (total == 0) return;
    cudaStream_t st = (cudaStream_t)stream;
    // contiguous along different axes on the two sides (a transposition of the last axis with another): tiles
    int a = -1, b = -1;
    for (int k = 0; k < d.rank; k++) {
        if (d.src[k] == 1 && a < 0) a = k;
        if (d.dst[k] == 1 && b < 0) b = k;
    }
    if (a >= 0 && b >= 0 && a != b && d.shape[a] >= 8 && d.shape[b] >= 8) {
        const long long tiles_a = (d.shape[a] + 31) / 32, tiles_b = (d.shape[b] + 31) / 32;
        const long long blocks = total / (d.shape[a] * d.shape[b]) * tiles_a * tiles_b;
        if (blocks <= 0x7fffffffLL) {
            switch (dtype_size(in.dtype)) {
                case 1: tiled_copy_kernel<uint8_t><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)in.ptr, (uint8_t*)out.ptr, d, a, b, tiles_a, tiles_b); break;
                case 2: tiled_copy_kernel<uint16_t><<<(unsigned)blocks, 256, 0, st>>>((const uint16_t*)in.ptr, (uint16_t*)out.ptr, d, a, b, tiles_a, tiles_b); break;
                case 4: tiled_copy_kernel<uint32_t><<<(unsigned)blocks, 256, 0, st>>>((const uint32_t*)in.ptr, (uint32_t*)out.ptr, d, a, b, tiles_a, tiles_b); break;
                default: tiled_copy_kernel<uint64_t><<<(unsigned)blocks, 256, 0, st>>>((const uint64_t*)in.ptr, (uint64_t*)out.ptr, d, a, b, tiles_a, tiles_b); break;
            }
            LB_CUDA(cudaGetLastError());
            return;
        }
    }
    const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, 148LL * 16);
    switch (dtype_size(in.dtype)) {
        case 1: strided_copy_kernel<uint8_t><<<blocks, 256, 0, st>>>((const uint8_t*)in.ptr, (uint8_t*)out.ptr, d, total); break;
        case 2: strided_copy_kernel<uint16_t><<<blocks, 256, 0, st>>>((const uint16_t*)in.ptr, (uint16_t*)out.ptr, d, total); break;
        case 4: strided_copy_kernel<uint32_t><<<blocks, 256, 0, st>>>((const uint32_t*)in.ptr, (uint32_t*)out.ptr, d, total); break;
        default: strided_copy_kernel<uint64_t><<<blocks, 256, 0, st>>>((const uint64_t*)in.ptr, (uint64_t*)out.ptr, d, total); break;
    }
    LB_CUDA(cudaGetLastError());
}

void attention_simt_fwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                        const lb_tensor* lse, void* stream) {
    AttnShape s = attn_shape(desc, q, k, v);
    fill_strides(s.o_s, o);
    driver();
    const long long warps = (long long)s.B * s.N * s.Sq;
    if (warps == 0) return;
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    cudaStream_t st = (cudaStream_t)stream;
    if (q.dtype == LB_F32) attention_simt_fwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)q.ptr, (const float*)k.ptr, (const float*)v.ptr, (float*)o.ptr, lse ? (float*)lse->ptr : nullptr, s);
    else if (q.dtype == LB_BF16) attention_simt_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)q.ptr, (const __nv_bfloat16*)k.ptr, (const __nv_bfloat16*)v.ptr, (__nv_bfloat16*)o.ptr, lse ? (float*)lse->ptr : nullptr, s);
    else fail(LB_ERR_UNSUPPORTED, "attention: float32 or bfloat16 operands");
    LB_CUDA(cudaGetLastError());
}

void attention_simt_bwd(const lb_attn_desc& desc, const lb_tensor& q, const lb_tensor& k, const lb_tensor& v, const lb_tensor& o,
                        const lb_tensor& g, const lb_tensor& lse, const lb_tensor& delta, const lb_tensor& dq, const lb_tensor& dk,
                        const lb_tensor& dv, void* stream) {
    AttnShape s = attn_shape(desc, q, k, v);
    fill_strides(s.o_s, o), fill_strides(s.g_s, g), fill_strides(s.dq_s, dq), fill_strides(s.dk_s, dk), fill_strides(s.dv_s, dv);
    driver();
    cudaStream_t st = (cudaStream_t)stream;
    const long long qw = (long long)s.B * s.N * s.Sq, kw = (long long)s.B * s.Nkv * s.Sk;
    if (qw == 0 || kw == 0) return;
    const unsigned qb = (unsigned)((qw * 32 + 255) / 256), kb = (unsigned)((kw * 32 + 255) / 256);
    if (q.dtype == LB_F32) {
        attention_delta_simt<float><<<qb, 256, 0, st>>>((const float*)o.ptr, (const float*)g.ptr, (float*)delta.ptr, s);
        attention_simt_dq_kernel<float><<<qb, 256, 0, st>>>((const float*)q.ptr, (const float*)k.ptr, (const float*)v.ptr, (const float*)g.ptr, (const float*)lse.ptr, (const float*)delta.ptr, (float*)dq.ptr, s);
        attention_simt_dkdv_kernel<float><<<kb, 256, 0, st>>>((const float*)q.ptr, (const float*)k.ptr, (const float*)v.ptr, (const float*)g.ptr, (const float*)lse.ptr, (const float*)delta.ptr, (float*)dk.ptr, (float*)dv.ptr, s);
    } else if (q.dtype == LB_BF16) {
        typedef __nv_bfloat16 H;
        attention_delta_simt<H><<<qb, 256, 0, st>>>((const H*)o.ptr, (const H*)g.ptr, (float*)delta.ptr, s);
        attention_simt_dq_kernel<H><<<qb, 256, 0, st>>>((const H*)q.ptr, (const H*)k.ptr, (const H*)v.ptr, (const H*)g.ptr, (const float*)lse.ptr, (const float*)delta.ptr, (H*)dq.ptr, s);
        attention_simt_dkdv_kernel<H><<<kb, 256, 0, st>>>((const H*)q.ptr, (const H*)k.ptr, (const H*)v.ptr, (const H*)g.ptr, (const float*)lse.ptr, (const float*)delta.ptr, (H*)dk.ptr, (H*)dv.ptr, s);
    } else {
        fail(LB_ERR_UNSUPPORTED, "attention: float32 or bfloat16 operands");
    }
    LB_CUDA(cudaGetLastError());
}

}  // namespace lb
