// Generator of loop-fused elementwise / reduction / row kernels for sm_100a.
//
// One fusion body (elementwise prims, layout prims, gathers, and reductions over the trailing axis) becomes ONE
// kernel over a [R, C] iteration space: a group of T threads walks each row in 16-byte vector chunks, reductions
// over the row are combined with warp shuffles (and shared memory across warps), and everything that reads a
// reduction result is recomputed from registers in a later phase over the same row, so each input element is
// read from HBM once. This is the counterpart of the reference's generated elementwise kernel
// (lumen/codegen/elementwise/cuda/mod.rs:54-333, kernel.py:56-167), of its Triton reduction kernels with fused
// prologue/epilogue (lumen/codegen/reduction/triton.rs) and of its row kernels for normalization diamonds
// (lumen/codegen/row/triton.rs), all of which only exist off-Blackwell.
//
// Numerics follow the reference interpreter (lumen/reference/mod.rs:442-695): one rounding to the result dtype
// after every primitive (16-bit floats are widened to f32, operated on once, rounded back), no multiply-add
// contraction (NVRTC --fmad=false), NaN-propagating max, integer division by zero = -1, two's complement wrap,
// saturating float->int casts, gather indices clamped. Row sums are combined in tree order, not the
// interpreter's sequential order: that is the one tolerance-level difference (reference tests allow 1e-5).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>

#include "fused.h"

namespace lb {
namespace {

const char* kPreamble = R"CUDA(
typedef long long i64; typedef unsigned long long u64; typedef unsigned int u32; typedef unsigned short u16;
typedef unsigned char u8; typedef signed char i8; typedef short i16; typedef int i32;
__device__ __forceinline__ float bf16_to_f32(u16 b) { return __uint_as_float(((u32)b) << 16); }
__device__ __forceinline__ u16 f32_to_bf16(float x) { u16 r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(x)); return r; }
__device__ __forceinline__ float rnd_bf16(float x) { return bf16_to_f32(f32_to_bf16(x)); }
__device__ __forceinline__ float f16_to_f32(u16 b) { float r; asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(b)); return r; }
__device__ __forceinline__ u16 f32_to_f16(float x) { u16 r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(x)); return r; }
__device__ __forceinline__ float rnd_f16(float x) { return f16_to_f32(f32_to_f16(x)); }
__device__ __forceinline__ float rnd_f32(float x) { return x; }
__device__ __forceinline__ double rnd_f64(double x) { return x; }
__device__ __forceinline__ float fmax_nan(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
// exp(x) of a softmax normaliser's term, x = value - row maximum <= 0, that is only summed: one multiply and one
// ex2.approx. Its relative error grows with |x| (to 5e-6 at -87) and results below 2^-126 flush to zero, but a term's
// weight in the sum (which holds exp(0) = 1) shrinks faster: the sum is within 2^-21 of the exactly rounded one.
__device__ __forceinline__ float exp_sum_term(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fmul_rn(x, 1.4426950408889634f))); return r; }
__device__ __forceinline__ double fmax_nan(double a, double b) { return (a != a || b != b) ? __longlong_as_double(0x7ff8000000000000LL) : fmax(a, b); }
__device__ __forceinline__ float fmin_nan(float a, float b) { float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ double fmin_nan(double a, double b) { return (a != a || b != b) ? __longlong_as_double(0x7ff8000000000000LL) : fmin(a, b); }
// Zero at run time (every launch of these kernels has one block along z), unknown at compile time. Integer negations are
// written RT_ZERO - x: with CUDA 12.9 for sm_100a, a chain of three or more signed 32-bit max (or min) whose operands
// are literal negations 0 - x comes out as the extremum over x and -x together (a stand-alone kernel shows it with
// `neg.s32` in inline assembly as well, so it happens after PTX); a subtraction from a register does not.
#define RT_ZERO blockIdx.z
template <class T> __device__ __forceinline__ T imax(T a, T b) { return a > b ? a : b; }
template <class T> __device__ __forceinline__ T imin(T a, T b) { return a < b ? a : b; }
// division by zero gives all ones and leaves the remainder a; a signed -1 divisor negates (wrapping at the lowest
// value, where the hardware division would trap or is undefined) - an unsigned divisor of all ones is an ordinary one
template <class T, class U> __device__ __forceinline__ T idiv(T a, T b) {
    if (b == 0) return (T)-1;
    if ((T)-1 < (T)0 && b == (T)-1) return (T)((U)RT_ZERO - (U)a);
    return a / b;
}
template <class T> __device__ __forceinline__ T irem(T a, T b) {
    if (b == 0) return a;
    if ((T)-1 < (T)0 && b == (T)-1) return 0;
    return a % b;
}
// float -> integer as a cast does: saturating, NaN to 0
template <class T> __device__ __forceinline__ T sat_cast(double x, double lo, double hi, T tlo, T thi) {
    if (x != x) return (T)0;
    if (x <= lo) return tlo;
    if (x >= hi) return thi;
    return (T)x;
}
template <int BYTES> struct VecBytes;
template <> struct VecBytes<16> { typedef uint4 type; };
template <> struct VecBytes<8> { typedef uint2 type; };
template <> struct VecBytes<4> { typedef u32 type; };
template <> struct VecBytes<2> { typedef u16 type; };
template <> struct VecBytes<1> { typedef u8 type; };
// V consecutive elements of T, moved in the widest pieces up to 16 bytes
template <class T, int V> __device__ __forceinline__ void ldv(const T* __restrict__ p, T* dst) {
    constexpr int B = sizeof(T) * V; constexpr int P = B >= 16 ? 16 : B; typedef typename VecBytes<P>::type W;
    #pragma unroll
    for (int k = 0; k < B / P; k++) ((W*)dst)[k] = __ldg((const W*)p + k);
}
template <class T, int V> __device__ __forceinline__ void ldv_plain(const T* p, T* dst) {
    constexpr int B = sizeof(T) * V; constexpr int P = B >= 16 ? 16 : B; typedef typename VecBytes<P>::type W;
    #pragma unroll
    for (int k = 0; k < B / P; k++) ((W*)dst)[k] = ((const W*)p)[k];
}
template <class T, int V> __device__ __forceinline__ void stv(T* p, const T* src) {
    constexpr int B = sizeof(T) * V; constexpr int P = B >= 16 ? 16 : B; typedef typename VecBytes<P>::type W;
    #pragma unroll
    for (int k = 0; k < B / P; k++) ((W*)p)[k] = ((const W*)src)[k];
}
template <class T> __device__ __forceinline__ T shfl_xor_any(T v, int m) {
    if (sizeof(T) == 8) { u64 b; memcpy(&b, &v, 8); b = __shfl_xor_sync(0xffffffffu, b, m); memcpy(&v, &b, 8); return v; }
    u32 b = 0; memcpy(&b, &v, sizeof(T)); b = __shfl_xor_sync(0xffffffffu, b, m); memcpy(&v, &b, sizeof(T)); return v;
}

// ---- two elements per step ("pair mode"): p2<T> holds lanes e and e+1; bfloat16 pairs stay packed in one register and
// use the native packed instructions (one rounding of the exact result per lane, as the reference interpreter rounds) ----
template <class T> struct p2 { T x, y; };
struct bf16x2 { u32 v; };
template <class T> __device__ __forceinline__ T L0(T s) { return s; }
template <class T> __device__ __forceinline__ T L1(T s) { return s; }
template <class T> __device__ __forceinline__ T L0(p2<T> v) { return v.x; }
template <class T> __device__ __forceinline__ T L1(p2<T> v) { return v.y; }
__device__ __forceinline__ float L0(bf16x2 v) { return __uint_as_float(v.v << 16); }
__device__ __forceinline__ float L1(bf16x2 v) { return __uint_as_float(v.v & 0xffff0000u); }
// rounds two floats to bfloat16 (nearest even) with one conversion; lane 0 in the low half
__device__ __forceinline__ bf16x2 mk_bf16x2(float lo, float hi) { bf16x2 r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r.v) : "f"(hi), "f"(lo)); return r; }
// packs two floats that already are bfloat16 values (no rounding)
__device__ __forceinline__ bf16x2 pk_bf16x2(float lo, float hi) { bf16x2 r; r.v = (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u); return r; }
__device__ __forceinline__ bf16x2 to_bf16x2(bf16x2 v) { return v; }
__device__ __forceinline__ bf16x2 to_bf16x2(float s) { bf16x2 r; r.v = (__float_as_uint(s) >> 16) * 0x10001u; return r; }
__device__ __forceinline__ bf16x2 ld_bf16x2(const u16* p) { bf16x2 r; r.v = *(const u32*)p; return r; }
__device__ __forceinline__ bf16x2 bf16x2_add(bf16x2 a, bf16x2 b) { bf16x2 r; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r.v) : "r"(a.v), "r"(b.v)); return r; }
__device__ __forceinline__ bf16x2 bf16x2_sub(bf16x2 a, bf16x2 b) { bf16x2 r; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r.v) : "r"(a.v), "r"(b.v)); return r; }
__device__ __forceinline__ bf16x2 bf16x2_mul(bf16x2 a, bf16x2 b) { bf16x2 r; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r.v) : "r"(a.v), "r"(b.v)); return r; }
__device__ __forceinline__ bf16x2 bf16x2_max(bf16x2 a, bf16x2 b) { bf16x2 r; asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r.v) : "r"(a.v), "r"(b.v)); return r; }
__device__ __forceinline__ bf16x2 bf16x2_min(bf16x2 a, bf16x2 b) { bf16x2 r; asm("min.NaN.bf16x2 %0, %1, %2;" : "=r"(r.v) : "r"(a.v), "r"(b.v)); return r; }
__device__ __forceinline__ bf16x2 bf16x2_neg(bf16x2 a) { bf16x2 r; r.v = a.v ^ 0x80008000u; return r; }
__device__ __forceinline__ bf16x2 bf16x2_abs(bf16x2 a) { bf16x2 r; r.v = a.v & 0x7fff7fffu; return r; }
// float32 pairs: the packed add / mul / fma of sm_100, one rounding per lane exactly as the scalar instructions
__device__ __forceinline__ p2<float> to_f32x2(p2<float> v) { return v; }
__device__ __forceinline__ p2<float> to_f32x2(float s) { p2<float> r = {s, s}; return r; }
__device__ __forceinline__ p2<float> f32x2_add(p2<float> a, p2<float> b) {
    p2<float> r;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ p2<float> f32x2_mul(p2<float> a, p2<float> b) {
    p2<float> r;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
// a - b as fma(b, -1, a): exact product, one rounding of the difference
__device__ __forceinline__ p2<float> f32x2_sub(p2<float> a, p2<float> b) {
    p2<float> r;
    asm("{\n\t.reg .b64 ra, rb, rm, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rm, {%6, %6};\n\tfma.rn.f32x2 rd, rb, rm, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(-1.0f));
    return r;
}
)CUDA";

struct CType {
    const char* compute;  // type values are computed in
    const char* memory;   // type stored in global memory
    const char* unsigned_t;
};

CType ctype(int dtype) {
    switch (dtype) {
        case LB_BOOL: return {"bool", "u8", "u8"};
        case LB_I8: return {"i8", "i8", "u8"};
        case LB_I16: return {"i16", "i16", "u16"};
        case LB_I32: return {"i32", "i32", "u32"};
        case LB_I64: return {"i64", "i64", "u64"};
        case LB_U8: return {"u8", "u8", "u8"};
        case LB_U16: return {"u16", "u16", "u16"};
        case LB_U32: return {"u32", "u32", "u32"};
        case LB_U64: return {"u64", "u64", "u64"};
        case LB_F16: return {"float", "u16", ""};
        case LB_BF16: return {"float", "u16", ""};
        case LB_F32: return {"float", "float", ""};
        case LB_F64: return {"double", "double", ""};
    }
    fail(LB_ERR_INVALID, "bad dtype");
}

const char* rnd_fn(int dtype) {
    switch (dtype) {
        case LB_F16: return "rnd_f16";
        case LB_BF16: return "rnd_bf16";
        case LB_F32: return "rnd_f32";
        case LB_F64: return "rnd_f64";
    }
    return "";
}

// memory value -> compute value
std::string from_memory(int dtype, const std::string& x) {
    switch (dtype) {
        case LB_BOOL: return "(" + x + " != 0)";
        case LB_F16: return "f16_to_f32(" + x + ")";
        case LB_BF16: return "bf16_to_f32(" + x + ")";
        default: return x;
    }
}
std::string to_memory(int dtype, const std::string& x) {
    switch (dtype) {
        case LB_BOOL: return "(u8)(" + x + " ? 1 : 0)";
        case LB_F16: return "f32_to_f16(" + x + ")";
        case LB_BF16: return "(u16)(__float_as_uint(" + x + ") >> 16)";  // values are already rounded to bf16
        default: return x;
    }
}

std::string float_literal(double v, int dtype) {
    if (dtype == LB_F64) {
        uint64_t b;
        memcpy(&b, &v, 8);
        return format("__longlong_as_double(0x%llxLL)", (unsigned long long)b);
    }
    float f = (float)v;
    uint32_t b;
    memcpy(&b, &f, 4);
    return format("__uint_as_float(0x%xu)", b);
}

// round-to-nearest-even f32 -> bf16 / f16 on the host, for constants
double host_round(double x, int dtype) {
    if (dtype == LB_F64) return x;
    // single rounding through a round-to-odd f32 (lumen/tensor/dtype.rs:217-239)
    float f = (float)x;
    if (dtype == LB_F32) return f;
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if (std::isfinite(f) && (double)f != x && !(bits & 1)) {
        bool outward = ((double)f < x) != std::signbit(f);
        bits = outward ? bits + 1 : bits - 1;
        memcpy(&f, &bits, 4);
    }
    if (dtype == LB_BF16) {
        if ((bits & 0x7fffffffu) > 0x7f800000u) return NAN;
        uint32_t r = 0x8000u;
        if ((bits & r) && (bits & (3 * r - 1))) bits += r;
        bits &= 0xffff0000u;
        memcpy(&f, &bits, 4);
        return f;
    }
    // f16
    if (std::isnan(f)) return NAN;
    double a = std::fabs((double)f), r;
    if (a >= 65520.0) r = INFINITY;
    else if (a < 6.103515625e-05) r = std::nearbyint(a * 16777216.0) / 16777216.0;
    else {
        int e;
        std::frexp(a, &e);
        double ulp = std::ldexp(1.0, e - 11);
        r = std::nearbyint(a / ulp) * ulp;
    }
    return std::signbit(f) ? -r : r;
}

struct Comp {
    std::string expr;  // the coordinate, may reference r, c0, e
    std::string base;  // when lane: expr == base + e, base a multiple of VEC not referencing e
    bool lane = false, e_dep = false, row_dep = false, c_dep = false;
    bool dyn = false;  // references a variable defined inside a phase (a gathered index)
    int64_t zero_known = 0;  // 1 when the coordinate is the constant 0
};
typedef std::vector<Comp> Index;

Comp zero_comp() {
    Comp c;
    c.expr = "0";
    c.zero_known = 1;
    return c;
}

struct Phase {
    std::string pre, body, post;
    std::map<std::string, std::string> memo;
    // reduction phases
    bool reduces = false;
    std::string acc, acc_type, init, combine_a_b;  // combine as a format with %A %B
    std::string result;
    bool chunked = true;  // false for the row epilogue (runs once per row, no column loop)
};

std::string subst(std::string s, const std::string& a, const std::string& b) {
    std::string out;
    for (size_t k = 0; k < s.size(); k++) {
        if (s[k] == '%' && k + 1 < s.size() && (s[k + 1] == 'A' || s[k + 1] == 'B')) {
            out += s[k + 1] == 'A' ? a : b;
            k++;
        } else {
            out += s[k];
        }
    }
    return out;
}

class Generator {
  public:
    Generator(const Module& module, const Graph& g) : module_(module), g_(g) {}

    FusedKernel run() {
        plan_space();
        // phases are created on demand while generating the outputs
        Phase main_phase, epilogue;
        epilogue.chunked = false;
        std::vector<std::pair<int, int>> full_outputs, row_outputs;  // (output position, value)
        for (size_t k = 0; k < g_.outputs.size(); k++) {
            const TensorType& t = g_.type(g_.outputs[k]);
            if (t.numel() == R_ * C_ && (C_ != 1 || !has_reduce_)) full_outputs.push_back({(int)k, g_.outputs[k]});
            else if (t.numel() == R_) row_outputs.push_back({(int)k, g_.outputs[k]});
            else
                fail(LB_ERR_UNSUPPORTED, format("fusion output %s does not span the [%lld, %lld] iteration space",
                                                t.str().c_str(), (long long)R_, (long long)C_));
        }
        // Row outputs first: generating them creates the reduction phases.
        for (auto [k, v] : row_outputs) {
            const TensorType& t = g_.type(v);
            Index idx = output_index(t, false);
            std::string val = gen(v, idx, epilogue);
            epilogue.pre += format("if (active && lane_in_row == 0) ((%s*)out%d)[r] = %s;\n", ctype(t.dtype).memory, k,
                                   to_memory(t.dtype, val).c_str());
        }
        // A full output is stored by the first phase that already computes its value (a reduction's prologue),
        // so it is neither recomputed nor re-read; otherwise by a final phase over the row.
        bool main_used = false;
        for (auto [k, v] : full_outputs) {
            const TensorType& t = g_.type(v);
            Index idx = output_index(t, true);
            Phase* home = &main_phase;
            for (Phase& ph : phases_)
                if (ph.chunked && ph.memo.count(key_of(v, idx))) {
                    home = &ph;
                    break;
                }
            main_used |= home == &main_phase;
            std::string val = gen(v, idx, *home);
            CType ct = ctype(t.dtype);
            std::string buf = format("ob%d", k);
            home->pre += format("__align__(16) %s %s[VEC];\n", ct.memory, buf.c_str());
            home->body += store_element(buf, t.dtype, val);
            home->post += format("if (active) stv<%s, VEC>((%s*)out%d + (r * (idx_t)NCOLS + c0), %s);\n", ct.memory,
                                 ct.memory, k, buf.c_str());
        }
        if (main_used) phases_.push_back(main_phase);
        if (!row_outputs.empty()) phases_.push_back(epilogue);
        return emit();
    }

  private:
    const Module& module_;
    const Graph& g_;
    int64_t R_ = 1, C_ = 1;
    int VEC_ = 1, T_ = 1, RPB_ = 1, NCH_ = 1;
    bool has_reduce_ = false;
    bool wide_index_ = false;
    int counter_ = 0;
    std::vector<Phase> phases_;
    std::map<std::string, std::string> reduce_memo_;
    std::string row_decls_;     // row-scope declarations (reduction results)
    std::string kernel_cache_;  // CTA-scope cached column loads
    std::string row_cache_;     // row-scope cached loads
    struct RowCache { std::string type, buf, load; int bytes; };
    std::vector<RowCache> row_caches_;  // the same loads one by one, for prefetching the next row block
    std::map<std::string, std::string> cached_loads_;
    int cached_regs_ = 0;

    std::string fresh(const char* prefix) { return format("%s%d", prefix, counter_++); }

    // ---- iteration space ----------------------------------------------------------------------------------
    void plan_space() {
        const TensorType* space = nullptr;
        for (const Node& n : g_.nodes) {
            if (n.op != "reduce_sum" && n.op != "reduce_max") continue;
            const TensorType& x = g_.type(n.inputs[0]);
            auto axes = n.ints("axes");
            std::sort(axes.begin(), axes.end());
            for (size_t k = 0; k < axes.size(); k++)
                if (axes[k] != (int64_t)(x.rank() - axes.size() + k))
                    fail(LB_ERR_UNSUPPORTED,
                         format("%s over axes other than the trailing ones of %s has no fused row kernel", n.op.c_str(),
                                x.str().c_str()));
            int64_t c = 1;
            for (auto a : axes) c *= x.shape[a];
            int64_t r = x.numel() / std::max<int64_t>(c, 1);
            if (has_reduce_ && (c != C_ || r != R_))
                fail(LB_ERR_UNSUPPORTED, "reductions over different row shapes in one fusion");
            has_reduce_ = true;
            C_ = c;
            R_ = c ? r : 0;
            space = &x;
        }
        if (!has_reduce_) {
            for (int v : g_.outputs)
                if (!space || g_.type(v).numel() > space->numel()) space = &g_.type(v);
            if (!space) fail(LB_ERR_INVALID, "fusion without outputs");
            // A pure elementwise space is flat: the row is the last dimension, widened by a divisor of the
            // leading dimensions until it is long enough to keep a thread group busy.
            C_ = space->rank() ? space->shape.back() : 1;
            // (the horizontal form keeps the last dimension as its row: every group's size is a multiple of it)
            const int64_t longest = 64LL * 1024 * 4;  // what one block takes as a row (64 chunks of 1024 threads x 4 elements)
            for (int d = space->rank() - 2; !multi_ && d >= 0 && C_ > 0 && C_ < 1024; d--) {
                int64_t n = space->shape[d], k = 1;
                while (k < n && (n % k != 0 || C_ * k < 1024)) k++;
                if (C_ * k > longest) {  // no divisor of this dimension gives a row of a good length: the largest that fits
                    for (k = std::min<int64_t>(n, 16384 / C_); k > 1 && n % k != 0;) k--;
                    C_ *= std::max<int64_t>(k, 1);
                    break;
                }
                C_ *= k;
                if (k < n) break;
            }
            if (!multi_ && C_ > longest) {  // a last dimension longer than a block's row: rows are a divisor of it
                int64_t c = 16384;
                while (c > 1 && C_ % c != 0) c--;
                C_ = c;
            }
            R_ = C_ ? space->numel() / C_ : 0;
        }
        // vector width: 16 bytes of the narrowest tensor spanning the space, dividing C
        int min_size = 8;
        auto consider = [&](const TensorType& t) {
            if (t.numel() == R_ * C_ || t.numel() == C_) min_size = std::min(min_size, dtype_size(t.dtype));
        };
        for (int v : g_.inputs) consider(g_.type(v));
        for (int v : g_.outputs) consider(g_.type(v));
        VEC_ = std::min(8, 16 / min_size);
        while (VEC_ > 1 && C_ % VEC_ != 0) VEC_ /= 2;
        int64_t nvec = std::max<int64_t>((C_ + VEC_ - 1) / VEC_, 1);
        int64_t want = (nvec + 3) / 4;
        T_ = 1;
        while (T_ < want && T_ < 1024) T_ *= 2;
        RPB_ = T_ >= 32 ? 1 : 256 / T_;
        if (T_ > 32) RPB_ = 1;
        else RPB_ = std::max(1, 256 / T_);
        NCH_ = (int)((nvec + T_ - 1) / T_);
        if (NCH_ > 64) fail(LB_ERR_UNSUPPORTED, format("rows of %lld elements are too long for the fused row kernel", (long long)C_));
        wide_index_ = R_ * C_ >= (1LL << 31) - 4096;
        for (int v : g_.inputs)
            if (g_.type(v).numel() >= (1LL << 31) - 4096) wide_index_ = true;
        if (multi_) wide_index_ = true;  // a group's row count is a run-time value
        pair_ = VEC_ >= 2 && computes_bf16();
    }

    // pair mode pays where packed bfloat16 instructions replace scalar ones
    bool computes_bf16() const {
        for (const Node& n : g_.nodes)
            if (g_.type(n.output).dtype == LB_BF16) return true;
        for (int v : g_.inputs)
            if (g_.type(v).dtype == LB_BF16) return true;
        return false;
    }

    Comp row_comp() {
        Comp c;
        c.expr = "r";
        c.row_dep = true;
        return c;
    }
    Comp col_comp() {
        Comp c;
        c.expr = "(c0 + e)";
        c.base = "c0";
        c.lane = c.e_dep = c.c_dep = true;
        return c;
    }

    // Drops redundant outer parentheses, "((r))" -> "r", so that the same coordinate reached through different
    // reshapes gets the same text: values and reductions are memoised by the text of their index.
    static std::string tidy(std::string s) {
        for (;;) {
            if (s.size() < 2 || s.front() != '(' || s.back() != ')') return s;
            int depth = 0;
            bool wraps = true;
            for (size_t k = 0; k + 1 < s.size(); k++) {
                if (s[k] == '(') depth++;
                if (s[k] == ')' && --depth == 0) wraps = false;
            }
            if (!wraps) return s;
            std::string inner = s.substr(1, s.size() - 2);
            bool simple = !inner.empty();
            for (char c : inner) simple &= ident_char(c);
            bool wrapped_again = inner.size() >= 2 && inner.front() == '(' && inner.back() == ')';
            if (wrapped_again) {
                int d = 0;
                for (size_t k = 0; k + 1 < inner.size(); k++) {
                    if (inner[k] == '(') d++;
                    if (inner[k] == ')' && --d == 0) wrapped_again = false;
                }
            }
            if (!simple && !wrapped_again) return s;
            s = inner;
        }
    }

    // coordinates of flat index `flat` in `shape`
    Index unravel(const Comp& flat, const std::vector<int64_t>& shape) {
        Index out(shape.size());
        int rank = (int)shape.size();
        bool keep_lane = flat.lane && rank > 0 && shape[rank - 1] % VEC_ == 0;
        int64_t stride = 1;
        for (int d = rank - 1; d >= 0; d--) {
            Comp c;
            c.row_dep = flat.row_dep;
            c.dyn = flat.dyn;
            c.c_dep = flat.c_dep;
            if (shape[d] == 1) {
                c = zero_comp();
            } else {
                const std::string src = tidy(keep_lane ? flat.base : flat.expr);
                std::string q = stride == 1 ? src : format("(%s / %lld)", src.c_str(), (long long)stride);
                // the leading coordinate needs no modulo: the flat index is in range
                std::string coord = d == 0 ? q : format("(%s %% %lld)", q.c_str(), (long long)shape[d]);
                if (keep_lane && d == rank - 1) {
                    c.base = coord;
                    c.expr = format("(%s + e)", coord.c_str());
                    c.lane = c.e_dep = true;
                } else {
                    c.expr = coord;
                    c.e_dep = keep_lane ? false : flat.e_dep;
                }
            }
            out[d] = c;
            stride *= shape[d];
        }
        return out;
    }

    Comp ravel(const Index& idx, const std::vector<int64_t>& shape) {
        Comp out;
        int rank = (int)shape.size();
        if (rank == 0) return zero_comp();
        bool lane = idx[rank - 1].lane && (rank == 1 || shape[rank - 1] % VEC_ == 0);
        for (int d = 0; d < rank - 1; d++)
            if (idx[d].e_dep) lane = false;
        std::string sum;
        int64_t stride = numel(shape);
        for (int d = 0; d < rank; d++) {
            stride /= std::max<int64_t>(shape[d], 1);
            const Comp& c = idx[d];
            out.row_dep |= c.row_dep;
            out.dyn |= c.dyn;
            out.c_dep |= c.c_dep;
            out.e_dep |= c.e_dep;
            if (c.zero_known || shape[d] == 1) continue;
            std::string term = (lane && d == rank - 1) ? c.base : c.expr;
            if (stride != 1) term = format("(idx_t)%s * %lld", term.c_str(), (long long)stride);
            sum += (sum.empty() ? "" : " + ") + term;
        }
        if (sum.empty()) sum = "0";
        if (lane) {
            out.lane = true;
            out.base = tidy("(" + sum + ")");
            out.expr = "(" + sum + " + e)";
        } else {
            out.expr = tidy("(" + sum + ")");
        }
        if (out.expr == "0") return zero_comp();
        return out;
    }

    Index output_index(const TensorType& t, bool full) {
        if (!full) return unravel(row_comp(), t.shape);
        if (t.rank() >= 1 && t.shape.back() == C_) {
            std::vector<int64_t> lead(t.shape.begin(), t.shape.end() - 1);
            Index idx = unravel(row_comp(), lead);
            idx.push_back(col_comp());
            return idx;
        }
        Comp flat;
        flat.base = format("(r * (idx_t)%lld + c0)", (long long)C_);
        flat.expr = format("(r * (idx_t)%lld + c0 + e)", (long long)C_);
        flat.lane = flat.e_dep = flat.c_dep = flat.row_dep = true;
        return unravel(flat, t.shape);
    }

    static std::string key_of(int v, const Index& idx) {
        std::string k = std::to_string(v);
        for (const Comp& c : idx) k += "|" + c.expr;
        return k;
    }
    static bool e_dep(const Index& idx) {
        for (const Comp& c : idx)
            if (c.e_dep) return true;
        return false;
    }
    static bool c_dep(const Index& idx) {
        for (const Comp& c : idx)
            if (c.c_dep) return true;
        return false;
    }

    // ---- pair mode -----------------------------------------------------------------------------------------
    // The element loop advances two elements per step. A value that depends on the element is a pair variable
    // (p2<T>, or packed bf16x2); its defining expression is written once with operand placeholders @k@ and
    // instantiated for lane 0 and lane 1. Values that do not depend on the element stay scalars.
    bool pair_ = false;
    std::map<std::string, int> pair_vars_;  // pair variable -> dtype (-1 for index variables)

    static bool ident_char(char c) { return std::isalnum((unsigned char)c) || c == '_'; }
    static bool mentions_e(const std::string& s) {
        for (size_t k = 0; k < s.size(); k++)
            if (s[k] == 'e' && (k == 0 || !ident_char(s[k - 1])) && (k + 1 == s.size() || !ident_char(s[k + 1]))) return true;
        return false;
    }
    // `expr` for lane 0 or 1: placeholders become L<lane>(operand), LX( becomes L<lane>(, the element index e
    // becomes (e + 1) in lane 1
    static std::string lane_of(const std::string& expr, int lane, const std::vector<std::string>* ops) {
        std::string a;
        const char* acc = lane ? "L1(" : "L0(";
        for (size_t k = 0; k < expr.size(); k++) {
            if (expr[k] == '@') {
                size_t end = expr.find('@', k + 1);
                int which = std::stoi(expr.substr(k + 1, end - k - 1));
                a += acc + (*ops)[which] + ")";
                k = end;
            } else if (expr.compare(k, 3, "LX(") == 0 && (k == 0 || !ident_char(expr[k - 1]))) {
                a += acc;
                k += 2;
            } else {
                a += expr[k];
            }
        }
        if (!lane) return a;
        std::string out;
        for (size_t k = 0; k < a.size(); k++) {
            if (a[k] == 'e' && (k == 0 || !ident_char(a[k - 1])) && (k + 1 == a.size() || !ident_char(a[k + 1]))) out += "(e + 1)";
            else out += a[k];
        }
        return out;
    }
    // a statement per lane (accumulations, stores)
    static std::string both_lanes(const std::string& stmt) { return lane_of(stmt, 0, nullptr) + lane_of(stmt, 1, nullptr); }
    static std::string whole_of(const std::string& expr, const std::vector<std::string>* ops) {
        std::string a;
        for (size_t k = 0; k < expr.size(); k++) {
            if (expr[k] == '@') {
                size_t end = expr.find('@', k + 1);
                a += (*ops)[std::stoi(expr.substr(k + 1, end - k - 1))];
                k = end;
            } else {
                a += expr[k];
            }
        }
        return a;
    }
    // an operand usable by a packed bf16x2 instruction: a packed pair, or a scalar that is the same for both lanes
    bool packable(const std::string& operand, int dtype = LB_BF16) const {
        auto it = pair_vars_.find(operand);
        if (it != pair_vars_.end()) return it->second == dtype;
        return !mentions_e(operand) && operand.find("LX(") == std::string::npos;
    }
    bool pairs_here(const Phase& ph, bool in_body) const { return pair_ && in_body && ph.chunked; }

    // Defines a variable holding `expr` in the right scope of `ph` and returns its name. In pair mode `ops` are the
    // operands behind the placeholders; `whole` marks an expression that already yields a packed bf16x2.
    std::string define(Phase& ph, const char* type, const std::string& expr, bool in_body,
                       const std::vector<std::string>* ops = nullptr, int dtype = -1, bool whole = false) {
        std::string name = fresh("v");
        if (!pairs_here(ph, in_body)) {
            std::string line = format("%s %s = %s;\n", type, name.c_str(), expr.c_str());
            (in_body && ph.chunked ? ph.body : ph.pre) += line;
            return name;
        }
        if (whole) {
            ph.body += format("%s %s = %s;\n", dtype == LB_BF16 ? "bf16x2" : "p2<float>", name.c_str(), whole_of(expr, ops).c_str());
        } else if (dtype == LB_BF16) {
            // one packed conversion rounds both lanes; values that already are bf16 are packed by their bits
            static const std::string rnd = "rnd_bf16(";
            bool rounds = expr.compare(0, rnd.size(), rnd) == 0 && expr.back() == ')';
            if (rounds) {
                int depth = 0;
                for (size_t k = rnd.size() - 1; k < expr.size(); k++) {
                    if (expr[k] == '(') depth++;
                    if (expr[k] == ')' && --depth == 0 && k + 1 != expr.size()) rounds = false;
                }
            }
            std::string inner = rounds ? expr.substr(rnd.size(), expr.size() - rnd.size() - 1) : expr;
            ph.body += format("bf16x2 %s = %s(%s, %s);\n", name.c_str(), rounds ? "mk_bf16x2" : "pk_bf16x2",
                              lane_of(inner, 0, ops).c_str(), lane_of(inner, 1, ops).c_str());
        } else {
            ph.body += format("p2<%s> %s = {%s, %s};\n", type, name.c_str(), lane_of(expr, 0, ops).c_str(), lane_of(expr, 1, ops).c_str());
        }
        pair_vars_[name] = dtype;
        return name;
    }

    // the statement(s) placing element e (and e + 1 in pair mode) of `val` in the staging array `buf`
    std::string store_element(const std::string& buf, int dtype, const std::string& val) {
        if (!pair_) return format("%s[e] = %s;\n", buf.c_str(), to_memory(dtype, val).c_str());
        auto it = pair_vars_.find(val);
        if (it != pair_vars_.end() && it->second == LB_BF16 && dtype == LB_BF16) return format("*(u32*)&%s[e] = %s.v;\n", buf.c_str(), val.c_str());
        return both_lanes(format("%s[e] = %s;\n", buf.c_str(), to_memory(dtype, "LX(" + val + ")").c_str()));
    }
    // the statement(s) folding element e (and e + 1) of `val` into `acc`
    std::string accumulate(const std::string& acc, const std::string& combine, const std::string& val) {
        if (!pair_) return format("%s = %s;\n", acc.c_str(), subst(combine, acc, val).c_str());
        return both_lanes(format("%s = %s;\n", acc.c_str(), subst(combine, acc, "LX(" + val + ")").c_str()));
    }

    // ---- loads ------------------------------------------------------------------------------------------
    std::string vector_element_;  // set by load_input: the staged array element (memory type) when the load is vectorised
    std::string load_input(int position, int v, const Index& idx, Phase& ph) {
        vector_element_.clear();
        const TensorType& t = g_.type(v);
        CType ct = ctype(t.dtype);
        Comp flat = ravel(idx, t.shape);
        std::string ptr = format("((const %s*)in%d)", ct.memory, position);
        if (flat.lane && ph.chunked) {
            // contiguous along the vector lane: one vector load per chunk
            bool column_only = !flat.row_dep && !flat.dyn && !column_mode_;  // same for every row: cache once per CTA
            bool cache_row = !column_only && !flat.dyn && !column_mode_ && multi_phase_hint_ && cached_regs_ + NCH_ * VEC_ <= 96;
            std::string key = format("in%d|%s", position, flat.base.c_str());
            if (column_only && cached_regs_ + NCH_ * VEC_ <= 128) {
                auto it = cached_loads_.find(key);
                if (it == cached_loads_.end()) {
                    std::string buf = fresh("col");
                    kernel_cache_ += format("__align__(16) %s %s[NCH][VEC];\n", ct.memory, buf.c_str());
                    kernel_cache_ += format("CHUNK_LOOP_BEGIN %s<%s, VEC>(%s + %s, %s[ch]); CHUNK_LOOP_END\n", inplace_ ? "ldv_plain" : "ldv", ct.memory,
                                            ptr.c_str(), flat.base.c_str(), buf.c_str());
                    cached_regs_ += NCH_ * VEC_ * std::max(1, dtype_size(t.dtype) / 4);
                    it = cached_loads_.emplace(key, buf).first;
                }
                vector_element_ = format("%s[ch][e]", it->second.c_str());
                return from_memory(t.dtype, vector_element_);
            }
            if (cache_row) {
                auto it = cached_loads_.find(key);
                if (it == cached_loads_.end()) {
                    std::string buf = fresh("row");
                    row_cache_ += format("__align__(16) %s %s[NCH][VEC];\n", ct.memory, buf.c_str());
                    row_cache_ += format("CHUNK_LOOP_BEGIN %s<%s, VEC>(%s + %s, %s[ch]); CHUNK_LOOP_END\n", inplace_ ? "ldv_plain" : "ldv", ct.memory,
                                         ptr.c_str(), flat.base.c_str(), buf.c_str());
                    row_caches_.push_back({ct.memory, buf,
                                           format("CHUNK_LOOP_BEGIN %s<%s, VEC>(%s + %s, %s_nx[ch]); CHUNK_LOOP_END\n", inplace_ ? "ldv_plain" : "ldv",
                                                  ct.memory, ptr.c_str(), flat.base.c_str(), buf.c_str()),
                                           NCH_ * VEC_ * dtype_size(t.dtype)});
                    cached_regs_ += NCH_ * VEC_ * std::max(1, dtype_size(t.dtype) / 4);
                    it = cached_loads_.emplace(key, buf).first;
                }
                vector_element_ = format("%s[ch][e]", it->second.c_str());
                return from_memory(t.dtype, vector_element_);
            }
            std::string pkey = "ld|" + key;
            auto it = ph.memo.find(pkey);
            if (it == ph.memo.end()) {
                std::string buf = fresh("ld");
                ph.pre += format("__align__(16) %s %s[VEC]; %s<%s, VEC>(%s + %s, %s);\n", ct.memory, buf.c_str(),
                                 inplace_ ? "ldv_plain" : "ldv", ct.memory, ptr.c_str(), flat.base.c_str(), buf.c_str());
                it = ph.memo.emplace(pkey, buf).first;
            }
            vector_element_ = format("%s[e]", it->second.c_str());
            return from_memory(t.dtype, vector_element_);
        }
        return from_memory(t.dtype, format(inplace_ ? "(*(%s + %s))" : "__ldg(%s + %s)", ptr.c_str(), flat.expr.c_str()));
    }

    bool multi_phase_hint_ = false;
    bool column_mode_ = false;   // reductions over the leading axes: partial sums per row slice, then a finalize pass
    bool inplace_ = false;       // an output aliases an input: plain loads, no __restrict__
    bool multi_ = false;         // one launch serves a table of tensor groups: pointers and row count per group
    std::vector<int> col_reduces_;  // values reduced over the leading axes, in node order
    int lead_rank_ = 0;

    // ---- values -----------------------------------------------------------------------------------------
    std::string gen(int v, const Index& idx, Phase& ph) {
        std::string key = key_of(v, idx);
        auto it = ph.memo.find(key);
        if (it != ph.memo.end()) return it->second;
        std::string name = gen_uncached(v, idx, ph);
        ph.memo[key] = name;
        return name;
    }

    // exp(a - m) with m a row maximum computed in this kernel (through reshapes / broadcasts), read by reduce_sum only
    bool normaliser_term(const Node& n) const {
        if (n.op != "exp" || g_.type(n.output).dtype != LB_F32) return false;
        const Node* sub = g_.node_of(n.inputs[0]);
        if (!sub || sub->op != "sub") return false;
        const Node* m = g_.node_of(sub->inputs[1]);
        while (m && (m->op == "broadcast_in_dim" || m->op == "reshape")) m = g_.node_of(m->inputs[0]);
        if (!m || m->op != "reduce_max") return false;
        // the maximum is taken over the values the difference is formed from (possibly widened first)
        int a = sub->inputs[0], x = m->inputs[0];
        if (a != x) return false;
        bool summed = false;
        for (const Node& u : g_.nodes)
            for (int in : u.inputs)
                if (in == n.output) {
                    if (u.op != "reduce_sum") return false;
                    summed = true;
                }
        for (int out : g_.outputs)
            if (out == n.output) return false;
        return summed;
    }

    std::string gen_uncached(int v, const Index& idx, Phase& ph) {
        const TensorType& t = g_.type(v);
        if ((int)idx.size() != t.rank()) fail(LB_ERR_INVALID, "internal: index rank mismatch");
        CType ct = ctype(t.dtype);
        const Node* n = g_.node_of(v);
        bool in_body = e_dep(idx);
        const bool pairs = pairs_here(ph, in_body);
        if (!n) {
            int position = (int)(std::find(g_.inputs.begin(), g_.inputs.end(), v) - g_.inputs.begin());
            std::string loaded = load_input(position, v, idx, ph);
            if (pairs && t.dtype == LB_BF16 && !vector_element_.empty())
                return define(ph, ct.compute, "ld_bf16x2(&" + vector_element_ + ")", in_body, nullptr, t.dtype, true);
            return define(ph, ct.compute, loaded, in_body, nullptr, t.dtype);
        }
        const std::string& op = n->op;
        // In pair mode operands are referred to by placeholders and instantiated per lane by define().
        std::vector<std::string> ops;
        auto operand = [&](const std::string& name) {
            if (!pairs) return name;
            ops.push_back(name);
            return format("@%d@", (int)ops.size() - 1);
        };
        auto arg = [&](int k) { return operand(gen(n->inputs[k], idx, ph)); };
        auto def = [&](const char* type, const std::string& e, bool body, bool whole = false) {
            return define(ph, type, e, body, &ops, (int)t.dtype, whole);
        };
        const bool packed = pairs && t.dtype == LB_BF16;
        bool flt = dtype_is_float(t.dtype);
        const char* rnd = rnd_fn(t.dtype);
        bool f64 = t.dtype == LB_F64;

        if (op == "add" || op == "sub" || op == "mul" || op == "div" || op == "max" || op == "min" || op == "rem" ||
            op == "pow") {
            std::string a = arg(0), b = arg(1), e;
            if (packed && (op == "add" || op == "sub" || op == "mul" || op == "max" || op == "min") && packable(ops[0]) && packable(ops[1]))
                return def(ct.compute, format("bf16x2_%s(to_bf16x2(%s), to_bf16x2(%s))", op.c_str(), a.c_str(), b.c_str()), in_body, true);
            if (pairs && t.dtype == LB_F32 && (op == "add" || op == "sub" || op == "mul") && packable(ops[0], LB_F32) && packable(ops[1], LB_F32))
                return def(ct.compute, format("f32x2_%s(to_f32x2(%s), to_f32x2(%s))", op.c_str(), a.c_str(), b.c_str()), in_body, true);
            if (flt) {
                if (op == "add") e = f64 ? a + " + " + b : "__fadd_rn(" + a + ", " + b + ")";
                else if (op == "sub") e = f64 ? a + " - " + b : "__fsub_rn(" + a + ", " + b + ")";
                else if (op == "mul") e = f64 ? a + " * " + b : "__fmul_rn(" + a + ", " + b + ")";
                else if (op == "div") e = f64 ? a + " / " + b : "__fdiv_rn(" + a + ", " + b + ")";
                else if (op == "max") e = "fmax_nan(" + a + ", " + b + ")";
                else if (op == "min") e = "fmin_nan(" + a + ", " + b + ")";
                else if (op == "rem") e = f64 ? "fmod(" + a + ", " + b + ")" : "fmodf(" + a + ", " + b + ")";
                else e = f64 ? "pow(" + a + ", " + b + ")" : "powf(" + a + ", " + b + ")";
                if (op != "max" && op != "min") e = std::string(rnd) + "(" + e + ")";
            } else {
                std::string T = ct.compute, U = ct.unsigned_t;
                // a constant 0 - x or x * -1 is a negation to the compiler: written RT_ZERO - x like `neg` (see RT_ZERO)
                const std::string zero = "((" + T + ")0LL)", minus_one = "((" + T + ")-1LL)";
                if (op == "add") e = "(" + T + ")((" + U + ")" + a + " + (" + U + ")" + b + ")";
                else if (op == "sub") e = "(" + T + ")((" + U + ")" + (a == zero ? std::string("RT_ZERO") : a) + " - (" + U + ")" + b + ")";
                else if (op == "mul" && (a == minus_one || b == minus_one)) e = "(" + T + ")((" + U + ")RT_ZERO - (" + U + ")" + (a == minus_one ? b : a) + ")";
                else if (op == "mul") e = "(" + T + ")((" + U + ")" + a + " * (" + U + ")" + b + ")";
                else if (op == "div") e = "idiv<" + T + ", " + U + ">(" + a + ", " + b + ")";
                else if (op == "rem") e = "irem<" + T + ">(" + a + ", " + b + ")";
                else if (op == "max") e = "imax<" + T + ">(" + a + ", " + b + ")";
                else if (op == "min") e = "imin<" + T + ">(" + a + ", " + b + ")";
                else fail(LB_ERR_UNSUPPORTED, op + " of integers");
            }
            return def(ct.compute, e, in_body);
        }
        if (op == "and" || op == "or" || op == "xor") {
            const char* sym = op == "and" ? "&" : op == "or" ? "|" : "^";
            std::string e = t.dtype == LB_BOOL ? format("(%s %s %s)", arg(0).c_str(), op == "and" ? "&&" : op == "or" ? "||" : "!=", arg(1).c_str())
                                               : format("(%s)(%s %s %s)", ct.compute, arg(0).c_str(), sym, arg(1).c_str());
            return def(ct.compute, e, in_body);
        }
        if (op == "eq" || op == "lt") {
            return def("bool", format("(%s %s %s)", arg(0).c_str(), op == "eq" ? "==" : "<", arg(1).c_str()), in_body);
        }
        if (op == "neg") {
            std::string a = arg(0);
            if (packed && packable(ops[0])) return def(ct.compute, "bf16x2_neg(to_bf16x2(" + a + "))", in_body, true);
            return def(ct.compute, flt ? "-" + a : format("(%s)((%s)RT_ZERO - (%s)%s)", ct.compute, ct.unsigned_t, ct.unsigned_t, a.c_str()), in_body);
        }
        if (op == "abs" || op == "sign" || op == "not") {
            std::string a = arg(0), e;
            if (packed && op == "abs" && packable(ops[0])) return def(ct.compute, "bf16x2_abs(to_bf16x2(" + a + "))", in_body, true);
            if (op == "abs") e = flt ? (f64 ? "fabs(" + a + ")" : "fabsf(" + a + ")") : format("(%s)(%s < 0 ? (%s)RT_ZERO - (%s)%s : (%s)%s)", ct.compute, a.c_str(), ct.unsigned_t, ct.unsigned_t, a.c_str(), ct.unsigned_t, a.c_str());
            else if (op == "sign") e = flt ? format("((%s == 0 || %s != %s) ? %s : (%s < 0 ? (%s)-1 : (%s)1))", a.c_str(), a.c_str(), a.c_str(), a.c_str(), a.c_str(), ct.compute, ct.compute) : format("(%s)((%s > 0) - (%s < 0))", ct.compute, a.c_str(), a.c_str());
            else e = t.dtype == LB_BOOL ? "!" + a : format("(%s)~%s", ct.compute, a.c_str());
            return def(ct.compute, e, in_body);
        }
        if (op == "exp" || op == "log" || op == "sqrt" || op == "tanh" || op == "logistic" || op == "rsqrt" ||
            op == "floor" || op == "ceil" || op == "exp2" || op == "log2" || op == "sin" || op == "cos") {
            std::string a = arg(0), e;
            if (f64) {
                if (op == "logistic") e = "1.0 / (1.0 + exp(-" + a + "))";
                else if (op == "rsqrt") e = "1.0 / sqrt(" + a + ")";
                else e = op + "(" + a + ")";
            } else {
                if (op == "logistic") e = "__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-" + a + ")))";
                else if (op == "rsqrt") e = "__fdiv_rn(1.0f, __fsqrt_rn(" + a + "))";
                else if (op == "sqrt") e = "__fsqrt_rn(" + a + ")";
                else if (normaliser_term(*n)) e = "exp_sum_term(" + a + ")";
                else e = op + "f(" + a + ")";
            }
            return def(ct.compute, std::string(rnd) + "(" + e + ")", in_body);
        }
        if (op == "is_finite") {
            const TensorType& x = g_.type(n->inputs[0]);
            std::string a = arg(0);
            return def("bool", dtype_is_float(x.dtype) ? "isfinite(" + a + ")" : "true", in_body);
        }
        if (op == "cast") {
            const TensorType& x = g_.type(n->inputs[0]);
            std::string a = arg(0), e;
            bool from_float = dtype_is_float(x.dtype);
            if (flt) {
                if (x.dtype == LB_BOOL) e = format("(%s ? (%s)1 : (%s)0)", a.c_str(), ct.compute, ct.compute);
                else e = format("%s((%s)%s)", rnd, ct.compute, a.c_str());
            } else if (t.dtype == LB_BOOL) {
                e = "(" + a + " != 0)";
            } else if (from_float) {
                static const char* lo[] = {"", "-128.0", "-32768.0", "-2147483648.0", "-9223372036854775808.0", "0.0", "0.0", "0.0", "0.0"};
                static const char* hi[] = {"", "127.0", "32767.0", "2147483647.0", "9223372036854775807.0", "255.0", "65535.0", "4294967295.0", "18446744073709551615.0"};
                static const char* tlo[] = {"", "-128", "-32768", "(-2147483647 - 1)", "(-9223372036854775807LL - 1)", "0", "0", "0u", "0ull"};
                static const char* thi[] = {"", "127", "32767", "2147483647", "9223372036854775807LL", "255", "65535", "4294967295u", "18446744073709551615ull"};
                e = format("sat_cast<%s>((double)%s, %s, %s, (%s)%s, (%s)%s)", ct.compute, a.c_str(), lo[t.dtype], hi[t.dtype], ct.compute, tlo[t.dtype], ct.compute, thi[t.dtype]);
            } else {
                e = format("(%s)%s", ct.compute, a.c_str());
            }
            return def(ct.compute, e, in_body);
        }
        if (op == "select") {
            return def(ct.compute, format("(%s ? %s : %s)", arg(0).c_str(), arg(1).c_str(), arg(2).c_str()), in_body);
        }
        if (op == "full") {
            const std::string& val = n->attr("fill_value");
            double x = val[0] == 'f' ? std::strtod(val.c_str() + 2, nullptr) : (double)std::stoll(val.substr(2));
            if (flt) return float_literal(host_round(x, t.dtype), t.dtype);
            if (t.dtype == LB_BOOL) return x != 0 ? "true" : "false";
            if (val[0] == 'f') fail(LB_ERR_UNSUPPORTED, "full: float fill value of an integer tensor");
            long long i = std::stoll(val.substr(2));
            return format("((%s)%lld%s)", ct.compute, i == INT64_MIN ? i + 1 : i, i == INT64_MIN ? "LL - 1" : "LL");
        }
        if (op == "iota") {
            const Comp& c = idx[n->integer("dimension")];
            std::string e = flt ? format("%s((%s)%s)", rnd, ct.compute, c.expr.c_str()) : format("(%s)%s", ct.compute, c.expr.c_str());
            return def(ct.compute, e, c.e_dep);
        }
        if (op == "broadcast_in_dim") {
            const TensorType& x = g_.type(n->inputs[0]);
            auto dims = n->ints("broadcast_dimensions");
            Index src(x.rank());
            for (int k = 0; k < x.rank(); k++) src[k] = x.shape[k] == 1 ? zero_comp() : idx[dims[k]];
            return gen(n->inputs[0], src, ph);
        }
        if (op == "transpose") {
            auto perm = n->ints("permutation");
            Index src(idx.size());
            for (size_t k = 0; k < perm.size(); k++) src[perm[k]] = idx[k];
            return gen(n->inputs[0], src, ph);
        }
        if (op == "reshape" || op == "device_wait" || op == "host_wait") {
            const TensorType& x = g_.type(n->inputs[0]);
            if (op != "reshape") return gen(n->inputs[0], idx, ph);
            // equal trailing dimensions pass through; the rest goes through the flat index
            int same = 0;
            while (same < x.rank() && same < t.rank() && x.shape[x.rank() - 1 - same] == t.shape[t.rank() - 1 - same]) same++;
            std::vector<int64_t> out_lead(t.shape.begin(), t.shape.end() - same), in_lead(x.shape.begin(), x.shape.end() - same);
            Index lead(idx.begin(), idx.end() - same);
            Index src = unravel(ravel(lead, out_lead), in_lead);
            src.insert(src.end(), idx.end() - same, idx.end());
            return gen(n->inputs[0], src, ph);
        }
        if (op == "slice") {
            auto start = n->ints("start_indices");
            Index src = idx;
            for (size_t k = 0; k < src.size(); k++) {
                if (start[k] == 0) continue;
                Comp& c = src[k];
                bool aligned = c.lane && start[k] % VEC_ == 0;
                if (c.lane && aligned) c.base = format("(%s + %lld)", c.base.c_str(), (long long)start[k]);
                else c.lane = false;
                c.expr = format("(%s + %lld)", c.expr.c_str(), (long long)start[k]);
                c.zero_known = 0;
            }
            return gen(n->inputs[0], src, ph);
        }
        if (op == "gather") {
            // out[..axis, i.., ..] = x[..axis, clamp(indices[i..]), ..]  (lumen/reference/mod.rs:731-749)
            const TensorType& x = g_.type(n->inputs[0]);
            const TensorType& ind = g_.type(n->inputs[1]);
            int axis = (int)n->integer("axis");
            Index sub(idx.begin() + axis, idx.begin() + axis + ind.rank());
            Comp picked;
            picked.e_dep = e_dep(sub);
            const bool pair_index = pairs_here(ph, picked.e_dep);
            std::string k = gen(n->inputs[1], sub, ph);
            if (pair_index) {
                ops.assign(1, k);
                k = "@0@";
            }
            picked.c_dep = c_dep(sub);
            picked.row_dep = true;
            picked.dyn = true;
            picked.expr = define(ph, "idx_t",
                                 format("(idx_t)imin<i64>(imax<i64>((i64)%s, 0), %lldLL)", k.c_str(),
                                        (long long)std::max<int64_t>(x.shape[axis] - 1, 0)),
                                 picked.e_dep, &ops, -1);
            if (pair_index) picked.expr = "LX(" + picked.expr + ")";
            Index src(idx.begin(), idx.begin() + axis);
            src.push_back(picked);
            src.insert(src.end(), idx.begin() + axis + ind.rank(), idx.end());
            return gen(n->inputs[0], src, ph);
        }
        if (op == "reduce_sum" || op == "reduce_max") return gen_reduce(*n, idx);
        fail(LB_ERR_UNSUPPORTED, "the fused kernel generator has no rule for primitive " + op);
    }

    std::string gen_reduce(const Node& n, const Index& idx) {
        if (column_mode_) {
            auto it = std::find(col_reduces_.begin(), col_reduces_.end(), n.output);
            if (it == col_reduces_.end()) fail(LB_ERR_UNSUPPORTED, n.op + ": mixed row and column reductions in one fusion");
            return format("tot%d[e]", (int)(it - col_reduces_.begin()));
        }
        if (e_dep(idx) || c_dep(idx))
            fail(LB_ERR_UNSUPPORTED, n.op + ": a row reduction read at a column-dependent index");
        std::string key = "red|" + key_of(n.output, idx);
        auto it = reduce_memo_.find(key);
        if (it != reduce_memo_.end()) return it->second;
        const TensorType& x = g_.type(n.inputs[0]);
        const TensorType& t = g_.type(n.output);
        auto axes = n.ints("axes");
        Index src = idx;
        if (axes.size() == 1) {
            src.push_back(col_comp());
        } else {
            std::vector<int64_t> tail(x.shape.end() - axes.size(), x.shape.end());
            Comp flat;
            flat.base = "c0";
            flat.expr = "(c0 + e)";
            flat.lane = flat.e_dep = flat.c_dep = true;
            Index tail_idx = unravel(flat, tail);
            src.insert(src.end(), tail_idx.begin(), tail_idx.end());
        }
        Phase ph;
        ph.reduces = true;
        CType ct = ctype(t.dtype);
        ph.acc_type = ct.compute;
        ph.acc = fresh("acc");
        ph.result = fresh("red");
        bool sum = n.op == "reduce_sum";
        bool flt = dtype_is_float(t.dtype);
        if (sum) {
            ph.init = flt ? (t.dtype == LB_F64 ? "0.0" : "0.0f") : format("(%s)0", ct.compute);
            if (flt) ph.combine_a_b = t.dtype == LB_F64 ? "(%A + %B)" : format("%s(__fadd_rn(%%A, %%B))", rnd_fn(t.dtype));
            else ph.combine_a_b = format("(%s)((%s)%%A + (%s)%%B)", ct.compute, ct.unsigned_t, ct.unsigned_t);
        } else {
            if (flt) {
                ph.init = float_literal(-INFINITY, t.dtype);
                ph.combine_a_b = "fmax_nan(%A, %B)";
            } else {
                static const char* lowest[] = {"false", "(i8)-128", "(i16)-32768", "(-2147483647 - 1)", "(-9223372036854775807LL - 1)", "(u8)0", "(u16)0", "0u", "0ull"};
                ph.init = lowest[t.dtype];
                ph.combine_a_b = t.dtype == LB_BOOL ? "(%A || %B)" : format("imax<%s>(%%A, %%B)", ct.compute);
            }
        }
        std::string val = gen(n.inputs[0], src, ph);
        ph.body += accumulate(ph.acc, ph.combine_a_b, val);
        row_decls_ += format("%s %s;\n", ct.compute, ph.result.c_str());
        phases_.push_back(ph);
        reduce_memo_[key] = ph.result;
        return ph.result;
    }

    // ---- emission ---------------------------------------------------------------------------------------
    std::string indent(const std::string& code, int n) {
        std::string pad(n, ' '), out;
        std::istringstream ss(code);
        for (std::string line; std::getline(ss, line);) out += pad + line + "\n";
        return out;
    }

    FusedKernel emit() {
        FusedKernel k;
        std::ostringstream s;
        bool guard = C_ % ((int64_t)T_ * VEC_) != 0;
        s << "// generated by lumen_b200: fused row kernel over [" << R_ << ", " << C_ << "], " << T_
          << " threads per row, " << RPB_ << " rows per block, vectors of " << VEC_ << "\n";
        s << kPreamble;
        s << "typedef " << (wide_index_ ? "long long" : "int") << " idx_t;\n";
        s << "#define VEC " << VEC_ << "\n#define NCH " << NCH_ << "\n#define TPR " << T_ << "\n#define RPB " << RPB_ << "\n";
        s << "#define NCOLS " << C_ << "LL\n#define NROWS " << (multi_ ? std::string("group_rows") : std::to_string(R_) + "LL") << "\n";
        s << "#define CHUNK_LOOP_BEGIN _Pragma(\"unroll\") for (int ch = 0; ch < NCH; ch++) { const idx_t c0 = (idx_t)(ch * TPR + lane_in_row) * VEC; "
          << (guard ? "if (c0 < NCOLS) {" : "{") << "\n";
        s << "#define CHUNK_LOOP_END }}\n";
        // row reductions
        int width = std::min(T_, 32);
        s << "template <class A, class F> __device__ __forceinline__ A row_reduce(A v, F f, A identity, void* smem) {\n";
        s << "    #pragma unroll\n    for (int m = " << width / 2 << "; m >= 1; m >>= 1) v = f(v, shfl_xor_any<A>(v, m));\n";
        if (T_ > 32) {
            s << "    A* sm = (A*)smem; const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;\n";
            s << "    if (lane == 0) sm[warp] = v;\n    __syncthreads();\n";
            s << "    v = lane < " << T_ / 32 << " ? sm[lane] : identity;\n";
            s << "    #pragma unroll\n    for (int m = 16; m >= 1; m >>= 1) v = f(v, shfl_xor_any<A>(v, m));\n";
            s << "    __syncthreads();\n";
        }
        s << "    return v;\n}\n";
        const char* restrict_kw = inplace_ ? "" : " __restrict__";
        const int n_ptrs = (int)(g_.inputs.size() + g_.outputs.size());
        if (multi_) {
            // Horizontal form (the reference's horizontal fusion of same-bodied kernels, lumen/graph_compiler/passes/
            // horizontal.rs:79): ONE launch applies the body to every group of a table passed by value - per group its
            // tensors' pointers and its row count. Only for bodies without reductions or row-constant operands.
            for (const Phase& ph : phases_)
                if (ph.reduces) fail(LB_ERR_UNSUPPORTED, "a horizontally fused kernel cannot hold a reduction");
            if (!kernel_cache_.empty() || !row_caches_.empty() || !row_decls_.empty())
                fail(LB_ERR_UNSUPPORTED, "a horizontally fused kernel takes full-shape operands and constants only");
            k.multi = true;
            k.multi_max_groups = std::max(1, (4000 - 16) / (8 * (n_ptrs + 1)));  // the table fits the 4 KB parameter space
            s << "struct MultiTable { int n; int pad; long long rows[" << k.multi_max_groups << "]; void* ptr[" << k.multi_max_groups << "]["
              << n_ptrs << "]; };\n";
            s << "extern \"C\" __global__ void __launch_bounds__(" << T_ * RPB_ << ") fused_kernel(const MultiTable table) {\n";
            // The groups' row blocks form ONE sequence dealt to the CTAs in turn: a group smaller than the grid does not
            // always land on the first CTAs (most parameters of a model have fewer row blocks than the grid has CTAs).
            s << "  long long blocks_before = 0;\n";
            s << "  for (int group = 0; group < table.n; group++) {\n";
            s << "    const long long group_rows = table.rows[group];\n";
            for (size_t i = 0; i < g_.inputs.size(); i++) s << "    const void*" << restrict_kw << " in" << i << " = table.ptr[group][" << i << "];\n";
            for (size_t i = 0; i < g_.outputs.size(); i++)
                s << "    void*" << restrict_kw << " out" << i << " = table.ptr[group][" << g_.inputs.size() + i << "];\n";
        } else {
            s << "extern \"C\" __global__ void __launch_bounds__(" << T_ * RPB_ << ") fused_kernel(";
            for (size_t i = 0; i < g_.inputs.size(); i++) s << (i ? ", " : "") << "const void*" << restrict_kw << " in" << i;
            for (size_t i = 0; i < g_.outputs.size(); i++)
                s << ((i || !g_.inputs.empty()) ? ", " : "") << "void*" << restrict_kw << " out" << i;
            s << ") {\n";
        }
        s << "    __shared__ unsigned long long red_smem[32];\n";
        s << "    const int lane_in_row = threadIdx.x % TPR, row_in_block = threadIdx.x / TPR;\n";
        s << "    const idx_t row_blocks = (idx_t)((NROWS + RPB - 1) / RPB);\n";
        s << indent(kernel_cache_, 4);
        // Rows cached in registers are loaded one row block ahead (while the current block's phases compute), when that
        // costs at most 64 bytes of registers per thread: a block's phases are a serial chain behind its loads.
        int cached_bytes = 0;
        for (const RowCache& c : row_caches_) cached_bytes += c.bytes;
        const bool prefetch = !inplace_ && !row_caches_.empty() && cached_bytes <= 64;
        std::string next_loads;
        if (prefetch) {
            for (const RowCache& c : row_caches_) {
                s << "    __align__(16) " << c.type << " " << c.buf << "_nx[NCH][VEC];\n";
                next_loads += c.load;
            }
            s << "    if ((idx_t)blockIdx.x < row_blocks) {\n        idx_t r = (idx_t)blockIdx.x * RPB + row_in_block;\n"
              << "        if (r >= NROWS) r = (idx_t)(NROWS - 1);\n" << indent(next_loads, 8) << "    }\n";
        }
        if (multi_)
            s << "    const idx_t first_rb = (idx_t)(((long long)blockIdx.x + gridDim.x - blocks_before % gridDim.x) % gridDim.x);\n"
              << "    blocks_before += row_blocks;\n";
        s << "    for (idx_t rb = " << (multi_ ? "first_rb" : "blockIdx.x") << "; rb < row_blocks; rb += gridDim.x) {\n";
        s << "        idx_t r = rb * RPB + row_in_block;\n";
        s << "        const bool active = r < NROWS;\n";
        s << "        if (!active) r = (idx_t)(NROWS - 1);\n";
        s << indent(row_decls_, 8);
        if (prefetch) {
            for (const RowCache& c : row_caches_) {
                s << "        __align__(16) " << c.type << " " << c.buf << "[NCH][VEC];\n";
                s << "        _Pragma(\"unroll\") for (int ch = 0; ch < NCH; ch++) { _Pragma(\"unroll\") for (int e = 0; e < VEC; e++) " << c.buf
                  << "[ch][e] = " << c.buf << "_nx[ch][e]; }\n";
            }
            s << "        if (rb + (idx_t)gridDim.x < row_blocks) {\n            idx_t r = (rb + (idx_t)gridDim.x) * RPB + row_in_block;\n"
              << "            if (r >= NROWS) r = (idx_t)(NROWS - 1);\n" << indent(next_loads, 12) << "        }\n";
        } else {
            s << indent(row_cache_, 8);
        }
        for (const Phase& ph : phases_) {
            s << "        {\n";
            if (ph.reduces) s << "            " << ph.acc_type << " " << ph.acc << " = " << ph.init << ";\n";
            if (ph.chunked) {
                s << "            CHUNK_LOOP_BEGIN\n";
                s << indent(ph.pre, 16);
                if (!ph.body.empty()) {
                    s << "                #pragma unroll\n                for (int e = 0; e < VEC; e += " << (pair_ ? 2 : 1) << ") {\n";
                    s << indent(ph.body, 20);
                    s << "                }\n";
                }
                s << indent(ph.post, 16);
                s << "            CHUNK_LOOP_END\n";
            } else {
                s << indent(ph.pre, 12);
            }
            if (ph.reduces) {
                s << "            " << ph.result << " = row_reduce<" << ph.acc_type << ">(" << ph.acc << ", [](" << ph.acc_type
                  << " a, " << ph.acc_type << " b) { return " << subst(ph.combine_a_b, "a", "b") << "; }, (" << ph.acc_type
                  << ")" << ph.init << ", red_smem);\n";
            }
            s << "        }\n";
        }
        s << (multi_ ? "    }\n  }\n}\n" : "    }\n}\n");
        k.source = s.str();
        k.rows = R_;
        k.cols = C_;
        k.threads = T_ * RPB_;
        k.rows_per_block = RPB_;
        k.vec = VEC_;
        k.n_inputs = (int)g_.inputs.size();
        k.n_outputs = (int)g_.outputs.size();
        for (int v : g_.inputs) k.types.push_back(g_.type(v));
        for (int v : g_.outputs) k.types.push_back(g_.type(v));
        return k;
    }

  public:
    void set_multi_phase(bool v) { multi_phase_hint_ = v; }
    // ---- column mode: reductions over the leading axes ------------------------------------------------------
    // Pass 1 (fused_kernel): grid (column blocks, row slices); a thread owns VEC columns and adds its slice's rows
    // in order. Pass 2 (fused_finalize): a thread adds the slices' partial sums in order and applies the epilogue.
    // The order of every sum is fixed, so results are bit-reproducible.
    static bool leading_axes(const Node& n, const TensorType& x, int* lead) {
        auto axes = n.ints("axes");
        std::sort(axes.begin(), axes.end());
        if (axes.empty() || (int)axes.size() >= x.rank()) return false;
        for (size_t k = 0; k < axes.size(); k++)
            if (axes[k] != (int64_t)k) return false;
        *lead = (int)axes.size();
        return true;
    }

    FusedKernel run_columns() {
        column_mode_ = true;
        const TensorType* space = nullptr;
        for (const Node& n : g_.nodes) {
            if (n.op != "reduce_sum" && n.op != "reduce_max") continue;
            const TensorType& x = g_.type(n.inputs[0]);
            int lead = 0;
            if (!leading_axes(n, x, &lead)) fail(LB_ERR_UNSUPPORTED, "mixed row and column reductions in one fusion");
            int64_t r = 1;
            for (int d = 0; d < lead; d++) r *= x.shape[d];
            int64_t c = x.numel() / std::max<int64_t>(r, 1);
            if (space && (r != R_ || c != C_)) fail(LB_ERR_UNSUPPORTED, "column reductions over different shapes in one fusion");
            space = &x, R_ = r, C_ = r ? c : 0, lead_rank_ = lead;
            col_reduces_.push_back(n.output);
        }
        has_reduce_ = true;
        int min_size = 8;
        for (int v : g_.inputs)
            if (g_.type(v).numel() == R_ * C_) min_size = std::min(min_size, dtype_size(g_.type(v).dtype));
        VEC_ = std::min(8, 16 / min_size);
        while (VEC_ > 1 && (C_ % VEC_ != 0 || space->shape.back() % VEC_ != 0)) VEC_ /= 2;
        wide_index_ = R_ * C_ >= (1LL << 31) - 4096;
        pair_ = VEC_ >= 2 && computes_bf16();
        // both passes: 256 threads = 32 column lanes (VEC columns each) x 8 row lanes (pass 2: slice lanes)
        const int threads = 256, col_lanes = 32, row_lanes = 8, fin_threads = 256;
        int64_t col_blocks = std::max<int64_t>((C_ + (int64_t)col_lanes * VEC_ - 1) / ((int64_t)col_lanes * VEC_), 1);
        int64_t fin_blocks = col_blocks;
        // enough slices to fill the GPU a few times over, each at least 64 rows long
        int64_t slices = std::min<int64_t>(std::max<int64_t>(1, (148 * 4 + col_blocks - 1) / col_blocks), std::max<int64_t>(R_ / 64, 1));
        int64_t rows_per_slice = (R_ + slices - 1) / std::max<int64_t>(slices, 1);
        slices = rows_per_slice ? (R_ + rows_per_slice - 1) / rows_per_slice : 1;

        std::vector<int64_t> lead_shape(space->shape.begin(), space->shape.begin() + lead_rank_);
        std::vector<int64_t> trail_shape(space->shape.begin() + lead_rank_, space->shape.end());
        Comp flat_c;
        flat_c.base = "c0", flat_c.expr = "(c0 + e)";
        flat_c.lane = flat_c.e_dep = flat_c.c_dep = true;

        // pass 1
        Phase part;
        std::ostringstream decl, store;
        size_t scratch = 0;
        std::vector<size_t> offsets;
        for (size_t k = 0; k < col_reduces_.size(); k++) {
            const Node& n = *g_.node_of(col_reduces_[k]);
            const TensorType& t = g_.type(n.output);
            CType ct = ctype(t.dtype);
            Index idx = unravel(row_comp(), lead_shape);
            Index tail = unravel(flat_c, trail_shape);
            idx.insert(idx.end(), tail.begin(), tail.end());
            bool prev = column_mode_;
            std::string val = gen(n.inputs[0], idx, part);
            column_mode_ = prev;
            std::string init, combine;
            reduce_ops(n, t, &init, &combine);
            decl << ct.compute << " acc" << k << "[VEC];\n#pragma unroll\nfor (int e = 0; e < VEC; e++) acc" << k << "[e] = " << init << ";\n";
            part.body += accumulate(format("acc%d[e]", (int)k), combine, val);
            offsets.push_back(scratch);
            int width = std::string(ct.compute) == "double" || std::string(ct.compute) == "i64" || std::string(ct.compute) == "u64" ? 8
                        : (std::string(ct.compute) == "float" || std::string(ct.compute) == "i32" || std::string(ct.compute) == "u32") ? 4
                        : dtype_size(t.dtype);
            // the 8 row lanes of a column are combined in lane order through shared memory, then lane 0 stores the slice's partial
            store << "__shared__ " << ct.compute << " red" << k << "[" << row_lanes << "][" << col_lanes << " * VEC];\n";
            store << "#pragma unroll\nfor (int e = 0; e < VEC; e++) red" << k << "[row_lane][col_lane * VEC + e] = acc" << k << "[e];\n__syncthreads();\n";
            store << "if (row_lane == 0 && in_range) {\n#pragma unroll\n    for (int e = 0; e < VEC; e++) {\n        " << ct.compute << " t = acc" << k
                  << "[e];\n        for (int y = 1; y < " << row_lanes << "; y++) t = " << subst(combine, "t", format("red%d[y][col_lane * VEC + e]", (int)k))
                  << ";\n        ((" << ct.compute << "*)((char*)scratch + " << scratch << "))[(idx_t)blockIdx.y * NCOLS + c0 + e] = t;\n    }\n}\n";
            scratch += (size_t)slices * C_ * width;
            scratch = (scratch + 255) & ~(size_t)255;
        }
        // pass 2
        Phase fin;
        std::ostringstream totals;
        for (size_t k = 0; k < col_reduces_.size(); k++) {
            const Node& n = *g_.node_of(col_reduces_[k]);
            const TensorType& t = g_.type(n.output);
            CType ct = ctype(t.dtype);
            std::string init, combine;
            reduce_ops(n, t, &init, &combine);
            // slice lane y adds slices y, y + 8, ... in order; the lanes are then combined in lane order
            totals << ct.compute << " tot" << k << "[VEC];\n#pragma unroll\nfor (int e = 0; e < VEC; e++) tot" << k << "[e] = " << init << ";\n";
            totals << "if (in_range) {\n#pragma unroll 4\n    for (int s = row_lane; s < SLICES; s += " << row_lanes << ") {\n#pragma unroll\n        for (int e = 0; e < VEC; e++) { "
                   << ct.compute << " pv = ((const " << ct.compute << "*)((const char*)scratch + " << offsets[k] << "))[(idx_t)s * NCOLS + c0 + e]; tot" << k
                   << "[e] = " << subst(combine, format("tot%d[e]", (int)k), "pv") << "; }\n    }\n}\n";
            totals << "__shared__ " << ct.compute << " fred" << k << "[" << row_lanes << "][" << col_lanes << " * VEC];\n";
            totals << "#pragma unroll\nfor (int e = 0; e < VEC; e++) fred" << k << "[row_lane][col_lane * VEC + e] = tot" << k << "[e];\n__syncthreads();\n";
            totals << "if (row_lane == 0) {\n#pragma unroll\n    for (int e = 0; e < VEC; e++)\n        for (int y = 1; y < " << row_lanes << "; y++) tot" << k << "[e] = "
                   << subst(combine, format("tot%d[e]", (int)k), format("fred%d[y][col_lane * VEC + e]", (int)k)) << ";\n}\n";
        }
        for (size_t k = 0; k < g_.outputs.size(); k++) {
            const TensorType& t = g_.type(g_.outputs[k]);
            if (t.numel() != C_) fail(LB_ERR_UNSUPPORTED, format("column-reduction fusion output %s does not have %lld elements", t.str().c_str(), (long long)C_));
            Index idx = unravel(flat_c, t.shape);
            std::string val = gen(g_.outputs[k], idx, fin);
            CType ct = ctype(t.dtype);
            fin.pre += format("__align__(16) %s ob%d[VEC];\n", ct.memory, (int)k);
            fin.body += store_element(format("ob%d", (int)k), t.dtype, val);
            fin.post += format("stv<%s, VEC>((%s*)out%d + c0, ob%d);\n", ct.memory, ct.memory, (int)k, (int)k);
        }

        std::ostringstream s;
        s << "// generated by lumen_b200: column reduction over [" << R_ << " rows, " << C_ << " columns], " << slices << " row slices\n";
        s << kPreamble;
        s << "typedef " << (wide_index_ ? "long long" : "int") << " idx_t;\n";
        s << "#define VEC " << VEC_ << "\n#define NCOLS " << C_ << "LL\n#define NROWS " << R_ << "LL\n#define SLICES " << slices
          << "\n#define ROWS_PER_SLICE " << rows_per_slice << "LL\n";
        std::string sig;
        for (size_t i = 0; i < g_.inputs.size(); i++) sig += format("const void* __restrict__ in%d, ", (int)i);
        for (size_t i = 0; i < g_.outputs.size(); i++) sig += format("void* __restrict__ out%d, ", (int)i);
        sig += "void* __restrict__ scratch";
        s << "extern \"C\" __global__ void __launch_bounds__(" << threads << ") fused_kernel(" << sig << ") {\n";
        s << "    const int col_lane = threadIdx.x & " << col_lanes - 1 << ", row_lane = threadIdx.x >> 5;\n";
        s << "    const idx_t c0 = ((idx_t)blockIdx.x * " << col_lanes << " + col_lane) * VEC;\n    const bool in_range = c0 < NCOLS;\n";
        s << indent(decl.str(), 4);
        s << "    const idx_t r_end = in_range ? (idx_t)(((idx_t)blockIdx.y + 1) * ROWS_PER_SLICE < NROWS ? ((idx_t)blockIdx.y + 1) * ROWS_PER_SLICE : NROWS) : 0;\n";
        s << "    for (idx_t r = (idx_t)blockIdx.y * ROWS_PER_SLICE + row_lane; r < r_end; r += " << row_lanes << ") {\n";
        s << indent(part.pre, 8);
        s << "        #pragma unroll\n        for (int e = 0; e < VEC; e += " << (pair_ ? 2 : 1) << ") {\n" << indent(part.body, 12) << "        }\n    }\n";
        s << indent(store.str(), 4);
        s << "}\n";
        s << "extern \"C\" __global__ void __launch_bounds__(" << fin_threads << ") fused_finalize(" << sig << ") {\n";
        s << "    const int col_lane = threadIdx.x & " << col_lanes - 1 << ", row_lane = threadIdx.x >> 5;\n";
        s << "    const idx_t c0 = ((idx_t)blockIdx.x * " << col_lanes << " + col_lane) * VEC;\n    const bool in_range = c0 < NCOLS;\n";
        s << indent(totals.str(), 4);
        s << "    if (row_lane != 0 || !in_range) return;\n";
        s << indent(fin.pre, 4);
        s << "    #pragma unroll\n    for (int e = 0; e < VEC; e += " << (pair_ ? 2 : 1) << ") {\n" << indent(fin.body, 8) << "    }\n";
        s << indent(fin.post, 4);
        s << "}\n";

        FusedKernel k;
        k.source = s.str();
        k.rows = R_, k.cols = C_, k.threads = threads, k.rows_per_block = 1, k.vec = VEC_;
        k.n_inputs = (int)g_.inputs.size(), k.n_outputs = (int)g_.outputs.size();
        for (int v : g_.inputs) k.types.push_back(g_.type(v));
        for (int v : g_.outputs) k.types.push_back(g_.type(v));
        k.two_pass = true;
        k.slices = (int)slices;
        k.col_blocks = col_blocks;
        k.fin_threads = fin_threads;
        k.fin_blocks = fin_blocks;
        k.scratch_bytes = scratch;
        return k;
    }

    // identity and combine format of a reduction node with result type `t`
    void reduce_ops(const Node& n, const TensorType& t, std::string* init, std::string* combine) {
        CType ct = ctype(t.dtype);
        bool sum = n.op == "reduce_sum", flt = dtype_is_float(t.dtype);
        if (sum) {
            *init = flt ? (t.dtype == LB_F64 ? "0.0" : "0.0f") : format("(%s)0", ct.compute);
            if (flt) *combine = t.dtype == LB_F64 ? "(%A + %B)" : format("%s(__fadd_rn(%%A, %%B))", rnd_fn(t.dtype));
            else *combine = format("(%s)((%s)%%A + (%s)%%B)", ct.compute, ct.unsigned_t, ct.unsigned_t);
        } else if (flt) {
            *init = float_literal(-INFINITY, t.dtype);
            *combine = "fmax_nan(%A, %B)";
        } else {
            static const char* lowest[] = {"false", "(i8)-128", "(i16)-32768", "(-2147483647 - 1)", "(-9223372036854775807LL - 1)", "(u8)0", "(u16)0", "0u", "0ull"};
            *init = lowest[t.dtype];
            *combine = t.dtype == LB_BOOL ? "(%A || %B)" : format("imax<%s>(%%A, %%B)", ct.compute);
        }
    }

    static bool wants_columns(const Graph& g) {
        bool any = false;
        for (const Node& n : g.nodes) {
            if (n.op != "reduce_sum" && n.op != "reduce_max") continue;
            int lead;
            if (!leading_axes(n, g.type(n.inputs[0]), &lead)) return false;
            any = true;
        }
        return any;
    }
    void set_inplace(bool v) { inplace_ = v; }
    void set_multi(bool v) { multi_ = v; }

};

}  // namespace

FusedKernel generate_fused(const Module& module) {
    const Graph& g = module.main();
    int reduces = 0;
    for (const Node& n : g.nodes)
        if (n.op == "reduce_sum" || n.op == "reduce_max") reduces++;
    Generator gen(module, g);
    gen.set_inplace(module.options.count("inplace") != 0);
    gen.set_multi(module.options.count("multi") != 0);
    if (module.options.count("multi") && (reduces || Generator::wants_columns(g)))
        fail(LB_ERR_UNSUPPORTED, "option multi: a horizontally fused kernel cannot hold a reduction");
    if (Generator::wants_columns(g)) return gen.run_columns();
    // With a reduction followed by further use of the row, inputs are kept in registers across phases.
    gen.set_multi_phase(reduces >= 1);
    return gen.run();
}

}  // namespace lb
