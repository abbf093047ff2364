// CPU ORACLE — TEST INFRASTRUCTURE ONLY. Nothing in the product path links, loads or calls this file.
//
// A restatement of lumen's reference interpreter (lumen/reference/mod.rs) for the primitives on the CUDA hot
// path: every primitive is evaluated element by element, integers in 128-bit two's complement wrapped to the
// result dtype, floats in f64 and rounded ONCE to the result dtype after every primitive (mod.rs:189-200), with
// the single correct f64->bf16/f16 rounding through a round-to-odd f32 (lumen/tensor/dtype.rs:217-239).
//
// Parity pins. The reference itself (Rust) cannot be built in this environment, so there is no oracle/_ref, and it
// holds no binary fixtures for this path. It does hold a NumPy model of the path in its tests
// (tests/test_transformer_example.py:211-264, tests/functional/test_attention.py:17-31):
// tests/golden/make_reference_fixtures.py lifts those functions out of the reference's files, RUNS them, and the
// committed outputs (tests/golden/reference_*.npz) are what tests/test_reference_fixtures.py holds this file to -
// the bfloat16 rounding bit for bit, RMSNorm, bfloat16 matmul, causal attention and the whole 2-layer forward at the
// reference's own tolerances. tests/test_oracle_pins.py adds the reference tests' closed-form checks (integer
// edge rules, saturating casts, sequential accumulation, layer norm spelling) and exact-rational rounding vectors.
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off -fopenmp). -ffp-contract=off matters: the float fast
// path of dot_general relies on separate, individually rounded multiplies and adds.
#ifdef _OPENMP
#include <omp.h>
#endif
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

typedef __int128 i128;

enum DType { BOOL, I8, I16, I32, I64, U8, U16, U32, U64, F16, BF16, F32, F64 };

const char* kNames[] = {"bool",   "int8",   "int16",   "int32",    "int64",   "uint8",  "uint16",
                        "uint32", "uint64", "float16", "bfloat16", "float32", "float64"};
const int kSize[] = {1, 1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};

DType parse_dtype(const std::string& s) {
    for (int i = 0; i < 13; i++)
        if (s == kNames[i]) return (DType)i;
    throw std::runtime_error("unknown dtype " + s);
}
bool is_float(DType d) { return d >= F16; }

struct Type {
    DType dtype;
    std::vector<int64_t> shape;
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : shape) n *= d;
        return n;
    }
};

// mod.rs:10-14
struct Values {
    bool flt = false;
    std::vector<double> f;
    std::vector<i128> i;
    size_t size() const { return flt ? f.size() : i.size(); }
};

// ---- rounding (mod.rs:166-220, dtype.rs:217-239) -----------------------------------------------------------
float round_to_odd(double x) {
    float f = (float)x;
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if (!std::isfinite(f) || (double)f == x || (bits & 1)) return f;
    bool outward = ((double)f < x) != std::signbit(f);
    bits = outward ? bits + 1 : bits - 1;
    memcpy(&f, &bits, 4);
    return f;
}

double bf16_round_f32(float f) {  // round to nearest even, the `half` crate's bf16::from_f32
    uint32_t b;
    memcpy(&b, &f, 4);
    if ((b & 0x7fffffffu) > 0x7f800000u) {
        b |= 0x00400000u;  // quiet the NaN, keep it a NaN
        b &= 0xffff0000u;
    } else {
        uint32_t round_bit = 0x8000u;
        if ((b & round_bit) && (b & (3 * round_bit - 1))) b += round_bit;  // > half, or half and odd
        b &= 0xffff0000u;
    }
    memcpy(&f, &b, 4);
    return (double)f;
}

double f16_round_f32(float f) {  // f32 -> binary16 (RNE) -> f64
    if (std::isnan(f)) return NAN;
    uint32_t b;
    memcpy(&b, &f, 4);
    uint32_t sign = b >> 31;
    float a = std::fabs(f);
    double r;
    if (a >= 65520.0f)
        r = INFINITY;  // rounds past the largest finite half (65504)
    else if (a < 6.103515625e-05f) {
        // subnormal halves: multiples of 2^-24, nearbyint is round-half-even in the default mode
        r = std::nearbyint((double)a * 16777216.0) / 16777216.0;
    } else {
        int e;
        std::frexp(a, &e);  // a = m * 2^e, m in [0.5, 1)
        double ulp = std::ldexp(1.0, e - 11);
        r = std::nearbyint((double)a / ulp) * ulp;
    }
    return sign ? -r : r;
}

double round_to(double x, DType d) {
    switch (d) {
        case F64: return x;
        case F32: return (double)(float)x;
        case BF16: return bf16_round_f32(round_to_odd(x));
        case F16: return f16_round_f32(round_to_odd(x));
        default: throw std::runtime_error("round: not a float dtype");
    }
}

i128 wrap(i128 x, DType d) {
    switch (d) {
        case BOOL: return x != 0;
        case U8: return (uint8_t)x;
        case U16: return (uint16_t)x;
        case U32: return (uint32_t)x;
        case U64: return (uint64_t)x;
        case I8: return (int8_t)x;
        case I16: return (int16_t)x;
        case I32: return (int32_t)x;
        case I64: return (int64_t)x;
        default: throw std::runtime_error("wrap: not an integer dtype");
    }
}

// Rust `as` casts from f64: saturating, NaN to 0 (mod.rs:203-220)
i128 saturate(double x, DType d) {
    if (d == BOOL) return x != 0.0;
    if (std::isnan(x)) return 0;
    double lo, hi;
    switch (d) {
        case U8: lo = 0, hi = 255; break;
        case U16: lo = 0, hi = 65535; break;
        case U32: lo = 0, hi = 4294967295.0; break;
        case U64: lo = 0, hi = 18446744073709551615.0; break;
        case I8: lo = -128, hi = 127; break;
        case I16: lo = -32768, hi = 32767; break;
        case I32: lo = -2147483648.0, hi = 2147483647.0; break;
        case I64: lo = -9223372036854775808.0, hi = 9223372036854775807.0; break;
        default: throw std::runtime_error("saturate: not an integer dtype");
    }
    if (x <= lo) return (i128)lo;
    if (x >= hi) {
        switch (d) {
            case U64: return (i128)UINT64_MAX;
            case I64: return (i128)INT64_MAX;
            default: return (i128)hi;
        }
    }
    return (i128)std::trunc(x);
}

int bits_of(DType d) { return d == BOOL ? 1 : 8 * kSize[d]; }
unsigned __int128 unsigned_bits(i128 x, int w) { return (unsigned __int128)x & (((unsigned __int128)1 << w) - 1); }
i128 signed_bits(i128 x, int w) {
    i128 b = (i128)unsigned_bits(x, w);
    return (w > 0 && b >= ((i128)1 << (w - 1))) ? b - ((i128)1 << w) : b;
}

// Zeros of opposite signs: -0 orders below +0, as IEEE 754-2019 maximum / minimum and the GPU's max / min instructions
// order them. The reference's interpreter calls Rust's f64::max / f64::min there (lumen/reference/mod.rs:234-240,385-391),
// which leave the sign of such a result to the platform.
double fmax_nan(double x, double y) {
    if (std::isnan(x) || std::isnan(y)) return NAN;
    if (x == y) return std::signbit(x) ? y : x;
    return std::max(x, y);
}
double fmin_nan(double x, double y) {
    if (std::isnan(x) || std::isnan(y)) return NAN;
    if (x == y) return std::signbit(x) ? x : y;
    return std::min(x, y);
}

// ---- graph text -------------------------------------------------------------------------------------------
struct Graph;
struct Node {
    std::string op;
    std::vector<int> inputs;
    int output;
    std::map<std::string, std::string> attrs;
};
struct Graph {
    std::vector<Type> types;  // indexed by value id (sparse ids allowed)
    std::vector<int> inputs, outputs;
    std::vector<Node> nodes;
};

std::vector<int64_t> parse_list(const std::string& s) {
    std::vector<int64_t> out;
    if (s.empty() || s == "-") return out;
    std::stringstream ss(s);
    std::string item;
    while (std::getline(ss, item, ',')) out.push_back(std::stoll(item));
    return out;
}

std::vector<std::shared_ptr<Graph>> parse_graphs(const std::string& text) {
    std::vector<std::shared_ptr<Graph>> graphs;
    std::shared_ptr<Graph> g;
    std::stringstream lines(text);
    std::string line;
    auto set_type = [&](int id, DType d, std::vector<int64_t> shape) {
        if ((int)g->types.size() <= id) g->types.resize(id + 1);
        g->types[id] = Type{d, std::move(shape)};
    };
    while (std::getline(lines, line)) {
        std::stringstream ts(line);
        std::vector<std::string> tok;
        std::string t;
        while (ts >> t) tok.push_back(t);
        if (tok.empty()) continue;
        if (tok[0] == "graph") {
            g = std::make_shared<Graph>();
        } else if (tok[0] == "in") {
            int id = std::stoi(tok[1]);
            set_type(id, parse_dtype(tok[2]), parse_list(tok[3]));
            g->inputs.push_back(id);
        } else if (tok[0] == "node") {
            Node n;
            n.output = std::stoi(tok[1]);
            n.op = tok[2];
            set_type(n.output, parse_dtype(tok[3]), parse_list(tok[4]));
            for (auto v : parse_list(tok[5])) n.inputs.push_back((int)v);
            for (size_t k = 6; k < tok.size(); k++) {
                auto eq = tok[k].find('=');
                n.attrs[tok[k].substr(0, eq)] = tok[k].substr(eq + 1);
            }
            g->nodes.push_back(std::move(n));
        } else if (tok[0] == "out") {
            for (auto v : parse_list(tok[1])) g->outputs.push_back((int)v);
        } else if (tok[0] == "end") {
            graphs.push_back(g);
        } else {
            throw std::runtime_error("graph text: unknown line '" + line + "'");
        }
    }
    if (graphs.empty()) throw std::runtime_error("graph text: no graph");
    return graphs;
}

// ---- indexing helpers ---------------------------------------------------------------------------------------
int64_t ravel(const std::vector<int64_t>& idx, const std::vector<int64_t>& shape) {
    int64_t flat = 0;
    for (size_t d = 0; d < shape.size(); d++) flat = flat * shape[d] + idx[d];
    return flat;
}

// Calls f(idx) for every index of `shape` in row-major order.
template <class F>
void for_each_index(const std::vector<int64_t>& shape, F f) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    if (n == 0) return;
    std::vector<int64_t> idx(shape.size(), 0);
    for (int64_t k = 0; k < n; k++) {
        f(idx);
        for (int d = (int)shape.size() - 1; d >= 0; d--) {
            if (++idx[d] < shape[d]) break;
            idx[d] = 0;
        }
    }
}

// Calls f(k, idx) for every index of `shape`, k its row-major number; ranges of k run on separate threads (each
// thread unravels the first index of its range, then counts on), so `f` must only write slot k of its output.
template <class F>
void for_each_index_parallel(const std::vector<int64_t>& shape, F f) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    if (n == 0) return;
    const int64_t chunk = 1 << 16, chunks = (n + chunk - 1) / chunk;
#pragma omp parallel for schedule(static) if (chunks > 1)
    for (int64_t c = 0; c < chunks; c++) {
        std::vector<int64_t> idx(shape.size(), 0);
        int64_t k = c * chunk, rest = k;
        for (int d = (int)shape.size() - 1; d >= 0; d--) {
            idx[d] = rest % shape[d];
            rest /= shape[d];
        }
        const int64_t end = std::min(n, k + chunk);
        for (; k < end; k++) {
            f(k, idx);
            for (int d = (int)shape.size() - 1; d >= 0; d--) {
                if (++idx[d] < shape[d]) break;
                idx[d] = 0;
            }
        }
    }
}

// mod.rs:393-405: out[index] = x[source(index)]. `source` is called from several threads.
template <class F>
Values gather_by(const Values& x, const Type& out, F source) {
    Values r;
    r.flt = x.flt;
    const int64_t n = out.numel();
    if (x.flt) {
        r.f.resize(n);
        for_each_index_parallel(out.shape, [&](int64_t k, const std::vector<int64_t>& idx) { r.f[k] = x.f[source(idx)]; });
    } else {
        r.i.resize(n);
        for_each_index_parallel(out.shape, [&](int64_t k, const std::vector<int64_t>& idx) { r.i[k] = x.i[source(idx)]; });
    }
    return r;
}

std::vector<int64_t> taken(const Values& idx, int64_t n) {  // mod.rs:414-423
    std::vector<int64_t> out(idx.i.size());
    i128 hi = std::max<i128>(n - 1, 0);
    for (size_t k = 0; k < out.size(); k++) out[k] = (int64_t)std::min(std::max<i128>(idx.i[k], 0), hi);
    return out;
}

std::vector<int64_t> free_dims(size_t rank, const std::vector<int64_t>& used) {
    std::vector<int64_t> out;
    for (size_t d = 0; d < rank; d++)
        if (std::find(used.begin(), used.end(), (int64_t)d) == used.end()) out.push_back(d);
    return out;
}

// x permuted so its dimensions come in the order `perm`, flattened row-major
template <class T>
std::vector<T> permuted(const std::vector<T>& x, const std::vector<int64_t>& shape, const std::vector<int64_t>& perm) {
    std::vector<int64_t> out_shape, strides(shape.size(), 1);
    for (int d = (int)shape.size() - 2; d >= 0; d--) strides[d] = strides[d + 1] * shape[d + 1];
    for (auto d : perm) out_shape.push_back(shape[d]);
    std::vector<T> out(x.size());
    for_each_index_parallel(out_shape, [&](int64_t flat, const std::vector<int64_t>& idx) {
        int64_t at = 0;
        for (size_t k = 0; k < perm.size(); k++) at += idx[k] * strides[perm[k]];
        out[flat] = x[at];
    });
    return out;
}

int64_t prod_of(const std::vector<int64_t>& shape, const std::vector<int64_t>& dims) {
    int64_t n = 1;
    for (auto d : dims) n *= shape[d];
    return n;
}

Values eval_graph(const Graph& g, const std::vector<std::shared_ptr<Graph>>& all, const std::vector<const Values*>& inputs,
                  std::vector<Values>* all_outputs);

double attr_value_f(const std::string& v) {
    // fill_value: b:<0|1>, i:<int>, f:<hex float>
    if (v[0] == 'f') return std::strtod(v.c_str() + 2, nullptr);
    return (double)std::stoll(v.substr(2));
}

// ---- eval (mod.rs:442-1128) -----------------------------------------------------------------------------
Values eval(const Node& n, const std::vector<const Values*>& a, const std::vector<const Type*>& ty, const Type& out,
            const std::vector<std::shared_ptr<Graph>>& all) {
    const std::string& p = n.op;
    DType dtype = out.dtype;
    Values r;
    auto attr = [&](const char* k) -> const std::string& {
        auto it = n.attrs.find(k);
        if (it == n.attrs.end()) throw std::runtime_error(p + ": missing attribute " + k);
        return it->second;
    };
    const int64_t N = out.numel();

    if (p == "add" || p == "sub" || p == "mul" || p == "div" || p == "max" || p == "eq" || p == "lt") {
        const Values &x = *a[0], &y = *a[1];
        if (!x.flt) {  // mod.rs:449-468
            r.i.resize(N);
#pragma omp parallel for if (N > 65536)
            for (int64_t k = 0; k < N; k++) {
                i128 A = x.i[k], B = y.i[k], v;
                if (p == "add") v = A + B;
                else if (p == "sub") v = A - B;
                else if (p == "mul") v = (i128)((unsigned __int128)A * (unsigned __int128)B);
                else if (p == "div") v = B == 0 ? -1 : A / B;  // division by zero yields -1
                else if (p == "max") v = std::max(A, B);
                else if (p == "eq") v = A == B;
                else v = A < B;
                r.i[k] = wrap(v, dtype);
            }
        } else if (p == "eq" || p == "lt") {  // mod.rs:473-474
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = p == "eq" ? x.f[k] == y.f[k] : x.f[k] < y.f[k];
        } else {  // mod.rs:475-489
            r.flt = true;
            r.f.resize(N);
            int op = p == "add" ? 0 : p == "sub" ? 1 : p == "mul" ? 2 : p == "div" ? 3 : 4;
#pragma omp parallel for if (N > 65536)
            for (int64_t k = 0; k < N; k++) {
                double A = x.f[k], B = y.f[k], v;
                switch (op) {
                    case 0: v = A + B; break;
                    case 1: v = A - B; break;
                    case 2: v = A * B; break;
                    case 3: v = A / B; break;
                    default: v = fmax_nan(A, B);
                }
                r.f[k] = round_to(v, dtype);
            }
        }
        return r;
    }
    if (p == "neg") {  // mod.rs:494-497
        const Values& x = *a[0];
        r.flt = x.flt;
        if (x.flt) {
            r.f.resize(N);
            for (int64_t k = 0; k < N; k++) r.f[k] = -x.f[k];
        } else {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = wrap(-x.i[k], dtype);
        }
        return r;
    }
    if (p == "abs" || p == "sign" || p == "not" || p == "rsqrt" || p == "floor" || p == "ceil" || p == "exp2" ||
        p == "log2" || p == "sin" || p == "cos" || p == "is_finite") {  // Unary, mod.rs:498-554
        const Values& x = *a[0];
        if (!x.flt) {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) {
                i128 A = x.i[k];
                if (p == "abs") r.i[k] = wrap(A < 0 ? -A : A, dtype);
                else if (p == "sign") r.i[k] = (A > 0) - (A < 0);
                else if (p == "not") r.i[k] = ty[0]->dtype == BOOL ? 1 - A : wrap(~A, dtype);
                else if (p == "is_finite") r.i[k] = 1;
                else throw std::runtime_error(p + " of an integer");
            }
            return r;
        }
        if (p == "is_finite") {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = std::isfinite(x.f[k]);
            return r;
        }
        r.flt = true;
        r.f.resize(N);
#pragma omp parallel for if (N > 65536)
        for (int64_t k = 0; k < N; k++) {
            double A = x.f[k], v;
            if (p == "abs") v = std::fabs(A);
            else if (p == "sign") v = (A == 0.0 || std::isnan(A)) ? A : (std::signbit(A) ? -1.0 : 1.0);
            else if (p == "rsqrt") v = 1.0 / std::sqrt(A);
            else if (p == "floor") v = std::floor(A);
            else if (p == "ceil") v = std::ceil(A);
            else if (p == "exp2") v = std::exp2(A);
            else if (p == "log2") v = std::log2(A);
            else if (p == "sin") v = std::sin(A);
            else if (p == "cos") v = std::cos(A);
            else throw std::runtime_error(p + " of a float");
            r.f[k] = round_to(v, dtype);
        }
        return r;
    }
    if (p == "min" || p == "pow" || p == "rem" || p == "and" || p == "or" || p == "xor") {  // Binary, mod.rs:555-602
        const Values &x = *a[0], &y = *a[1];
        if (!x.flt) {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) {
                i128 A = x.i[k], B = y.i[k];
                if (p == "rem") r.i[k] = B == 0 ? A : A % B;  // remainder by zero yields the dividend
                else if (p == "min") r.i[k] = std::min(A, B);
                else if (p == "and") r.i[k] = wrap(A & B, dtype);
                else if (p == "or") r.i[k] = wrap(A | B, dtype);
                else if (p == "xor") r.i[k] = wrap(A ^ B, dtype);
                else throw std::runtime_error(p + " of integers");
            }
            return r;
        }
        r.flt = true;
        r.f.resize(N);
        for (int64_t k = 0; k < N; k++) {
            double A = x.f[k], B = y.f[k];
            if (p == "pow") r.f[k] = round_to(std::pow(A, B), dtype);
            else if (p == "rem") r.f[k] = round_to(std::fmod(A, B), dtype);
            else if (p == "min") r.f[k] = fmin_nan(A, B);
            else throw std::runtime_error(p + " of floats");
        }
        return r;
    }
    if (p == "exp" || p == "log" || p == "sqrt" || p == "tanh" || p == "logistic") {  // mod.rs:603-617
        const Values& x = *a[0];
        r.flt = true;
        r.f.resize(N);
        int op = p == "exp" ? 0 : p == "log" ? 1 : p == "sqrt" ? 2 : p == "tanh" ? 3 : 4;
#pragma omp parallel for if (N > 16384)
        for (int64_t k = 0; k < N; k++) {
            double A = x.f[k], v;
            switch (op) {
                case 0: v = std::exp(A); break;
                case 1: v = std::log(A); break;
                case 2: v = std::sqrt(A); break;
                case 3: v = std::tanh(A); break;
                default: v = 1.0 / (1.0 + std::exp(-A));
            }
            r.f[k] = round_to(v, dtype);
        }
        return r;
    }
    if (p == "cast") {  // mod.rs:618-633
        const Values& x = *a[0];
        if (!x.flt && is_float(dtype)) {
            r.flt = true;
            r.f.resize(N);
            for (int64_t k = 0; k < N; k++) {
                i128 A = x.i[k];
                r.f[k] = dtype == F64 ? (double)A : dtype == F32 ? (double)(float)A : round_to((double)A, dtype);
            }
        } else if (!x.flt) {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = wrap(x.i[k], dtype);
        } else if (is_float(dtype)) {
            r.flt = true;
            r.f.resize(N);
#pragma omp parallel for if (N > 65536)
            for (int64_t k = 0; k < N; k++) r.f[k] = round_to(x.f[k], dtype);
        } else {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = saturate(x.f[k], dtype);
        }
        return r;
    }
    if (p == "select") {  // mod.rs:634-644
        const Values &pred = *a[0], &x = *a[1], &y = *a[2];
        r.flt = x.flt;
        if (x.flt) {
            r.f.resize(N);
            for (int64_t k = 0; k < N; k++) r.f[k] = pred.i[k] != 0 ? x.f[k] : y.f[k];
        } else {
            r.i.resize(N);
            for (int64_t k = 0; k < N; k++) r.i[k] = pred.i[k] != 0 ? x.i[k] : y.i[k];
        }
        return r;
    }
    if (p == "reduce_sum" || p == "reduce_max") {  // mod.rs:645-695
        // Each output accumulates its elements in row-major order of the input, the accumulator rounded
        // (wrapped) to the result dtype after every add. Moving the kept dimensions ahead of the reduced ones
        // keeps that order within each output and lets outputs run in parallel.
        const Type& x = *ty[0];
        auto axes = parse_list(attr("axes"));
        auto kept = free_dims(x.shape.size(), axes);
        std::sort(axes.begin(), axes.end());
        std::vector<int64_t> perm = kept;
        perm.insert(perm.end(), axes.begin(), axes.end());
        int64_t inner = prod_of(x.shape, axes);
        bool sum = p == "reduce_sum";
        r.flt = a[0]->flt;
        if (r.flt) {
            auto v = permuted(a[0]->f, x.shape, perm);
            r.f.resize(N);
#pragma omp parallel for if (N > 64)
            for (int64_t o = 0; o < N; o++) {
                double acc = sum ? 0.0 : -INFINITY;
                const double* row = v.data() + o * inner;
                for (int64_t k = 0; k < inner; k++) acc = sum ? round_to(acc + row[k], dtype) : fmax_nan(acc, row[k]);
                r.f[o] = acc;
            }
        } else {
            auto v = permuted(a[0]->i, x.shape, perm);
            r.i.resize(N);
            bool is_signed = dtype >= I8 && dtype <= I64;
            i128 lowest = is_signed ? -((i128)1 << (bits_of(dtype) - 1)) : 0;  // mod.rs:223-231
            for (int64_t o = 0; o < N; o++) {
                i128 acc = sum ? 0 : lowest;
                for (int64_t k = 0; k < inner; k++)
                    acc = sum ? wrap(acc + v[o * inner + k], dtype) : std::max(acc, v[o * inner + k]);
                r.i[o] = acc;
            }
        }
        return r;
    }
    if (p == "dot_general") {  // mod.rs:881-973
        const Type &lhs = *ty[0], &rhs = *ty[1];
        auto lc = parse_list(attr("lhs_contracting")), rc = parse_list(attr("rhs_contracting"));
        auto lb = parse_list(attr("lhs_batch")), rb = parse_list(attr("rhs_batch"));
        DType accum = parse_dtype(attr("accum_dtype"));
        auto lused = lb, rused = rb;
        lused.insert(lused.end(), lc.begin(), lc.end());
        rused.insert(rused.end(), rc.begin(), rc.end());
        auto lfree = free_dims(lhs.shape.size(), lused), rfree = free_dims(rhs.shape.size(), rused);
        int64_t B = prod_of(lhs.shape, lb), M = prod_of(lhs.shape, lfree), Nn = prod_of(rhs.shape, rfree),
                K = prod_of(lhs.shape, lc);
        // canonical [B, M, K] and [B, K, N]: the contracting index runs in the reference's order (row-major over
        // the contracting dims as listed), and each output sums its K terms sequentially.
        std::vector<int64_t> lperm = lb, rperm = rb;
        lperm.insert(lperm.end(), lfree.begin(), lfree.end());
        lperm.insert(lperm.end(), lc.begin(), lc.end());
        rperm.insert(rperm.end(), rc.begin(), rc.end());
        rperm.insert(rperm.end(), rfree.begin(), rfree.end());
        if (a[0]->flt) {
            auto L = permuted(a[0]->f, lhs.shape, lperm), R = permuted(a[1]->f, rhs.shape, rperm);
            r.flt = true;
            r.f.resize(N);
            if (accum == F32) {
                // round(acc + round(x*y, f32), f32) in f64 equals the plain f32 multiply and add (operands are
                // f32 or narrower; no contraction: -ffp-contract=off), vectorised across the output row.
                std::vector<float> Lf(L.begin(), L.end()), Rf(R.begin(), R.end());
                // Tiles of 32 rows x 512 columns: a tile's slice of the right operand (K x 512 floats) stays in cache
                // while its rows use it. Every output still adds its K products one after the other in k order.
                const int64_t MB = 32, NB = 512, mt = (M + MB - 1) / MB, nt = (Nn + NB - 1) / NB;
#pragma omp parallel for collapse(3) schedule(dynamic)
                for (int64_t b = 0; b < B; b++)
                    for (int64_t tj = 0; tj < nt; tj++)
                        for (int64_t tm = 0; tm < mt; tm++) {
                            const int64_t j0 = tj * NB, jn = std::min(NB, Nn - j0);
                            float acc[NB];
                            for (int64_t m = tm * MB; m < std::min(M, (tm + 1) * MB); m++) {
                                for (int64_t j = 0; j < jn; j++) acc[j] = 0.0f;
                                const float* lrow = Lf.data() + (b * M + m) * K;
                                for (int64_t k = 0; k < K; k++) {
                                    const float x = lrow[k];
                                    const float* rrow = Rf.data() + (b * K + k) * Nn + j0;
                                    for (int64_t j = 0; j < jn; j++) {
                                        float prod = x * rrow[j];
                                        acc[j] = acc[j] + prod;
                                    }
                                }
                                for (int64_t j = 0; j < jn; j++) r.f[(b * M + m) * Nn + j0 + j] = round_to((double)acc[j], dtype);
                            }
                        }
            } else {
#pragma omp parallel for collapse(2)
                for (int64_t b = 0; b < B; b++)
                    for (int64_t m = 0; m < M; m++)
                        for (int64_t j = 0; j < Nn; j++) {
                            double acc = 0.0;
                            for (int64_t k = 0; k < K; k++)
                                acc = round_to(acc + round_to(L[(b * M + m) * K + k] * R[(b * K + k) * Nn + j], accum),
                                               accum);
                            r.f[(b * M + m) * Nn + j] = round_to(acc, dtype);
                        }
            }
        } else {
            auto L = permuted(a[0]->i, lhs.shape, lperm), R = permuted(a[1]->i, rhs.shape, rperm);
            r.i.resize(N);
            for (int64_t b = 0; b < B; b++)
                for (int64_t m = 0; m < M; m++)
                    for (int64_t j = 0; j < Nn; j++) {
                        i128 acc = 0;
                        for (int64_t k = 0; k < K; k++)
                            acc = wrap(acc + (i128)((unsigned __int128)L[(b * M + m) * K + k] *
                                                    (unsigned __int128)R[(b * K + k) * Nn + j]),
                                       dtype);
                        r.i[(b * M + m) * Nn + j] = acc;
                    }
        }
        return r;
    }
    if (p == "reshape" || p == "device_wait" || p == "host_wait") return *a[0];  // mod.rs:974
    if (p == "broadcast_in_dim") {  // mod.rs:975-989
        const Type& x = *ty[0];
        auto dims = parse_list(attr("broadcast_dimensions"));
        return gather_by(*a[0], out, [&](const std::vector<int64_t>& idx) {
            int64_t flat = 0;
            for (size_t k = 0; k < dims.size(); k++) flat = flat * x.shape[k] + (x.shape[k] == 1 ? 0 : idx[dims[k]]);
            return flat;
        });
    }
    if (p == "transpose") {  // mod.rs:990-1002
        const Type& x = *ty[0];
        auto perm = parse_list(attr("permutation"));
        std::vector<int64_t> strides(x.shape.size(), 1);
        for (int d = (int)x.shape.size() - 2; d >= 0; d--) strides[d] = strides[d + 1] * x.shape[d + 1];
        return gather_by(*a[0], out, [&](const std::vector<int64_t>& idx) {  // thread-safe: no shared scratch
            int64_t flat = 0;
            for (size_t k = 0; k < perm.size(); k++) flat += idx[k] * strides[perm[k]];
            return flat;
        });
    }
    if (p == "slice") {  // mod.rs:1009-1015
        const Type& x = *ty[0];
        auto start = parse_list(attr("start_indices"));
        return gather_by(*a[0], out, [&](const std::vector<int64_t>& idx) {  // thread-safe: no shared scratch
            int64_t flat = 0;
            for (size_t k = 0; k < start.size(); k++) flat = flat * x.shape[k] + idx[k] + start[k];
            return flat;
        });
    }
    if (p == "concatenate") {  // mod.rs:1016-1058
        int64_t d = std::stoll(attr("dimension"));
        Values all_v;
        all_v.flt = a[0]->flt;
        std::vector<int64_t> starts, bases;
        int64_t start = 0, base = 0;
        for (size_t k = 0; k < a.size(); k++) {
            starts.push_back(start);
            bases.push_back(base);
            start += ty[k]->shape[d];
            base += ty[k]->numel();
            if (all_v.flt) all_v.f.insert(all_v.f.end(), a[k]->f.begin(), a[k]->f.end());
            else all_v.i.insert(all_v.i.end(), a[k]->i.begin(), a[k]->i.end());
        }
        return gather_by(all_v, out, [&](const std::vector<int64_t>& idx) {
            size_t k = std::upper_bound(starts.begin(), starts.end(), idx[d]) - starts.begin() - 1;
            std::vector<int64_t> src = idx;
            src[d] -= starts[k];
            return bases[k] + ravel(src, ty[k]->shape);
        });
    }
    if (p == "full") {  // mod.rs:1059-1068
        const std::string& v = attr("fill_value");
        Values one;
        if (is_float(dtype)) {
            one.flt = true;
            one.f = {round_to(attr_value_f(v), dtype)};
        } else if (v[0] == 'f') {
            one.i = {saturate(attr_value_f(v), dtype)};
        } else if (v[0] == 'i') {
            one.i = {wrap((i128)std::stoll(v.substr(2)), dtype)};
        } else {
            one.i = {v[2] == '1'};
        }
        Values filled;  // every element the one value
        filled.flt = one.flt;
        if (one.flt) filled.f.assign(N, one.f[0]);
        else filled.i.assign(N, one.i[0]);
        return filled;
    }
    if (p == "iota") {  // mod.rs:1069-1080
        int64_t d = std::stoll(attr("dimension"));
        Values range;
        range.flt = is_float(dtype);
        for (int64_t k = 0; k < out.shape[d]; k++) {
            if (range.flt) range.f.push_back(round_to((double)k, dtype));
            else range.i.push_back(wrap(k, dtype));
        }
        return gather_by(range, out, [&](const std::vector<int64_t>& idx) { return idx[d]; });
    }
    if (p == "gather") {  // mod.rs:731-749
        const Type &x = *ty[0], &ind = *ty[1];
        int64_t axis = std::stoll(attr("axis"));
        auto picked = taken(*a[1], x.shape[axis]);
        size_t ir = ind.shape.size();
        return gather_by(*a[0], out, [&](const std::vector<int64_t>& idx) {
            std::vector<int64_t> sub(idx.begin() + axis, idx.begin() + axis + ir);
            int64_t k = picked[ravel(sub, ind.shape)];
            std::vector<int64_t> src(idx.begin(), idx.begin() + axis);
            src.push_back(k);
            src.insert(src.end(), idx.begin() + axis + ir, idx.end());
            return ravel(src, x.shape);
        });
    }
    if (p == "scatter_add") {  // mod.rs:765-808
        const Type &x = *ty[0], &ind = *ty[1], &u = *ty[2];
        int64_t axis = std::stoll(attr("axis"));
        auto picked = taken(*a[1], x.shape[axis]);
        size_t ir = ind.shape.size();
        std::vector<int64_t> at;
        for_each_index(u.shape, [&](const std::vector<int64_t>& idx) {
            std::vector<int64_t> sub(idx.begin() + axis, idx.begin() + axis + ir);
            int64_t k = picked[ravel(sub, ind.shape)];
            std::vector<int64_t> src(idx.begin(), idx.begin() + axis);
            src.push_back(k);
            src.insert(src.end(), idx.begin() + axis + ir, idx.end());
            at.push_back(ravel(src, x.shape));
        });
        r = *a[0];
        if (r.flt)
            for (size_t k = 0; k < at.size(); k++) r.f[at[k]] = round_to(r.f[at[k]] + a[2]->f[k], dtype);
        else
            for (size_t k = 0; k < at.size(); k++) r.i[at[k]] = wrap(r.i[at[k]] + a[2]->i[k], dtype);
        return r;
    }
    if (p == "fusion") {  // mod.rs:1122-1125
        return eval_graph(*all.at(std::stoi(attr("body"))), all, a, nullptr);
    }
    if (p == "all_reduce")
        throw std::runtime_error("all_reduce: collectives across processes run in a plan, not the reference interpreter");
    throw std::runtime_error("oracle: unknown primitive " + p);
}

// mod.rs:49-89. Returns output 0; all outputs through `all_outputs` when given.
// Inputs are borrowed (a fusion body reads its operands in place); every other value is owned by `env`.
Values eval_graph(const Graph& g, const std::vector<std::shared_ptr<Graph>>& all, const std::vector<const Values*>& inputs,
                  std::vector<Values>* all_outputs) {
    std::vector<Values> env(g.types.size());
    std::vector<const Values*> at(g.types.size(), nullptr);
    std::vector<std::vector<Values>> extra(g.types.size());
    for (size_t k = 0; k < g.inputs.size(); k++) at[g.inputs[k]] = inputs[k];
    static const bool profile = std::getenv("ORACLE_PROFILE") != nullptr;  // per-primitive wall time on stderr
    for (const Node& n : g.nodes) {
        std::vector<const Values*> args;
        std::vector<const Type*> types;
        for (int v : n.inputs) {
            args.push_back(at[v]);
            types.push_back(&g.types[v]);
        }
        if (n.op == "fusion") {
            const Graph& body = *all.at(std::stoi(n.attrs.at("body")));
            std::vector<Values> outs;
            eval_graph(body, all, args, &outs);
            env[n.output] = std::move(outs[0]);
            for (size_t k = 1; k < outs.size(); k++) extra[n.output].push_back(std::move(outs[k]));
        } else if (n.op == "fusion_output") {
            at[n.output] = &extra[n.inputs[0]].at(std::stoi(n.attrs.at("index")) - 1);  // extra[] is not resized after its fusion
            continue;
        } else if (n.op == "reshape" || n.op == "device_wait" || n.op == "host_wait") {
            at[n.output] = at[n.inputs[0]];  // same values (mod.rs:974): no copy
            continue;
        } else {
            const double t0 = profile ? omp_get_wtime() : 0.0;
            env[n.output] = eval(n, args, types, g.types[n.output], all);
            if (profile) fprintf(stderr, "oracle %-18s %10lld elements %8.3f s\n", n.op.c_str(), (long long)g.types[n.output].numel(), omp_get_wtime() - t0);
        }
        at[n.output] = &env[n.output];
    }
    if (all_outputs) {
        all_outputs->clear();
        for (int v : g.outputs) all_outputs->push_back(*at[v]);
    }
    return g.outputs.empty() ? Values() : *at[g.outputs[0]];
}

// ---- raw buffers <-> Values (mod.rs:91-163) -----------------------------------------------------------------
double half_bits_to_double(uint16_t h) {
    int s = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    double v = e == 0 ? std::ldexp((double)m, -24) : e == 31 ? (m ? NAN : INFINITY) : std::ldexp(1024.0 + m, e - 25);
    return s ? -v : v;
}
uint16_t double_to_half_bits(double x) {  // x is already representable
    if (std::isnan(x)) return 0x7e00;
    uint16_t s = std::signbit(x) ? 0x8000 : 0;
    double a = std::fabs(x);
    if (std::isinf(a)) return s | 0x7c00;
    if (a == 0) return s;
    if (a < 6.103515625e-05) return s | (uint16_t)std::lround(a * 16777216.0);
    int e;
    double m = std::frexp(a, &e);  // a = m 2^e, m in [0.5,1)
    return s | (uint16_t)((e + 14) << 10) | (uint16_t)(std::lround(m * 2048.0) - 1024);
}

Values load(const void* ptr, const Type& t) {
    Values v;
    int64_t n = t.numel();
    v.flt = is_float(t.dtype);
    if (v.flt) v.f.resize(n);
    else v.i.resize(n);
    for (int64_t k = 0; k < n; k++) {
        switch (t.dtype) {
            case BOOL: v.i[k] = ((const uint8_t*)ptr)[k] != 0; break;
            case I8: v.i[k] = ((const int8_t*)ptr)[k]; break;
            case I16: v.i[k] = ((const int16_t*)ptr)[k]; break;
            case I32: v.i[k] = ((const int32_t*)ptr)[k]; break;
            case I64: v.i[k] = ((const int64_t*)ptr)[k]; break;
            case U8: v.i[k] = ((const uint8_t*)ptr)[k]; break;
            case U16: v.i[k] = ((const uint16_t*)ptr)[k]; break;
            case U32: v.i[k] = ((const uint32_t*)ptr)[k]; break;
            case U64: v.i[k] = ((const uint64_t*)ptr)[k]; break;
            case F16: v.f[k] = half_bits_to_double(((const uint16_t*)ptr)[k]); break;
            case BF16: {
                uint32_t b = (uint32_t)((const uint16_t*)ptr)[k] << 16;
                float f;
                memcpy(&f, &b, 4);
                v.f[k] = f;
                break;
            }
            case F32: v.f[k] = ((const float*)ptr)[k]; break;
            case F64: v.f[k] = ((const double*)ptr)[k]; break;
        }
    }
    return v;
}

void store(const Values& v, const Type& t, void* ptr) {
    int64_t n = t.numel();
    for (int64_t k = 0; k < n; k++) {
        switch (t.dtype) {
            case BOOL: ((uint8_t*)ptr)[k] = v.i[k] != 0; break;
            case I8: ((int8_t*)ptr)[k] = (int8_t)v.i[k]; break;
            case I16: ((int16_t*)ptr)[k] = (int16_t)v.i[k]; break;
            case I32: ((int32_t*)ptr)[k] = (int32_t)v.i[k]; break;
            case I64: ((int64_t*)ptr)[k] = (int64_t)v.i[k]; break;
            case U8: ((uint8_t*)ptr)[k] = (uint8_t)v.i[k]; break;
            case U16: ((uint16_t*)ptr)[k] = (uint16_t)v.i[k]; break;
            case U32: ((uint32_t*)ptr)[k] = (uint32_t)v.i[k]; break;
            case U64: ((uint64_t*)ptr)[k] = (uint64_t)v.i[k]; break;
            case F16: ((uint16_t*)ptr)[k] = double_to_half_bits(v.f[k]); break;
            case BF16: {
                float f = (float)v.f[k];
                uint32_t b;
                memcpy(&b, &f, 4);
                ((uint16_t*)ptr)[k] = (uint16_t)(b >> 16);
                break;
            }
            case F32: ((float*)ptr)[k] = (float)v.f[k]; break;
            case F64: ((double*)ptr)[k] = v.f[k]; break;
        }
    }
}

}  // namespace

extern "C" {

// Evaluates the last graph of `text` (mod.rs:17-46). `inputs[k]` / `outputs[k]` are dense row-major buffers of
// the graph's declared input / output types. Returns 0, or 1 with a message in `err`.
int oracle_run(const char* text, int n_inputs, const void** inputs, int n_outputs, void** outputs, char* err,
               int err_len) {
    try {
        auto graphs = parse_graphs(text);
        const Graph& g = *graphs.back();
        if ((int)g.inputs.size() != n_inputs)
            throw std::runtime_error("the graph takes " + std::to_string(g.inputs.size()) + " inputs, got " +
                                     std::to_string(n_inputs));
        if ((int)g.outputs.size() != n_outputs)
            throw std::runtime_error("the graph has " + std::to_string(g.outputs.size()) + " outputs, got " +
                                     std::to_string(n_outputs));
        std::vector<Values> in;
        for (int k = 0; k < n_inputs; k++) in.push_back(load(inputs[k], g.types[g.inputs[k]]));
        std::vector<Values> out;
        std::vector<const Values*> in_ptrs;
        for (const Values& v : in) in_ptrs.push_back(&v);
        eval_graph(g, graphs, in_ptrs, &out);
        for (int k = 0; k < n_outputs; k++) store(out[k], g.types[g.outputs[k]], outputs[k]);
        return 0;
    } catch (const std::exception& e) {
        snprintf(err, err_len, "%s", e.what());
        return 1;
    }
}

// Threads the OpenMP loops above run on (what a timed CPU baseline reports as its core count).
int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Sets the thread count of the loops above (a launcher may have exported OMP_NUM_THREADS=1 for its workers).
void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

// round(x, dtype) of mod.rs:189-200, exposed so tests can pin the rounding on its own.
double oracle_round(double x, const char* dtype) { return round_to(x, parse_dtype(dtype)); }
}
