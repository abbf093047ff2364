#include "common.h"

#include <cstring>

namespace lb {

static thread_local std::string g_last_error;

void set_last_error(const std::string& message) { g_last_error = message; }

std::string format(const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return buf;
}

static const char* kNames[] = {"bool",   "int8",   "int16",   "int32",    "int64",   "uint8",  "uint16",
                               "uint32", "uint64", "float16", "bfloat16", "float32", "float64"};
static const int kSizes[] = {1, 1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};

const char* dtype_name(int d) { return (d >= 0 && d <= LB_F64) ? kNames[d] : "?"; }
int dtype_size(int d) {
    if (d < 0 || d > LB_F64) fail(LB_ERR_INVALID, format("unknown dtype code %d", d));
    return kSizes[d];
}
int dtype_from_name(const std::string& name) {
    for (int d = 0; d <= LB_F64; d++)
        if (name == kNames[d]) return d;
    fail(LB_ERR_INVALID, "unknown dtype " + name);
}

int64_t numel(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
}

void check_dense(const lb_tensor& t, int dtype, const std::vector<int64_t>& shape, const char* what) {
    auto describe = [&]() {
        std::string s = format("%s: expected dense %s[", what, dtype_name(dtype));
        for (size_t d = 0; d < shape.size(); d++) s += (d ? "," : "") + std::to_string(shape[d]);
        s += format("], got %s[", dtype_name(t.dtype));
        for (int d = 0; d < t.rank; d++) s += (d ? "," : "") + std::to_string(t.shape[d]);
        s += "] strides [";
        for (int d = 0; d < t.rank; d++) s += (d ? "," : "") + std::to_string(t.stride[d]);
        return s + "]";
    };
    if (t.dtype != dtype || t.rank != (int)shape.size()) fail(LB_ERR_INVALID, describe());
    int64_t stride = 1;
    for (int d = t.rank - 1; d >= 0; d--) {
        if (t.shape[d] != shape[d] || (t.shape[d] > 1 && t.stride[d] != stride)) fail(LB_ERR_INVALID, describe());
        stride *= shape[d];
    }
    if (numel(shape) > 0 && t.ptr == nullptr) fail(LB_ERR_INVALID, std::string(what) + ": null data pointer");
}

}  // namespace lb

extern "C" const char* lb_last_error(void) { return lb::g_last_error.c_str(); }
extern "C" const char* lb_version(void) { return "lumen_b200 0.1 sm_100a (CUDA 12.9, NVRTC fused kernels, tcgen05 GEMM/attention)"; }
