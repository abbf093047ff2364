// CUDA glue for generated kernels: driver entry points resolved through the runtime (the library links no
// libcuda, so it loads on machines without a driver), NVRTC compilation to sm_100a cubins, and a process-wide
// module cache. Plays the role of the reference's driver.rs (lumen/runtime/kernel/cuda/driver.rs:134-294).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <string>

#include "common.h"

namespace lb {

#define LB_CUDA(expr)                                                                                     \
    do {                                                                                                  \
        cudaError_t err__ = (expr);                                                                       \
        if (err__ != cudaSuccess)                                                                         \
            ::lb::fail(LB_ERR_CUDA, ::lb::format("%s: %s (%s:%d)", #expr, cudaGetErrorString(err__), __FILE__, \
                                                 __LINE__));                                              \
    } while (0)

struct Driver {
    CUresult (*cuModuleLoadData)(CUmodule*, const void*);
    CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*);
    CUresult (*cuLaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                               CUstream, void**, void**);
    CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int);
    CUresult (*cuGetErrorString)(CUresult, const char**);
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
};

// Resolves the driver entry points on first use; throws LB_ERR_CUDA when no driver/GPU is usable.
const Driver& driver();
void check_cu(CUresult r, const char* what);

struct DeviceInfo {
    int device = 0;
    int sms = 0;
    int cc_major = 0, cc_minor = 0;
};
// Properties of the current device (cached per device); throws unless it is compute capability 10.x.
const DeviceInfo& device_info();

// Device word kernels set (to LB_ERR_TIMEOUT) when a bounded wait gives up; allocated once per device, on first use
// with that device current.
int* status_word();
// Adds `word` (device memory of the current device, e.g. a __device__ variable's address) to the words that
// read_status() reads for this device.
void register_status_word(int* word);
// Synchronises the current device, then reads and clears every status word registered for it; the first non-zero
// value, else 0. Allocates nothing.
int read_status();
// True the first time it is called with `key` while this device is current: one-time set-up per (device, kernel),
// such as cudaFuncSetAttribute, which applies to the current device only.
bool first_use_on_device(const void* key);
// What an autotuner (or a caller) may fix for one GEMM instead of the built-in choices; 0 = choose.
struct GemmTuning {
    int splits = 0;   // K ranges (needs scratch for that many float32 partial tiles)
    int group_m = 0;  // rows of tiles walked together before moving along N (L2 reuse of the B operand)
};

// SM count of the current device, or a B200's 148 where no device is usable (plan lowering on a CPU-only machine).
int sm_count_hint();

// Compiles CUDA C++ `source` for sm_100a and returns the cubin. `name` labels diagnostics.
std::string nvrtc_compile(const std::string& name, const std::string& source);
// Loads a cubin into the current context and returns `kernel`'s function handle (modules live until exit).
CUfunction load_kernel(const std::string& cubin, const char* kernel);

}  // namespace lb
