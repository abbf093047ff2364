// A diagnostic entry that exercises the wind-down path of the bounded device waits without any fault: one CTA waits
// on a barrier nobody arrives on, with a SHORT budget given by the caller, gives up, raises the status word and
// returns normally. The context stays usable; lb_device_status() then reports LB_ERR_TIMEOUT once and clears.
#include "device.h"
#include "sm100.cuh"

namespace lb {
int* static_status_word();

namespace {
__global__ void wait_timeout_kernel(long long budget, int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        sm100::mbar_init(&bar, 1);
        sm100::fence_barrier_init();
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = sm100::mbar_wait(&bar, 0, &abort_flag, budget);  // phase 0 never completes
    __syncthreads();
    // every role of a real kernel leaves its loops when the abort flag is up; here the other lanes just observe it
    if (threadIdx.x == 0 && (!ok || abort_flag)) atomicExch(status, LB_ERR_TIMEOUT);
}
}  // namespace
}  // namespace lb

extern "C" int lb_debug_wait_timeout(long long cycles, int static_word, void* stream) {
    return lb::guarded([&] {
        if (cycles <= 0 || cycles > 100000000LL)
            lb::fail(LB_ERR_INVALID, "lb_debug_wait_timeout: the budget must be between 1 and 100,000,000 cycles (a fraction of a second)");
        lb::device_info();
        int* word = static_word ? lb::static_status_word() : lb::status_word();
        lb::wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(cycles, word);
        LB_CUDA(cudaGetLastError());
    });
}
