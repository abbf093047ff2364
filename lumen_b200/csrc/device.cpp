#include "device.h"

#include <nvrtc.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <vector>

namespace lb {

static std::mutex g_mutex;

const Driver& driver() {
    static Driver d;
    static bool ready = false;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (ready) return d;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0)
        fail(LB_ERR_CUDA, format("no usable CUDA device (%s): this backend has no CPU fallback",
                                 err == cudaSuccess ? "0 devices" : cudaGetErrorString(err)));
    LB_CUDA(cudaFree(nullptr));  // make sure the primary context exists
    auto get = [](const char* symbol, void** fn) {
        cudaDriverEntryPointQueryResult status;
        cudaError_t e = cudaGetDriverEntryPoint(symbol, fn, cudaEnableDefault, &status);
        if (e != cudaSuccess || status != cudaDriverEntryPointSuccess || *fn == nullptr)
            fail(LB_ERR_CUDA, format("driver entry point %s is unavailable", symbol));
    };
    get("cuModuleLoadData", (void**)&d.cuModuleLoadData);
    get("cuModuleGetFunction", (void**)&d.cuModuleGetFunction);
    get("cuLaunchKernel", (void**)&d.cuLaunchKernel);
    get("cuFuncSetAttribute", (void**)&d.cuFuncSetAttribute);
    get("cuGetErrorString", (void**)&d.cuGetErrorString);
    get("cuTensorMapEncodeTiled", (void**)&d.cuTensorMapEncodeTiled);
    ready = true;
    return d;
}

void check_cu(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return;
    const char* text = nullptr;
    driver().cuGetErrorString(r, &text);
    fail(LB_ERR_CUDA, format("%s: %s (CUresult %d)", what, text ? text : "unknown error", (int)r));
}

const DeviceInfo& device_info() {
    static std::map<int, DeviceInfo> cache;
    driver();  // fails with a clear message when there is no usable device
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    DeviceInfo info;
    info.device = dev;
    LB_CUDA(cudaDeviceGetAttribute(&info.sms, cudaDevAttrMultiProcessorCount, dev));
    LB_CUDA(cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    LB_CUDA(cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (info.cc_major != 10)
        fail(LB_ERR_CUDA, format("device %d is sm_%d%d: this backend is built for sm_100a (B200) only", dev,
                                 info.cc_major, info.cc_minor));
    return cache[dev] = info;
}

// Status words by device ordinal. A kernel raises the word of the device it runs on; lb_device_status() reads every word
// registered for the current device. The first entry of a device's list is the word status_word() allocated.
static std::map<int, std::vector<int*>> g_status_words;
static std::map<int, bool> g_has_main_word;

static int current_device() {
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    return dev;
}

int* status_word() {
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(g_mutex);
    auto& words = g_status_words[dev];
    if (!g_has_main_word[dev]) {
        int* word = nullptr;
        LB_CUDA(cudaMalloc(&word, sizeof(int)));
        LB_CUDA(cudaMemset(word, 0, sizeof(int)));
        words.insert(words.begin(), word);
        g_has_main_word[dev] = true;
    }
    return words.front();
}

void register_status_word(int* word) {
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(g_mutex);
    auto& words = g_status_words[dev];
    for (int* w : words)
        if (w == word) return;
    words.push_back(word);
}

int read_status() {
    const int dev = current_device();
    std::vector<int*> words;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        words = g_status_words[dev];
    }
    LB_CUDA(cudaDeviceSynchronize());
    int result = 0;
    for (int* word : words) {  // plain copies: nothing here allocates
        int host = 0;
        LB_CUDA(cudaMemcpy(&host, word, sizeof(int), cudaMemcpyDeviceToHost));
        if (host != 0) {
            LB_CUDA(cudaMemset(word, 0, sizeof(int)));
            if (result == 0) result = host;
        }
    }
    return result;
}

bool first_use_on_device(const void* key) {
    static std::set<std::pair<int, const void*>> seen;
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(g_mutex);
    return seen.emplace(dev, key).second;
}

int sm_count_hint() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return 148;  // a B200's; used when lowering a plan on a machine without a GPU
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        cudaGetLastError();
        return 148;
    }
    return sms;
}

std::string nvrtc_compile(const std::string& name, const std::string& source) {
    nvrtcProgram prog;
    if (nvrtcCreateProgram(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr) != NVRTC_SUCCESS)
        fail(LB_ERR_CUDA, "nvrtcCreateProgram failed");
    // --fmad=false: every multiply and add is rounded on its own, as the reference interpreter rounds after each
    // primitive (its CUDA emitter spells explicit-rounding adds/multiplies, lumen/codegen/emitter/cuda.rs:72-93).
    // LUMEN_B200_PTXAS_VERBOSE=1: registers, spills and shared memory of every generated kernel on stderr
    static const bool verbose = getenv("LUMEN_B200_PTXAS_VERBOSE") != nullptr;
    std::vector<const char*> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", "-default-device",
                                     "--prec-div=true",            "--prec-sqrt=true", "--ftz=false"};
    if (verbose) opts.push_back("--ptxas-options=-v");
    nvrtcResult rc = nvrtcCompileProgram(prog, (int)opts.size(), opts.data());
    if (rc != NVRTC_SUCCESS) {
        size_t n = 0;
        nvrtcGetProgramLogSize(prog, &n);
        std::string log(n, '\0');
        nvrtcGetProgramLog(prog, log.data());
        nvrtcDestroyProgram(&prog);
        fail(LB_ERR_CUDA, "NVRTC failed for " + name + ":\n" + log);
    }
    if (verbose) {
        size_t ln = 0;
        nvrtcGetProgramLogSize(prog, &ln);
        std::string log(ln, '\0');
        nvrtcGetProgramLog(prog, log.data());
        fprintf(stderr, "[lumen_b200] %s: %s\n", name.c_str(), log.c_str());
    }
    size_t n = 0;
    nvrtcGetCUBINSize(prog, &n);
    std::string cubin(n, '\0');
    nvrtcGetCUBIN(prog, cubin.data());
    nvrtcDestroyProgram(&prog);
    if (n == 0) fail(LB_ERR_CUDA, "NVRTC produced no cubin for " + name);
    return cubin;
}

CUfunction load_kernel(const std::string& cubin, const char* kernel) {
    const Driver& d = driver();
    CUmodule module;
    check_cu(d.cuModuleLoadData(&module, cubin.data()), "cuModuleLoadData");
    CUfunction fn;
    check_cu(d.cuModuleGetFunction(&fn, module, kernel), "cuModuleGetFunction");
    return fn;
}

}  // namespace lb
