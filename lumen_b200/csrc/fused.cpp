#include "fused.h"

#include <map>
#include <memory>
#include <mutex>

namespace lb {

static std::mutex g_cache_mutex;
static std::map<std::string, std::unique_ptr<lb_fusion>> g_cache;  // by body text; entries live until exit

static lb_fusion* compile(const std::string& text) {
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    auto it = g_cache.find(text);
    if (it != g_cache.end()) return it->second.get();
    Module module = parse_module(text);
    auto f = std::make_unique<lb_fusion>();
    const Graph& main = module.main();
    bool nothing = !main.outputs.empty();  // every output empty (an empty batch): there is nothing to generate or launch
    for (int v : main.outputs) nothing &= main.type(v).numel() == 0;
    if (nothing) {
        f->kernel.empty = true;
        f->kernel.n_inputs = (int)main.inputs.size(), f->kernel.n_outputs = (int)main.outputs.size();
        for (int v : main.inputs) f->kernel.types.push_back(main.type(v));
        for (int v : main.outputs) f->kernel.types.push_back(main.type(v));
        f->kernel.source = "// no kernel: every output of this fusion is empty\n";
    } else {
        f->kernel = generate_fused(module);
        f->cubin = nvrtc_compile("fused_kernel", f->kernel.source);
    }
    f->scratch_bytes = f->kernel.scratch_bytes;
    lb_fusion* raw = f.get();
    g_cache.emplace(text, std::move(f));
    return raw;
}

static void launch(lb_fusion* f, const lb_tensor* tensors, int n, void* scratch, void* stream) {
    const FusedKernel& k = f->kernel;
    if (k.multi) fail(LB_ERR_INVALID, "this kernel was generated in horizontal form (option multi): launch it with a table of groups");
    if (n != k.n_inputs + k.n_outputs)
        fail(LB_ERR_INVALID, format("fused kernel takes %d inputs and %d outputs, got %d tensors", k.n_inputs,
                                    k.n_outputs, n));
    std::vector<void*> ptrs(n);
    std::vector<void*> params(n);
    for (int i = 0; i < n; i++) {
        check_dense(tensors[i], k.types[i].dtype, k.types[i].shape, i < k.n_inputs ? "fusion input" : "fusion output");
        // vector accesses assume 16-byte aligned tensors (the plan aligns every buffer to 256 bytes)
        if (k.vec > 1 && ((uintptr_t)tensors[i].ptr & 15) != 0)
            fail(LB_ERR_INVALID, format("fusion tensor %d is not 16-byte aligned", i));
        ptrs[i] = tensors[i].ptr;
        params[i] = &ptrs[i];
    }
    if (k.empty || (k.rows == 0 && !k.two_pass)) return;  // empty grid: nothing to launch (lumen/runtime/kernel/cuda/mod.rs:131-133)
    const DeviceInfo& dev = device_info();
    lb_fusion::Loaded fn;
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        lb_fusion::Loaded& slot = f->loaded[dev.device];
        if (!slot.function) {
            slot.function = load_kernel(f->cubin, "fused_kernel");
            if (k.two_pass) slot.finalize = load_kernel(f->cubin, "fused_finalize");
        }
        fn = slot;
    }
    if (k.two_pass) {
        if (k.cols == 0) return;
        if (((uintptr_t)scratch & 15) != 0) fail(LB_ERR_INVALID, "fusion scratch must be 16-byte aligned");
        params.push_back(&scratch);
        check_cu(driver().cuLaunchKernel(fn.function, (unsigned)k.col_blocks, (unsigned)k.slices, 1, (unsigned)k.threads, 1, 1, 0,
                                         (CUstream)stream, params.data(), nullptr),
                 "cuLaunchKernel(fused_kernel)");
        check_cu(driver().cuLaunchKernel(fn.finalize, (unsigned)k.fin_blocks, 1, 1, (unsigned)k.fin_threads, 1, 1, 0, (CUstream)stream,
                                         params.data(), nullptr),
                 "cuLaunchKernel(fused_finalize)");
        return;
    }
    int64_t row_blocks = (k.rows + k.rows_per_block - 1) / k.rows_per_block;
    int per_sm = std::max(1, 2048 / k.threads);
    int64_t grid = std::min<int64_t>(row_blocks, (int64_t)dev.sms * per_sm);
    check_cu(driver().cuLaunchKernel(fn.function, (unsigned)grid, 1, 1, (unsigned)k.threads, 1, 1, 0, (CUstream)stream,
                                     params.data(), nullptr),
             "cuLaunchKernel(fused_kernel)");
}

void launch_fusion(lb_fusion* f, const lb_tensor* tensors, int n, void* scratch, void* stream) { launch(f, tensors, n, scratch, stream); }

void launch_fusion_multi(lb_fusion* f, const lb_tensor* tensors, int n_groups, void* stream) {
    const FusedKernel& k = f->kernel;
    if (!k.multi) fail(LB_ERR_INVALID, "horizontal launch of a kernel that was not generated with option multi");
    const int per = k.n_inputs + k.n_outputs;
    const DeviceInfo& dev = device_info();
    lb_fusion::Loaded fn;
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        lb_fusion::Loaded& slot = f->loaded[dev.device];
        if (!slot.function) slot.function = load_kernel(f->cubin, "fused_kernel");
        fn = slot;
    }
    // the table as the generated source lays it out: { int n; int pad; long long rows[MAX]; void* ptr[MAX][per]; }
    const int max_groups = k.multi_max_groups;
    std::vector<char> table(8 + (size_t)max_groups * 8 + (size_t)max_groups * per * 8);
    for (int first = 0; first < n_groups; first += max_groups) {
        const int count = std::min(max_groups, n_groups - first);
        std::fill(table.begin(), table.end(), 0);
        *(int*)table.data() = count;
        long long* rows = (long long*)(table.data() + 8);
        void** ptrs = (void**)(table.data() + 8 + (size_t)max_groups * 8);
        long long most_blocks = 1;
        for (int g = 0; g < count; g++) {
            const lb_tensor* t = tensors + (size_t)(first + g) * per;
            int64_t n = -1;
            for (int i = 0; i < per; i++) {
                int64_t numel = 1, dense = 1;
                for (int d = t[i].rank - 1; d >= 0; d--) {
                    if (t[i].shape[d] != 1 && t[i].stride[d] != dense) fail(LB_ERR_INVALID, "horizontal launch: tensors must be dense");
                    dense *= t[i].shape[d], numel *= t[i].shape[d];
                }
                if (t[i].dtype != k.types[i].dtype)
                    fail(LB_ERR_INVALID, format("horizontal launch: tensor %d of group %d is %s, the kernel takes %s", i, first + g,
                                                dtype_name(t[i].dtype), dtype_name(k.types[i].dtype)));
                if (k.types[i].rank() == 0) {  // a 0-d operand of the body (a run-time scalar): one element, read as it is
                    if (numel != 1) fail(LB_ERR_INVALID, format("horizontal launch: tensor %d of group %d must hold one element", i, first + g));
                    ptrs[(size_t)g * per + i] = t[i].ptr;
                    continue;
                }
                if (n < 0) n = numel;
                if (numel != n || n % k.cols != 0)
                    fail(LB_ERR_INVALID, format("horizontal launch: the tensors of group %d must share an element count that is a multiple of %lld",
                                                first + g, (long long)k.cols));
                if (k.vec > 1 && ((uintptr_t)t[i].ptr & 15) != 0) fail(LB_ERR_INVALID, "horizontal launch: tensors must be 16-byte aligned");
                ptrs[(size_t)g * per + i] = t[i].ptr;
            }
            rows[g] = n / k.cols;
            most_blocks = std::max<long long>(most_blocks, (rows[g] + k.rows_per_block - 1) / k.rows_per_block);
        }
        const int per_sm = std::max(1, 2048 / k.threads);
        const long long grid = std::min<long long>(most_blocks, (long long)dev.sms * per_sm);
        void* params[1] = {table.data()};
        check_cu(driver().cuLaunchKernel(fn.function, (unsigned)grid, 1, 1, (unsigned)k.threads, 1, 1, 0, (CUstream)stream, params, nullptr),
                 "cuLaunchKernel(fused_kernel, horizontal)");
    }
}
lb_fusion* compile_fusion(const std::string& text) { return compile(text); }

}  // namespace lb

extern "C" {

int lb_fusion_compile(const char* body_text, lb_fusion** out) {
    return lb::guarded([&] {
        if (!body_text || !out) lb::fail(LB_ERR_INVALID, "lb_fusion_compile: null argument");
        *out = lb::compile(body_text);
    });
}
int lb_fusion_check(const char* body_text) {
    return lb::guarded([&] {
        if (!body_text) lb::fail(LB_ERR_INVALID, "lb_fusion_check: null argument");
        lb::generate_fused(lb::parse_module(body_text));  // throws what lb_fusion_compile would; no NVRTC, nothing cached
    });
}
int lb_fusion_num_inputs(const lb_fusion* f) { return f ? f->kernel.n_inputs : -1; }
int lb_fusion_num_outputs(const lb_fusion* f) { return f ? f->kernel.n_outputs : -1; }
const char* lb_fusion_source(const lb_fusion* f) { return f ? f->kernel.source.c_str() : ""; }
size_t lb_fusion_scratch_bytes(const lb_fusion* f) { return f ? f->scratch_bytes : 0; }

int lb_fusion_launch(const lb_fusion* f, const lb_tensor* tensors, int n_tensors, void* scratch, void* stream) {
    return lb::guarded([&] {
        if (!f || (!tensors && n_tensors)) lb::fail(LB_ERR_INVALID, "lb_fusion_launch: null argument");
        if (f->scratch_bytes && !scratch) lb::fail(LB_ERR_INVALID, "lb_fusion_launch: this fusion needs scratch memory");
        lb::launch(const_cast<lb_fusion*>(f), tensors, n_tensors, scratch, stream);
    });
}

int lb_fusion_launch_groups(const lb_fusion* f, const lb_tensor* tensors, int n_groups, void* stream) {
    return lb::guarded([&] {
        if (!f || (!tensors && n_groups)) lb::fail(LB_ERR_INVALID, "lb_fusion_launch_groups: null argument");
        lb::launch_fusion_multi(const_cast<lb_fusion*>(f), tensors, n_groups, stream);
    });
}

int lb_launch_fused(const char* body_text, const lb_tensor* tensors, int n_inputs, int n_outputs, void* stream) {
    return lb::guarded([&] {
        if (!body_text) lb::fail(LB_ERR_INVALID, "lb_launch_fused: null body");
        lb_fusion* f = lb::compile(body_text);
        if (f->scratch_bytes) lb::fail(LB_ERR_UNSUPPORTED, "lb_launch_fused: this fusion needs scratch memory; use lb_fusion_launch");
        if (n_inputs != f->kernel.n_inputs || n_outputs != f->kernel.n_outputs)
            lb::fail(LB_ERR_INVALID, lb::format("the fusion takes %d inputs and %d outputs, got %d and %d",
                                                f->kernel.n_inputs, f->kernel.n_outputs, n_inputs, n_outputs));
        lb::launch(f, tensors, n_inputs + n_outputs, nullptr, stream);
    });
}
}
