// Fused elementwise / reduction / row kernels: generation (fused_codegen.cpp), compilation cache and launch.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "device.h"
#include "graph_text.h"

namespace lb {

struct FusedKernel {
    std::string source;
    int64_t rows = 0, cols = 0;
    int threads = 0, rows_per_block = 1, vec = 1;
    int n_inputs = 0, n_outputs = 0;
    std::vector<TensorType> types;  // inputs then outputs
    // column reductions: a partial-sum pass over (col_blocks x slices) blocks, then a finalize pass; both take a
    // trailing scratch pointer of scratch_bytes
    bool two_pass = false;
    int slices = 1;
    int64_t col_blocks = 1;
    int fin_threads = 128;
    int64_t fin_blocks = 1;
    size_t scratch_bytes = 0;
    // horizontal form (module option `multi`): the kernel takes a table of tensor groups by value; the body's own
    // shape [rows, cols] only fixes `cols`, every group brings its row count
    bool multi = false;
    int multi_max_groups = 0;
    bool empty = false;  // every output has zero elements: no kernel was generated, a launch does nothing
};

// Generates the kernel for the main graph of `module` (a fusion body). Throws LB_ERR_UNSUPPORTED naming the
// primitive or layout there is no rule for.
FusedKernel generate_fused(const Module& module);

}  // namespace lb

struct lb_fusion;
namespace lb {
lb_fusion* compile_fusion(const std::string& text);
void launch_fusion(lb_fusion* f, const lb_tensor* tensors, int n, void* scratch, void* stream);
// Horizontal launch of a kernel compiled with `option multi`: `tensors` holds n_groups * (inputs + outputs) dense
// tensors, group after group; every tensor of a group has the same number of elements, a multiple of the kernel's
// column count.
void launch_fusion_multi(lb_fusion* f, const lb_tensor* tensors, int n_groups, void* stream);
}

struct lb_fusion {
    lb::FusedKernel kernel;
    struct Loaded {
        CUfunction function = nullptr, finalize = nullptr;
    };
    std::map<int, Loaded> loaded;  // by device ordinal: the cubin is loaded into a device's context on its first launch there
    std::string cubin;
    size_t scratch_bytes = 0;
};
