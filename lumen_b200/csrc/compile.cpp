// lb_compile: the backend's own lowering of a fused graph to a plan, the counterpart of the reference's device target
// `Cuda::lower(module, device) -> Result<Box<dyn Plan>, String>` (lumen/graph_compiler/device.rs:88-112,
// lumen/codegen/devices/cuda/mod.rs:140-189): it takes the module AFTER the pass pipeline - a main graph whose work
// sits in `fusion` nodes - and gives every fusion a step, every value a place and the plan its workspace size. A node
// it has no kernel for is rejected with a message naming the primitive, as the reference's lowering does.
//
// Intermediates share the workspace by live range (first fit, largest first); outputs may be written into donated
// inputs; all-reduced gradients lie side by side in an arena at the start of the workspace and are reduced in buckets by
// `all_reduce` / `wait` steps; runs of same-bodied elementwise steps become one horizontally fused launch; a
// concatenation copies its operands into place. lumen_b200/compiler.py is the same lowering on the Python side (it also
// produces concatenations in place) and emits the same plan text for lb_plan_create; both end in the same run loop.
#include <algorithm>
#include <cstring>
#include <map>
#include <numeric>
#include <set>
#include <sstream>

#include "device.h"
#include "fused.h"
#include "graph_text.h"

extern "C" size_t lb_gemm_scratch_bytes(int64_t m, int64_t n, int64_t k, int64_t batch);

namespace lb {
namespace {

constexpr size_t kAlign = 256;

struct View {
    std::string base;  // "w", "i<k>" or "o<k>"
    int buffer = -1;    // base "w": the workspace buffer the view lies in
    size_t offset = 0;  // bytes from the base (from the start of the buffer for base "w")
    int dtype = LB_F32;
    std::vector<int64_t> shape, strides;  // strides in elements
    bool dense() const {
        int64_t expect = 1;
        for (int d = (int)shape.size() - 1; d >= 0; d--) {
            if (shape[d] != 1 && strides[d] != expect) return false;
            expect *= shape[d];
        }
        return true;
    }
};

std::vector<int64_t> dense_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> s(shape.size(), 1);
    for (int d = (int)shape.size() - 2; d >= 0; d--) s[d] = s[d + 1] * shape[d + 1];
    return s;
}

// Strides of `new_shape` over the same memory, or false when the reshape would need a copy (NumPy's no-copy rule):
// runs of old dimensions that are contiguous among themselves are regrouped into the new dimensions they cover.
bool reshape_strides(const std::vector<int64_t>& shape, const std::vector<int64_t>& strides, const std::vector<int64_t>& new_shape,
                     std::vector<int64_t>* out) {
    std::vector<std::pair<int64_t, int64_t>> old;
    for (size_t d = 0; d < shape.size(); d++)
        if (shape[d] != 1) old.push_back({shape[d], strides[d]});
    out->assign(new_shape.size(), 0);
    size_t oi = 0, ni = 0;
    while (ni < new_shape.size()) {
        if (new_shape[ni] == 1) {
            (*out)[ni++] = 1;
            continue;
        }
        if (oi >= old.size()) return false;
        int64_t chunk = old[oi].first, last_stride = old[oi].second, size_new = new_shape[ni];
        size_t oj = oi + 1, nj = ni;
        while (size_new != chunk) {
            if (size_new < chunk) {
                nj++;
                while (nj < new_shape.size() && new_shape[nj] == 1) nj++;
                if (nj >= new_shape.size()) return false;
                size_new *= new_shape[nj];
            } else {
                if (oj >= old.size() || old[oj].second * old[oj].first != last_stride) return false;
                chunk *= old[oj].first, last_stride = old[oj].second, oj++;
            }
        }
        int64_t stride = last_stride;
        for (size_t k = nj + 1; k-- > ni;) {
            if (new_shape[k] == 1) {
                (*out)[k] = 1;
                continue;
            }
            (*out)[k] = stride;
            stride *= new_shape[k];
        }
        oi = oj, ni = nj + 1;
    }
    return oi >= old.size();
}

// The `graph k ... end` blocks of a module text, in order.
std::vector<std::string> graph_blocks(const std::string& text) {
    std::vector<std::string> blocks;
    std::istringstream in(text);
    std::string line, cur;
    bool inside = false;
    while (std::getline(in, line)) {
        if (line.rfind("graph ", 0) == 0) inside = true, cur = "graph 0\n";
        else if (inside) {
            cur += line + "\n";
            if (line == "end") blocks.push_back(cur), inside = false;
        }
    }
    return blocks;
}

struct Lowering {
    const Module& module;
    const Graph& g;
    std::vector<std::string> blocks;
    bool deterministic;
    std::map<int, View> views;              // value -> where it lives
    std::map<int, int> output_slot;         // value -> index among the graph's outputs
    std::map<std::string, int> module_ids;  // fusion body text -> module index
    std::vector<std::string> modules;
    // what a generated-kernel step is made of: input to the horizontal fusion
    struct Generated {
        const Graph* body = nullptr;
        std::string label;
        bool inplace = false, scratch = false;
        std::vector<int> ids;  // tensor ids: inputs then outputs
    };
    struct Step {
        std::string line;
        std::vector<int> tensor_ids;  // every tensor the step names: its buffers are live at the step
        bool is_generated = false;
        Generated gen;
    };
    std::vector<Step> steps;
    std::vector<int> pending;   // tensors named since the last step was appended: they belong to the next one
    std::vector<View> tensors;  // by tensor id
    // a workspace buffer with the first and last step that name it: buffers whose step ranges do not meet share memory.
    // All-reduced gradients live in the arena at the start of the workspace, in order of production, to the end.
    struct Buffer {
        size_t bytes = 0, place = 0;
        int first = 1 << 30, last = -1;
        bool arena = false, pinned_end = false;
    };
    std::vector<Buffer> buffers;
    std::set<int> reduced_values;  // operands of all_reduce nodes
    std::set<int> zero_tables;     // zero-filled values read only as the table of scatter_add nodes: never materialised
    struct Comm {
        int ready = 0;  // the collective is queued before this step
        View view;
        int op = 0;
    };
    std::vector<Comm> comms;
    long long bucket_bytes = 64LL << 20;
    size_t arena_bytes = 0;
    int num_buckets = 0;

    std::map<int, int> donate;  // output index -> input index whose memory the output is written into
    // attention gradients that only feed a last-axis concatenation are produced directly inside the concatenation's
    // buffer: value -> (concatenation, column offset in elements, columns of its slot)
    struct Slot {
        int cat;
        int64_t col, width;
    };
    std::map<int, Slot> placed;
    std::map<int, View> concat_views;  // concatenation value -> its dense storage, made when its first operand is

    Lowering(const Module& m, const std::string& text, bool det) : module(m), g(m.main()), blocks(graph_blocks(text)), deterministic(det) {}

    View concat_storage(int cat) {
        auto it = concat_views.find(cat);
        if (it != concat_views.end()) return it->second;
        const TensorType& ct = g.type(cat);
        return concat_views[cat] = fresh(ct.dtype, ct.shape, cat);
    }

    View fresh(int dtype, const std::vector<int64_t>& shape, int value = -1) {
        auto slot_in_cat = value >= 0 ? placed.find(value) : placed.end();
        if (slot_in_cat != placed.end()) {
            // rows of `width` columns at column `col` of the concatenation's rows, seen in the value's own shape
            const Slot& at = slot_in_cat->second;
            View v = concat_storage(at.cat);
            const int64_t row = g.type(at.cat).shape.back(), rows = numel(shape) / at.width;
            std::vector<int64_t> strides;
            if (!reshape_strides({rows, at.width}, {row, 1}, shape, &strides)) fail(LB_ERR_INVALID, "lb_compile: a concatenation slot that does not hold its operand's shape");
            v.offset += (size_t)at.col * dtype_size(dtype);
            v.dtype = dtype, v.shape = shape, v.strides = strides;
            return v;
        }
        View v;
        v.dtype = dtype, v.shape = shape, v.strides = dense_strides(shape);
        auto slot = value >= 0 ? output_slot.find(value) : output_slot.end();
        if (slot != output_slot.end()) {
            auto given = donate.find(slot->second);  // a graph output is produced in place: in its own buffer, or in a donated input's
            v.base = given != donate.end() ? "i" + std::to_string(given->second) : "o" + std::to_string(slot->second);
        } else {
            size_t bytes = (size_t)numel(shape) * dtype_size(dtype);
            Buffer b;
            b.bytes = (std::max<size_t>(bytes, 1) + kAlign - 1) / kAlign * kAlign;
            b.arena = value >= 0 && reduced_values.count(value) != 0;
            v.base = "w", v.buffer = (int)buffers.size(), v.offset = 0;
            buffers.push_back(b);
        }
        return v;
    }
    View scratch(size_t bytes) { return fresh(LB_U8, {(int64_t)bytes}); }

    // The id of `v` as an operand of the step being built (the one appended next).
    int tid(const View& v) {
        tensors.push_back(v);
        pending.push_back((int)tensors.size() - 1);
        return (int)tensors.size() - 1;
    }
    void push_step(const std::string& line) {
        Step st;
        st.line = line, st.tensor_ids = pending;
        pending.clear();
        steps.push_back(st);
    }
    // The arena first: all-reduced gradients side by side in order of production (what the buckets are cut from).
    void place_arena() {
        size_t at = 0;
        for (Buffer& b : buffers)
            if (b.arena) b.place = at, at += b.bytes;
        arena_bytes = at;
    }
    // Live ranges from the final step list, then first fit above the arena, largest buffers first: a buffer goes to the
    // lowest offset where it meets no placed buffer that is live at one of its steps. Returns the workspace size.
    size_t place() {
        for (Buffer& b : buffers) b.first = 1 << 30, b.last = -1;
        for (size_t k = 0; k < steps.size(); k++)
            for (int id : steps[k].tensor_ids) {
                const View& v = tensors[(size_t)id];
                if (v.buffer < 0) continue;
                Buffer& b = buffers[(size_t)v.buffer];
                b.first = std::min(b.first, (int)k), b.last = std::max(b.last, (int)k);
            }
        for (Buffer& b : buffers)
            if ((b.arena || b.pinned_end) && b.last >= 0) b.last = (int)steps.size();
        std::vector<int> order;
        for (size_t k = 0; k < buffers.size(); k++)
            if (!buffers[k].arena) order.push_back((int)k);
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return buffers[(size_t)x].bytes > buffers[(size_t)y].bytes; });
        std::vector<int> placed;
        size_t top = arena_bytes;
        for (int id : order) {
            Buffer& b = buffers[(size_t)id];
            if (b.last < 0) continue;  // never an operand of a step
            std::vector<std::pair<size_t, size_t>> spans;
            for (int other : placed) {
                const Buffer& p = buffers[(size_t)other];
                if (!(p.last < b.first || b.last < p.first)) spans.push_back({p.place, p.place + p.bytes});
            }
            std::sort(spans.begin(), spans.end());
            size_t at = arena_bytes;
            for (const auto& span : spans) {
                if (at + b.bytes <= span.first) break;
                at = std::max(at, span.second);
            }
            b.place = at;
            placed.push_back(id);
            top = std::max(top, at + b.bytes);
        }
        return top;
    }
    int module_id(const std::string& text) {
        auto it = module_ids.find(text);
        if (it != module_ids.end()) return it->second;
        modules.push_back(text);
        return module_ids[text] = (int)modules.size() - 1;
    }
    const View& view_of(int value, const char* what) {
        auto it = views.find(value);
        if (it == views.end()) fail(LB_ERR_INVALID, format("lb_compile: %s reads value %%%d before it is produced", what, value));
        return it->second;
    }

    // outputs of a fusion node: its own value (body output 0) and its fusion_output nodes' values by index
    std::vector<int> fusion_outputs(const Node& n, const Graph& body) {
        std::vector<int> outs(body.outputs.size(), -1);
        outs[0] = n.output;
        for (const Node& u : g.nodes)
            if (u.op == "fusion_output" && u.inputs.at(0) == n.output) outs.at((size_t)u.integer("index")) = u.output;
        return outs;
    }

    // scale, causal flag and causal shift of a traced attention body: the constant that multiplies the scores and the
    // shift added to the query index of the iota comparison
    void attention_params(const Graph& body, double* scale, int* causal, long long* offset) {
        *scale = 1.0, *causal = 0, *offset = 0;
        std::map<int, std::string> consts;
        std::map<int, int> bcast;
        std::set<int> dots;
        for (const Node& n : body.nodes) {
            if (n.op == "dot_general") dots.insert(n.output);
            if (n.op == "full") consts[n.output] = n.attr("fill_value");
            if (n.op == "broadcast_in_dim") bcast[n.output] = n.inputs.at(0);
        }
        auto const_of = [&](int v) -> const std::string* {
            auto b = bcast.find(v);
            if (b != bcast.end()) v = b->second;
            auto c = consts.find(v);
            return c == consts.end() ? nullptr : &c->second;
        };
        bool have_scale = false;
        for (const Node& n : body.nodes) {
            if (n.op == "mul" && !have_scale) {
                bool on_scores = false;
                for (int i : n.inputs) on_scores |= dots.count(i) != 0;
                if (on_scores)
                    for (int i : n.inputs) {
                        const std::string* c = dots.count(i) ? nullptr : const_of(i);
                        if (c && c->rfind("f:", 0) == 0) *scale = std::strtod(c->c_str() + 2, nullptr), have_scale = true;
                    }
            }
            if (n.op == "iota") *causal = 1;
            if (n.op == "add" && *causal && body.type(n.output).dtype == LB_I64)
                for (int i : n.inputs) {
                    const std::string* c = const_of(i);
                    if (c && c->rfind("i:", 0) == 0) *offset = std::strtoll(c->c_str() + 2, nullptr, 10);
                }
        }
    }

    // The view of `value` when it is dense, else a dense copy made once: by a `transpose` step for the transposed view of
    // a dense matrix, which is what transposed weights and cotangents are, by a `copy` step for any other view.
    View dense_operand(int value, const std::string& label) {
        const View in = view_of(value, label.c_str());
        if (in.dense() && in.offset % 16 == 0) return in;
        if (in.dense()) {
            // a slice that starts inside a 16-byte line (rows of 24 bytes, from row 1): generated kernels load whole
            // lines, so the slice is copied to an aligned place first
            View copy = fresh(in.dtype, in.shape);
            push_step("s copy materialize_view " + std::to_string(tid(in)) + " " + std::to_string(tid(copy)) + "\n");
            views[value] = copy;
            return copy;
        }
        std::vector<std::pair<int64_t, int64_t>> live;
        for (size_t d = 0; d < in.shape.size(); d++)
            if (in.shape[d] != 1) live.push_back({in.shape[d], in.strides[d]});
        const int size = dtype_size(in.dtype);
        if (live.size() != 2 || live[0].second != 1 || live[1].second != live[0].first || (size != 2 && size != 4)) {
            // any other view (a slice, a permutation of more axes): a dense copy made by the copy step's strided kernel
            View copy = fresh(in.dtype, in.shape);
            push_step("s copy materialize_view " + std::to_string(tid(in)) + " " + std::to_string(tid(copy)) + "\n");
            views[value] = copy;
            return copy;
        }
        const int64_t rows = live[1].first, cols = live[0].first;  // the memory is a dense [rows, cols]; the value is its transpose
        View src = in, copy = fresh(in.dtype, {cols, rows});
        src.shape = {rows, cols}, src.strides = {cols, 1};
        push_step("s transpose materialize_transpose " + std::to_string(tid(src)) + " " + std::to_string(tid(copy)) + "\n");
        copy.shape = in.shape, copy.strides = dense_strides(in.shape);
        views[value] = copy;  // later readers use the copy too
        return copy;
    }

    void lower_generated(const Node& n, const Graph& body, int body_index, const std::string& label) {
        std::vector<View> dense_inputs;
        for (int v : n.inputs) dense_inputs.push_back(dense_operand(v, label));  // may add transpose steps: before this step's operands are listed
        // an output written into a donated input that the kernel also reads: the kernel is generated without the
        // read-only / no-alias promises on its pointers
        std::vector<int> outs_here = fusion_outputs(n, body);
        bool inplace = false;
        for (int o : outs_here) {
            auto slot = o >= 0 ? output_slot.find(o) : output_slot.end();
            auto given = slot != output_slot.end() ? donate.find(slot->second) : donate.end();
            if (given == donate.end()) continue;
            const std::string base = "i" + std::to_string(given->second);
            for (const View& in : dense_inputs) inplace |= in.base == base;
        }
        bool nothing = true;  // every output empty (an empty batch): no kernel, no step, as the reference skips a zero-size grid
        for (size_t k = 0; k < outs_here.size(); k++) nothing &= body.type(body.outputs[k]).numel() == 0;
        if (nothing) {
            for (size_t k = 0; k < outs_here.size(); k++)
                if (outs_here[k] >= 0) views[outs_here[k]] = fresh(body.type(body.outputs[k]).dtype, body.type(body.outputs[k]).shape, outs_here[k]);
            return;
        }
        const int m = module_id((inplace ? "option inplace\n" : "") + blocks.at((size_t)body_index));
        lb_fusion* f = compile_fusion(modules[(size_t)m]);  // rejects what the generator has no rule for, naming the primitive
        std::vector<int> ids;
        for (const View& in : dense_inputs) {
            ids.push_back(tid(in));
        }
        const std::vector<int>& outs = outs_here;
        for (size_t k = 0; k < outs.size(); k++) {
            const TensorType& t = body.type(body.outputs[k]);
            View o = fresh(t.dtype, t.shape, outs[k]);
            if (outs[k] >= 0) views[outs[k]] = o;
            ids.push_back(tid(o));
        }
        int scratch_id = -1;
        if (f->scratch_bytes) scratch_id = tid(scratch(f->scratch_bytes));
        std::ostringstream s;
        s << "s fusion " << label << " " << m << " " << scratch_id << " " << ids.size();
        for (int id : ids) s << " " << id;
        Generated rec;
        rec.body = &body, rec.label = label, rec.inplace = inplace, rec.scratch = scratch_id >= 0, rec.ids = ids;
        push_step(s.str() + "\n");
        steps.back().is_generated = true, steps.back().gen = rec;
    }

    // ---- horizontal fusion (lumen/graph_compiler/passes/horizontal.rs:79): runs of consecutive, mutually independent
    // generated steps whose bodies are the same elementwise program up to its shape become ONE launch over a table of
    // tensor groups - the per-parameter optimizer updates of a training step.
    static std::string shape_text(const std::vector<int64_t>& shape) {
        if (shape.empty()) return "-";
        std::string out;
        for (size_t d = 0; d < shape.size(); d++) out += (d ? "," : "") + std::to_string(shape[d]);
        return out;
    }
    // `body` in the graph text format with every occurrence of `shape` (value types and `shape=` attributes) replaced
    static std::string body_text(const Graph& body, const std::vector<int64_t>& shape, const std::vector<int64_t>& new_shape) {
        std::ostringstream out;
        out << "graph 0\n";
        auto typed = [&](int v) {
            const TensorType& t = body.type(v);
            return std::string(dtype_name(t.dtype)) + " " + shape_text(t.shape == shape ? new_shape : t.shape);
        };
        for (int v : body.inputs) out << "in " << v << " " << typed(v) << "\n";
        for (const Node& n : body.nodes) {
            out << "node " << n.output << " " << n.op << " " << typed(n.output) << " ";
            if (n.inputs.empty()) out << "-";
            for (size_t k = 0; k < n.inputs.size(); k++) out << (k ? "," : "") << n.inputs[k];
            for (const auto& kv : n.attrs) {
                std::string value = kv.second;
                if (kv.first == "shape" && parse_int_list(value) == shape && !shape.empty()) value = shape_text(new_shape);
                out << " " << kv.first << "=" << value;
            }
            out << "\n";
        }
        out << "out ";
        for (size_t k = 0; k < body.outputs.size(); k++) out << (k ? "," : "") << body.outputs[k];
        out << "\nend\n";
        return out.str();
    }
    // The shape a body is elementwise over (every other value a scalar: a constant or a 0-d operand), or false.
    static bool flat_shape(const Graph& body, std::vector<int64_t>* shape) {
        static const std::set<std::string> elementwise = {"add", "sub", "mul", "div", "max", "min", "neg", "abs", "sign", "exp", "log", "sqrt",
                                                          "rsqrt", "tanh", "logistic", "cast", "select", "eq", "lt", "not", "and", "or"};
        bool have = false;
        for (int v : body.inputs) {
            const std::vector<int64_t>& s = body.type(v).shape;
            if (s.empty()) continue;
            if (!have) *shape = s, have = true;
            if (s != *shape) return false;
        }
        if (!have) return false;
        for (const Node& n : body.nodes) {
            const std::vector<int64_t>& s = body.type(n.output).shape;
            if (n.op == "full") {
                if (!s.empty()) return false;
            } else if (n.op == "broadcast_in_dim") {
                if (!body.type(n.inputs.at(0)).shape.empty() || s != *shape) return false;
            } else if (elementwise.count(n.op)) {
                if (s != *shape && !s.empty()) return false;
            } else {
                return false;
            }
        }
        for (int v : body.outputs)
            if (body.type(v).shape != *shape) return false;
        return true;
    }

    void fuse_horizontally() {
        std::vector<Step> out;
        auto buffer_key = [&](int id) { return tensors[(size_t)id].base + "#" + std::to_string(tensors[(size_t)id].buffer); };
        for (size_t i = 0; i < steps.size();) {
            std::vector<int64_t> shape;
            if (!steps[i].is_generated || steps[i].gen.scratch || !flat_shape(*steps[i].gen.body, &shape)) {
                out.push_back(steps[i++]);
                continue;
            }
            const Generated& head = steps[i].gen;
            const std::string signature = body_text(*head.body, shape, {1, 7919});  // a shape no tensor has: equal texts = the same program
            std::set<std::string> written, seen;
            size_t j = i;
            while (j < steps.size()) {
                std::vector<int64_t> sj;
                if (!steps[j].is_generated) break;
                const Generated& m = steps[j].gen;
                if (m.scratch || m.inplace != head.inplace || !flat_shape(*m.body, &sj) || body_text(*m.body, sj, {1, 7919}) != signature) break;
                const size_t n_in = m.body->inputs.size();
                std::set<std::string> ins, outs;
                for (size_t k = 0; k < m.ids.size(); k++) (k < n_in ? ins : outs).insert(buffer_key(m.ids[k]));
                bool clash = false;  // depends on, or overwrites something of, an earlier member
                for (const std::string& key : ins) clash |= written.count(key) != 0;
                for (const std::string& key : outs) clash |= written.count(key) != 0 || seen.count(key) != 0;
                if (clash) break;
                written.insert(outs.begin(), outs.end());
                seen.insert(ins.begin(), ins.end()), seen.insert(outs.begin(), outs.end());
                j++;
            }
            if (j - i < 2) {
                out.push_back(steps[i++]);
                continue;
            }
            // the kernel's row length: the greatest common divisor of the members' sizes, at most 4096
            size_t full = 0;
            while (head.body->type(head.body->inputs[full]).shape.empty()) full++;
            int64_t cols = 0;
            for (size_t k = i; k < j; k++) cols = std::gcd(cols, (int64_t)numel(tensors[(size_t)steps[k].gen.ids[full]].shape));
            while (cols > 4096 && cols % 2 == 0) cols /= 2;
            const std::string text = std::string(head.inplace ? "option inplace\n" : "") + "option multi\n" + body_text(*head.body, shape, {2, cols});
            const int module = module_id(text);
            compile_fusion(modules[(size_t)module]);
            Step merged;  // names every member's tensors: they are all live at the one launch
            std::ostringstream line;
            line << "s multi " << head.label << "_x" << (j - i) << " " << module << " " << (j - i);
            for (size_t k = i; k < j; k++)
                for (int id : steps[k].gen.ids) line << " " << id, merged.tensor_ids.push_back(id);
            merged.line = line.str() + "\n";
            out.push_back(merged);
            i = j;
        }
        steps = out;
    }

    // Cuts the all-reduced gradients (side by side in the arena, in order of production) into buckets of at least
    // `bucket_bytes` and gives each two steps: `all_reduce` of the bucket as one flat tensor, right after the step that
    // produces its last gradient, and `wait` before the first later step that names one of its gradients
    // (lumen/plan/step/triton.rs:122-177, lumen/graph_compiler/schedule.rs:17-41). Every rank lowers the same module,
    // so every rank queues the same collectives in the same order.
    void insert_collectives() {
        struct Bucket {
            size_t start, end;
            int ready, dtype, op;
            std::set<int> buffers;
        };
        std::vector<Bucket> buckets;
        std::vector<const Comm*> sorted;
        for (const Comm& c : comms) sorted.push_back(&c);
        std::sort(sorted.begin(), sorted.end(), [&](const Comm* x, const Comm* y) { return buffers[(size_t)x->view.buffer].place < buffers[(size_t)y->view.buffer].place; });
        for (const Comm* c : sorted) {
            const Buffer& b = buffers[(size_t)c->view.buffer];
            const size_t start = b.place + c->view.offset, end = b.place + b.bytes;
            const bool same = !buckets.empty() && buckets.back().end == start && buckets.back().dtype == c->view.dtype && buckets.back().op == c->op;
            if (!same || (long long)(buckets.back().end - buckets.back().start) >= bucket_bytes) {
                buckets.push_back({start, end, c->ready, c->view.dtype, c->op, {c->view.buffer}});
            } else {
                buckets.back().end = end, buckets.back().ready = std::max(buckets.back().ready, c->ready);
                buckets.back().buffers.insert(c->view.buffer);
            }
        }
        std::stable_sort(buckets.begin(), buckets.end(), [](const Bucket& x, const Bucket& y) { return x.ready < y.ready; });
        num_buckets = (int)buckets.size();
        std::map<size_t, std::vector<Step>> reduce_before, wait_before;
        for (size_t k = 0; k < buckets.size(); k++) {
            const Bucket& b = buckets[k];
            size_t first_use = steps.size();
            for (size_t i = (size_t)b.ready; i < steps.size() && first_use == steps.size(); i++)
                for (int id : steps[i].tensor_ids)
                    if (b.buffers.count(tensors[(size_t)id].buffer)) first_use = i;
            View flat;  // the bucket as one tensor at its place in the workspace (alignment padding is reduced along with it)
            flat.base = "w", flat.offset = b.start, flat.dtype = b.dtype;
            flat.shape = {(int64_t)((b.end - b.start) / dtype_size(b.dtype))}, flat.strides = {1};
            tensors.push_back(flat);
            Step reduce, wait;
            reduce.line = "s all_reduce all_reduce " + std::to_string(tensors.size() - 1) + " " + std::to_string(b.op) + "\n";
            wait.line = "s wait device_wait " + std::to_string(k) + "\n";
            reduce_before[(size_t)b.ready].push_back(reduce);
            wait_before[first_use].push_back(wait);
        }
        std::vector<Step> out;
        for (size_t i = 0; i <= steps.size(); i++) {
            for (const Step& st : reduce_before[i]) out.push_back(st);
            for (const Step& st : wait_before[i]) out.push_back(st);
            if (i < steps.size()) out.push_back(steps[i]);
        }
        steps = out;
    }

    // A `dot_general` of the main graph itself (the fusion pass leaves a product without a tail as it is).
    void lower_bare_dot(const Node& n) {
        emit_gemm(n, n.output, g.type(n.output), 0, "dot_general", [&](int value) { return view_of(value, "dot_general"); });
    }

    void lower_dot(const Node& n, const Graph& body, const std::string& label) {
        const Node* dot = nullptr;
        int epilogue = 0;
        for (const Node& b : body.nodes) {
            if (b.op == "dot_general") {
                if (dot) fail(LB_ERR_UNSUPPORTED, "lb_compile: a dot_general fusion with two products has no kernel");
                dot = &b;
            }
        }
        if (!dot) fail(LB_ERR_INVALID, "lb_compile: a dot_general fusion without a dot_general");
        // tails (the GEMM's epilogues): none; 1 max(product, 0); 2 other + product; 3 select(0 < other, product, 0), a relu's
        // backward with `other` the relu's output. Constants are zeros broadcast to the product's shape.
        std::set<int> zero_fills, zeros;
        std::map<int, const Node*> by_output;
        for (const Node& bn : body.nodes) {
            by_output[bn.output] = &bn;
            if (bn.op == "full") {
                const std::string& c = bn.attr("fill_value");
                if (c == "i:0" || std::strtod(c.c_str() + 2, nullptr) == 0.0) zero_fills.insert(bn.output);
            }
        }
        for (const Node& bn : body.nodes)
            if (bn.op == "broadcast_in_dim" && zero_fills.count(bn.inputs.at(0))) zeros.insert(bn.output);
        int other = -1;
        std::set<const Node*> used = {dot};
        const Node* tail = by_output.count(body.outputs.at(0)) ? by_output[body.outputs.at(0)] : nullptr;
        auto has = [](const std::vector<int>& v, int x) { return std::find(v.begin(), v.end(), x) != v.end(); };
        if (tail == dot) {
            epilogue = 0;
        } else if (tail && tail->op == "max" && has(tail->inputs, dot->output) && (zeros.count(tail->inputs[0]) || zeros.count(tail->inputs[1]))) {
            epilogue = 1;
        } else if (tail && tail->op == "add" && has(tail->inputs, dot->output)) {
            epilogue = 2, other = tail->inputs[0] == dot->output ? tail->inputs[1] : tail->inputs[0];
        } else if (tail && tail->op == "select" && tail->inputs.at(1) == dot->output && zeros.count(tail->inputs.at(2))) {
            const Node* cond = by_output.count(tail->inputs[0]) ? by_output[tail->inputs[0]] : nullptr;
            if (!cond || cond->op != "lt" || !zeros.count(cond->inputs.at(0)))
                fail(LB_ERR_UNSUPPORTED, "lb_compile: dot_general fusion: the select's condition is not `0 < operand`");
            epilogue = 3, other = cond->inputs.at(1);
            used.insert(cond);
        } else {
            fail(LB_ERR_UNSUPPORTED, format("lb_compile: primitive `%s` after the product of a dot_general fusion has no epilogue", tail ? tail->op.c_str() : "?"));
        }
        if (tail) used.insert(tail);
        for (const Node& bn : body.nodes)
            if (!used.count(&bn) && bn.op != "full" && bn.op != "broadcast_in_dim")
                fail(LB_ERR_UNSUPPORTED, format("lb_compile: primitive `%s` in a dot_general fusion has no epilogue", bn.op.c_str()));
        auto operand = [&](int body_value) -> View {
            for (size_t k = 0; k < body.inputs.size(); k++)
                if (body.inputs[k] == body_value) return view_of(n.inputs.at(k), label.c_str());
            fail(LB_ERR_UNSUPPORTED, "lb_compile: a dot_general operand computed inside its fusion");
            return View{};
        };
        View aux;
        if (other >= 0) aux = operand(other);  // fails when the epilogue operand is computed inside the fusion
        static const char* const kNames[] = {"dot_general", "dot_general_relu", "dot_general_add", "dot_general_relu_backward"};
        emit_gemm(*dot, n.output, body.type(body.outputs.at(0)), epilogue, kNames[epilogue], operand, other >= 0 ? &aux : nullptr);
    }

    template <class Operand>
    void emit_gemm(const Node& dot_node, int result, const TensorType& t, int epilogue, const std::string& label, Operand operand,
                   const View* aux = nullptr) {
        const Node* dot = &dot_node;
        if (!dot->ints("lhs_batch").empty() || dot->ints("lhs_contracting").size() != 1 || dot->ints("rhs_contracting").size() != 1)
            fail(LB_ERR_UNSUPPORTED, "lb_compile: dot_general with batch dimensions or several contracting dimensions");
        View a = operand(dot->inputs.at(0)), b = operand(dot->inputs.at(1));
        if (a.shape.size() != 2 || b.shape.size() != 2) fail(LB_ERR_UNSUPPORTED, "lb_compile: dot_general operands must be matrices");
        // A as [M, K] and B as [K, N]: a contraction over the other dimension is the transposed VIEW of the operand
        if (dot->ints("lhs_contracting")[0] == 0) std::swap(a.shape[0], a.shape[1]), std::swap(a.strides[0], a.strides[1]);
        if (dot->ints("rhs_contracting")[0] == 1) std::swap(b.shape[0], b.shape[1]), std::swap(b.strides[0], b.strides[1]);
        // A [K, N] weight whose K rows lie 8 KB or more apart (N contiguous, N >= 4096 16-bit elements) is a slow TMA
        // operand: every 128-byte row of a tile comes from a different DRAM page. Transposing it once per run costs
        // microseconds; the product then reads the K-major copy through the transposed view.
        {
            const int64_t k = b.shape[0], n = b.shape[1];
            const int size = dtype_size(b.dtype);
            if (b.strides[0] == n && b.strides[1] == 1 && size == 2 && n * size >= 8192 && k * n * size <= (64LL << 20) && a.shape[0] >= 8 * k) {
                View copy = fresh(b.dtype, {n, k});
                push_step("s transpose weight_transpose " + std::to_string(tid(b)) + " " + std::to_string(tid(copy)) + "\n");
                b = copy;
                b.shape = {k, n}, b.strides = {1, k};
            }
        }
        View d = fresh(t.dtype, t.shape, result);
        views[result] = d;
        const size_t sb = lb_gemm_scratch_bytes(a.shape[0], b.shape[1], a.shape[1], 1);
        std::ostringstream s;
        s << "s gemm " << label << " " << tid(a) << " " << tid(b) << " " << tid(d) << " " << epilogue << " " << (sb ? tid(scratch(sb)) : -1) << " " << (aux ? tid(*aux) : -1);
        push_step(s.str() + "\n");
    }

    void lower_attention(const Node& n, const Graph& body, const std::string& name, const std::string& label) {
        double scale;
        int causal;
        long long offset;
        if (n.has("attention")) {
            // set by the attention matcher: `key:value;...` with the scale, the mask and every operand's dimension roles
            std::map<std::string, std::string> found;
            std::istringstream in(n.attr("attention"));
            std::string item;
            while (std::getline(in, item, ';')) {
                size_t colon = item.find(':');
                if (colon != std::string::npos) found[item.substr(0, colon)] = item.substr(colon + 1);
            }
            for (const char* role : {"q", "k", "v", "o"})
                if (found.count(role) && found[role] != "BSNH")
                    fail(LB_ERR_UNSUPPORTED, format("lb_compile: attention operand %s is laid out %s; this lowering takes [B, S, N, H] operands", role, found[role].c_str()));
            scale = std::strtod(found["scale"].c_str(), nullptr), causal = std::atoi(found["causal"].c_str()), offset = std::atoll(found["offset"].c_str());
        } else {
            attention_params(body, &scale, &causal, &offset);
        }
        char hex[64];
        snprintf(hex, sizeof(hex), "%a", scale);
        std::vector<int> outs = fusion_outputs(n, body);
        std::ostringstream s;
        if (name == "flash_attention") {
            const View &q = view_of(n.inputs.at(0), "flash_attention"), &k = view_of(n.inputs.at(1), "flash_attention"), &v = view_of(n.inputs.at(2), "flash_attention");
            if (q.shape.size() != 4) fail(LB_ERR_UNSUPPORTED, "lb_compile: flash_attention takes [B, S, N, H] operands");
            const int64_t B = q.shape[0], S = q.shape[1], N = q.shape[2];
            View o = fresh(q.dtype, q.shape, outs[0]);
            views[outs[0]] = o;
            View lse = fresh(LB_F32, {B, N, S}, outs.size() > 1 ? outs[1] : -1);
            if (outs.size() > 1 && outs[1] >= 0) {
                View as_traced = lse;
                as_traced.shape = g.type(outs[1]).shape, as_traced.strides = dense_strides(as_traced.shape);
                views[outs[1]] = as_traced;
            }
            s << "s attn_fwd " << label << " " << tid(q) << " " << tid(k) << " " << tid(v) << " " << tid(o) << " " << tid(lse);
        } else {
            // q, k, v, o, lse, dO -> dq, dk, dv
            const View& q = view_of(n.inputs.at(0), "flash_attention_backward");
            if (q.shape.size() != 4 || n.inputs.size() != 6) fail(LB_ERR_UNSUPPORTED, "lb_compile: flash_attention_backward takes q, k, v, o, lse, dO");
            const int64_t B = q.shape[0], S = q.shape[1], N = q.shape[2], H = q.shape[3];
            View lse = view_of(n.inputs.at(4), "flash_attention_backward");
            lse.shape = {B, N, S}, lse.strides = dense_strides(lse.shape);
            View delta = fresh(LB_F32, {B, N, S});
            s << "s attn_bwd " << label;
            for (int k : {0, 1, 2, 3}) s << " " << tid(view_of(n.inputs.at((size_t)k), "flash_attention_backward"));
            s << " " << tid(view_of(n.inputs.at(5), "flash_attention_backward")) << " " << tid(lse) << " " << tid(delta);
            for (size_t k = 0; k < 3; k++) {
                const View& like = view_of(n.inputs.at(k), "flash_attention_backward");
                View grad = fresh(like.dtype, like.shape, outs.at(k));
                views[outs[k]] = grad;
                s << " " << tid(grad);
            }
            if (!deterministic && q.dtype == LB_BF16 && H == 64) s << " " << tid(fresh(LB_F32, q.shape));  // the atomic-dQ form's accumulator
        }
        s << " " << hex << " " << causal << " " << offset;
        push_step(s.str() + "\n");
    }

    // Operands of a last-axis concatenation that are (reshapes of) attention-backward gradients used nowhere else.
    void find_concat_placements() {
        std::map<int, int> uses;  // value -> readers other than fusion_output
        for (const Node& n : g.nodes)
            if (n.op != "fusion_output")
                for (int v : n.inputs) uses[v]++;
        auto from_attention_backward = [&](int v) {
            const Node* p = g.node_of(v);
            if (p && p->op == "fusion_output") p = g.node_of(p->inputs.at(0));
            return p && p->op == "fusion" && p->attr("name") == "flash_attention_backward";
        };
        for (const Node& n : g.nodes) {
            if (n.op != "concatenate") continue;
            const TensorType& ct = g.type(n.output);
            if ((size_t)n.integer("dimension") + 1 != ct.shape.size()) continue;
            std::vector<std::pair<int, Slot>> found;
            int64_t col = 0;
            bool ok = true;
            for (int v : n.inputs) {
                int src = v;
                const Node* p = g.node_of(src);
                if (p && p->op == "reshape" && uses[src] == 1) src = p->inputs.at(0);
                const int64_t width = g.type(v).shape.back(), last = g.type(src).shape.empty() ? 0 : g.type(src).shape.back();
                if (!from_attention_backward(src) || uses[src] != 1 || last == 0 || width % last != 0) {
                    ok = false;
                    break;
                }
                found.push_back({src, Slot{n.output, col, width}});
                col += width;
            }
            if (ok)
                for (const auto& f : found) placed[f.first] = f.second;
        }
    }

    std::string run() {
        find_concat_placements();
        for (const Node& n : g.nodes)
            if (n.op == "all_reduce") reduced_values.insert(n.inputs.at(0));
        for (size_t k = 0; k < g.outputs.size(); k++) output_slot.emplace(g.outputs[k], (int)k);  // the first slot of a value listed twice
        for (size_t k = 0; k < g.inputs.size(); k++) {
            const TensorType& t = g.type(g.inputs[k]);
            View v;
            v.base = "i" + std::to_string(k), v.dtype = t.dtype, v.shape = t.shape, v.strides = dense_strides(t.shape);
            views[g.inputs[k]] = v;
        }
        for (const Node& n : g.nodes) {
            if (n.op == "fusion_output") continue;  // placed with its fusion
            if (n.op == "device_wait" || n.op == "host_wait") {  // the reduced value is the operand's memory; the wait is a step of its bucket
                views[n.output] = view_of(n.inputs.at(0), n.op.c_str());
                continue;
            }
            if (n.op == "all_reduce") {
                // in place, queued once the operand's producer - the last step that names its buffer - has been queued
                const View src = view_of(n.inputs.at(0), "all_reduce");
                if (!src.dense() || src.buffer < 0 || !buffers[(size_t)src.buffer].arena)
                    fail(LB_ERR_UNSUPPORTED, "lb_compile: all_reduce of a strided view, of a graph input or of a view of another value");
                static const std::map<std::string, int> ops = {{"sum", 0}, {"prod", 1}, {"max", 2}, {"min", 3}};
                auto op = ops.find(n.attr("op"));
                if (op == ops.end()) fail(LB_ERR_UNSUPPORTED, format("lb_compile: all_reduce with op %s", n.attr("op").c_str()));
                Comm c;
                c.view = src, c.op = op->second;
                for (size_t k = steps.size(); k-- > 0 && c.ready == 0;)
                    for (int id : steps[k].tensor_ids)
                        if (tensors[(size_t)id].buffer == src.buffer) c.ready = (int)k + 1;
                buffers[(size_t)src.buffer].pinned_end = true;
                comms.push_back(c);
                views[n.output] = src;
                continue;
            }
            if (n.op == "reshape") {
                View v = view_of(n.inputs.at(0), "reshape");
                std::vector<int64_t> strides;
                if (!reshape_strides(v.shape, v.strides, g.type(n.output).shape, &strides)) {
                    v = dense_operand(n.inputs.at(0), "reshape");  // the view's elements are not evenly spaced in the new shape: a dense copy first
                    strides = dense_strides(g.type(n.output).shape);
                }
                v.shape = g.type(n.output).shape, v.strides = strides;
                views[n.output] = v;
                continue;
            }
            if (n.op == "transpose") {  // a view: the strides are permuted with the shape
                const View& src = view_of(n.inputs.at(0), "transpose");
                View v = src;
                const std::vector<int64_t> perm = n.ints("permutation");
                for (size_t d = 0; d < perm.size(); d++) v.shape[d] = src.shape.at((size_t)perm[d]), v.strides[d] = src.strides.at((size_t)perm[d]);
                views[n.output] = v;
                continue;
            }
            if (n.op == "dot_general") {
                lower_bare_dot(n);
                continue;
            }
            if (n.op == "slice") {  // a view: the same strides from the first element of the slice
                View v = view_of(n.inputs.at(0), "slice");
                const std::vector<int64_t> start = n.ints("start_indices");
                int64_t first = 0;
                for (size_t d = 0; d < start.size(); d++) first += start[d] * v.strides.at(d);
                v.offset += (size_t)first * dtype_size(v.dtype);
                v.shape = g.type(n.output).shape;
                views[n.output] = v;
                continue;
            }
            if (n.op == "full") {
                const std::string& c = n.attr("fill_value");
                const TensorType& t = g.type(n.output);
                const bool zero = c == "i:0" || std::strtod(c.c_str() + 2, nullptr) == 0.0;
                if (zero) {
                    // zeros that only scatter_add nodes add into (an embedding gradient's start): the kernel writes its
                    // sums over nothing instead of reading a zero-filled table
                    bool tables_only = true, used = false;
                    for (const Node& u : g.nodes)
                        for (size_t k = 0; k < u.inputs.size(); k++)
                            if (u.inputs[k] == n.output) used = true, tables_only &= u.op == "scatter_add" && k == 0;
                    for (int o : g.outputs) tables_only &= o != n.output;
                    if (used && tables_only) {
                        zero_tables.insert(n.output);
                        continue;
                    }
                }
                View v = fresh(t.dtype, t.shape, n.output);
                views[n.output] = v;
                if (zero) {
                    push_step("s fill zeros " + std::to_string(tid(v)) + " 0\n");
                } else if (numel(t.shape) > 0) {
                    // any other constant (a padding value beside a concatenation): a generated kernel that has no operands
                    std::ostringstream body;
                    body << "graph 0\nnode 0 full " << dtype_name(t.dtype) << " " << shape_text(t.shape) << " -";
                    for (const auto& kv : n.attrs) body << " " << kv.first << "=" << kv.second;
                    body << "\nout 0\nend\n";
                    const int m = module_id(body.str());
                    compile_fusion(modules[(size_t)m]);
                    push_step("s fusion constant " + std::to_string(m) + " -1 1 " + std::to_string(tid(v)) + "\n");
                }
                continue;
            }
            if (n.op == "scatter_add") {
                const bool from_zeros = zero_tables.count(n.inputs.at(0)) != 0;
                const View ids = view_of(n.inputs.at(1), "scatter_add"), upd = view_of(n.inputs.at(2), "scatter_add");
                const TensorType& t = g.type(n.output);
                if (t.shape.size() != 2) fail(LB_ERR_UNSUPPORTED, "lb_compile: scatter_add is lowered for [rows, width] tables");
                View o = fresh(t.dtype, t.shape, n.output);
                views[n.output] = o;
                const int64_t rows = t.shape[0], width = t.shape[1], picks = numel(ids.shape);
                // sorted form: counts, cursor, starts, order, sorted (int32 each); atomic form: float32 rows
                const size_t bytes = deterministic ? (size_t)(3 * rows + 1 + 2 * picks) * 4 : (size_t)rows * width * 4;
                std::ostringstream st;
                st << "s scatter_add scatter_add " << (from_zeros ? -1 : tid(view_of(n.inputs.at(0), "scatter_add"))) << " " << tid(ids) << " " << tid(upd) << " " << tid(o) << " " << tid(scratch(bytes)) << " "
                   << (deterministic ? 1 : 0);
                push_step(st.str() + "\n");
                continue;
            }
            if (n.op == "concatenate" && concat_views.count(n.output)) {  // its operands were produced in place
                views[n.output] = concat_views[n.output];
                continue;
            }
            if (n.op == "concatenate") {
                // each operand is copied to its place: [outer, part] rows of the operand into rows `pitch` apart of the result
                const TensorType& t = g.type(n.output);
                const size_t axis = (size_t)n.integer("dimension");
                View o = fresh(t.dtype, t.shape, n.output);
                views[n.output] = o;
                int64_t outer = 1, inner = 1;
                for (size_t d = 0; d < axis; d++) outer *= t.shape[d];
                for (size_t d = axis + 1; d < t.shape.size(); d++) inner *= t.shape[d];
                int64_t at = 0;
                for (int v : n.inputs) {
                    const View src = dense_operand(v, "concatenate");
                    const int64_t part = src.shape.at(axis) * inner;
                    View from = src, to = o;
                    from.shape = {outer, part}, from.strides = {part, 1};
                    to.shape = {outer, part}, to.strides = {t.shape[axis] * inner, 1};
                    to.offset += (size_t)at * dtype_size(t.dtype);
                    push_step("s copy concatenate " + std::to_string(tid(from)) + " " + std::to_string(tid(to)) + "\n");
                    at += part;
                }
                continue;
            }
            if (n.op != "fusion")
                fail(LB_ERR_UNSUPPORTED, format("lb_compile: primitive `%s` outside a fusion has no kernel; the module must have been through the "
                                                "fusion pass", n.op.c_str()));
            const int body_index = (int)n.integer("body");
            if (body_index < 0 || body_index + 1 >= (int)module.graphs.size() || body_index >= (int)blocks.size())
                fail(LB_ERR_INVALID, "lb_compile: a fusion refers to a body the module does not hold");
            const Graph& body = *module.graphs[(size_t)body_index];
            const std::string name = n.attr("name"), label = n.has("label") ? n.attr("label") : name;
            if (name == "dot_general") lower_dot(n, body, label);
            else if (name == "flash_attention" || name == "flash_attention_backward") lower_attention(n, body, name, label);
            else lower_generated(n, body, body_index, label);
        }
        // outputs that ended up somewhere else (an input returned as it is, a reshape of another value) are copied out
        for (size_t k = 0; k < g.outputs.size(); k++) {
            const View& v = view_of(g.outputs[k], "the output list");
            auto given = donate.find((int)k);
            const std::string want = given != donate.end() ? "i" + std::to_string(given->second) : "o" + std::to_string(k);
            if (v.base == want && v.offset == 0) continue;
            if (!v.dense()) {
                // a 2-d transpose (a weight gradient returned as the transposed view of the product that made it) is
                // written into the output by the transpose kernel, any other view by the copy step below
                std::vector<std::pair<int64_t, int64_t>> live;
                for (size_t d = 0; d < v.shape.size(); d++)
                    if (v.shape[d] != 1) live.push_back({v.shape[d], v.strides[d]});
                const int size = dtype_size(v.dtype);
                if (live.size() == 2 && live[0].second == 1 && live[1].second == live[0].first && (size == 2 || size == 4)) {
                    const int64_t rows = live[1].first, cols = live[0].first;  // the memory is a dense [rows, cols]
                    View src = v, dst = v;
                    src.shape = {rows, cols}, src.strides = {cols, 1};
                    dst.base = want, dst.buffer = -1, dst.offset = 0, dst.shape = {cols, rows}, dst.strides = {rows, 1};
                    push_step("s transpose output_transpose " + std::to_string(tid(src)) + " " + std::to_string(tid(dst)) + "\n");
                    continue;
                }
            }
            View dst = v;
            dst.base = want, dst.buffer = -1, dst.offset = 0, dst.strides = dense_strides(v.shape);
            push_step("s copy output_copy " + std::to_string(tid(v)) + " " + std::to_string(tid(dst)) + "\n");
        }
        place_arena();
        if (!comms.empty()) insert_collectives();
        fuse_horizontally();
        std::ostringstream text;
        for (size_t k = 0; k < modules.size(); k++) text << "module " << k << "\n" << modules[k] << "endmodule\n";
        const size_t workspace = place();
        text << "plan " << g.inputs.size() << " " << g.outputs.size() << " " << workspace << "\n";
        for (size_t id = 0; id < tensors.size(); id++) {
            const View& v = tensors[id];
            text << "t " << id << " " << dtype_name(v.dtype) << " " << v.base << " " << (v.buffer >= 0 ? buffers[(size_t)v.buffer].place + v.offset : v.offset)
                 << " " << v.shape.size();
            for (int64_t n : v.shape) text << " " << n;
            for (int64_t n : v.strides) text << " " << n;
            text << "\n";
        }
        for (const Step& st : steps) text << st.line;
        text << "end\n";
        return text.str();
    }
};

}  // namespace
}  // namespace lb

extern "C" int lb_compile(const char* module_text, int device, const lb_config* config, lb_plan** out) {
    return lb::guarded([&] {
        if (!module_text || !out) lb::fail(LB_ERR_INVALID, "lb_compile: null argument");
        if (device >= 0) {
            int count = 0;
            if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0) {
                if (device >= count) lb::fail(LB_ERR_INVALID, lb::format("lb_compile: device %d of %d", device, count));
                LB_CUDA(cudaSetDevice(device));
            }
        }
        const std::string text(module_text);
        lb::Module module = lb::parse_module(text);
        lb::Lowering lowering(module, text, !config || config->deterministic != 0);
        if (config && config->bucket_bytes > 0) lowering.bucket_bytes = config->bucket_bytes;
        if (config && config->n_donate > 0) {
            if (!config->donate) lb::fail(LB_ERR_INVALID, "lb_compile: n_donate without a donate list");
            const lb::Graph& main = module.main();
            for (int k = 0; k < config->n_donate; k++) {
                const int out_index = config->donate[2 * k], in_index = config->donate[2 * k + 1];
                if (out_index < 0 || out_index >= (int)main.outputs.size() || in_index < 0 || in_index >= (int)main.inputs.size())
                    lb::fail(LB_ERR_INVALID, lb::format("lb_compile: donation %d -> %d names an output or input the graph does not have", out_index, in_index));
                const lb::TensorType &o = main.type(main.outputs[(size_t)out_index]), &i = main.type(main.inputs[(size_t)in_index]);
                if (o.dtype != i.dtype || o.shape != i.shape)
                    lb::fail(LB_ERR_INVALID, lb::format("lb_compile: output %d is not typed like input %d whose memory it is given", out_index, in_index));
                lowering.donate[out_index] = in_index;
            }
        }
        const std::string plan_text = lowering.run();
        int rc = lb_plan_create(plan_text.c_str(), out);
        if (rc != LB_OK) lb::fail(rc, lb_last_error());
    });
}
