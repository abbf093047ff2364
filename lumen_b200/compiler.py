"""Lowers a traced graph of fusions, dots and views to a plan: the host-side counterpart of the reference's
`Device::lower` = placement in one workspace + one kernel per step (lumen/codegen/devices/cuda/mod.rs:140-189,
lumen/plan/compile.rs:17-330).

Placement rules kept from the reference (lumen/plan/README.md:36-48): reshapes, slices and waits alias their
operand's buffer; donated outputs (weights written by the optimizer) live in the donor input; everything else is
packed into the workspace by live range, largest first, at the lowest non-overlapping 256-byte aligned offset; the
operands of a concatenation are written in place into its buffer (the reference's place_concats pass). Gradients
that are all-reduced live in one contiguous arena at the start of the workspace, in order of production, and are
reduced in a few large buckets: each bucket's `all_reduce` is a plan step queued as soon as its last gradient has been
produced, its `wait` a step placed before the first reader (lumen/plan/step/triton.rs:122-177,
lumen/graph_compiler/schedule.rs:17-41). Runs of independent elementwise fusions with one body - the per-parameter
optimizer updates - are merged into one horizontally fused launch (lumen/graph_compiler/passes/horizontal.rs:79).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from lumen_b200 import graph as G
from lumen_b200.graph import SIZE_OF

ALIGN = 256
ROW_FUSIONS = ("elementwise", "row", "reduction")


@dataclass
class Buffer:
    kind: str  # 'i', 'o' or 'w'
    index: int = 0
    nbytes: int = 0
    first: int = 0  # first step that touches it
    last: int = 0  # last step that touches it
    offset: int = 0
    arena: bool = False  # all-reduced gradient: placed in the arena, alive to the end
    pinned_end: bool = False


@dataclass
class View:
    buffer: Buffer
    offset: int  # bytes
    dtype: str
    shape: tuple
    strides: tuple  # elements

    @property
    def dense(self) -> bool:
        """Row-major without gaps; the stride of a dimension of size 1 addresses nothing and is not compared."""
        want = dense_strides(self.shape)
        return math.prod(self.shape) <= 1 or all(n == 1 or s == w for n, s, w in zip(self.shape, self.strides, want))


@dataclass
class Comm:
    ready_step: int  # the collective may start once steps [0, ready_step) are queued
    view: View
    op: str


@dataclass
class CompiledPlan:
    text: str
    workspace_bytes: int
    n_inputs: int
    n_outputs: int
    comms: list = field(default_factory=list)  # Comm, in program order
    arena_bytes: int = 0
    labels: list = field(default_factory=list)
    kernel_launches: int = 0  # kernels one run launches (a column reduction is 2, split-K 2, attention backward 3, scatter-add 2)
    buckets: list = field(default_factory=list)  # {"start", "end", "ready", "dtype", "op"} per all_reduce step, in queue order


def dense_strides(shape):
    strides, s = [], 1
    for n in reversed(shape):
        strides.append(s)
        s *= n
    return tuple(reversed(strides))


def reshape_view(shape, strides, new_shape):
    """Strides of `new_shape` over the same memory, or None when the reshape needs a copy (NumPy's no-copy rule)."""
    old = [(n, s) for n, s in zip(shape, strides) if n != 1]
    new_strides = [0] * len(new_shape)
    oi, ni = 0, 0
    new = [n for n in new_shape]
    while ni < len(new):
        if new[ni] == 1:
            new_strides[ni] = 1
            ni += 1
            continue
        if oi >= len(old):
            return None
        # gather old dims into a contiguous chunk covering one or more new dims
        n_old, s_old = old[oi]
        chunk, last_stride = n_old, s_old
        oj = oi + 1
        nj = ni
        size_new = new[nj]
        while size_new != chunk:
            if size_new < chunk:
                nj += 1
                while nj < len(new) and new[nj] == 1:
                    nj += 1
                if nj >= len(new):
                    return None
                size_new *= new[nj]
            else:
                if oj >= len(old) or old[oj][1] * old[oj][0] != last_stride:
                    return None
                chunk *= old[oj][0]
                last_stride = old[oj][1]
                oj += 1
        stride = last_stride
        for k in range(nj, ni - 1, -1):
            if new[k] == 1:
                new_strides[k] = 1
                continue
            new_strides[k] = stride
            stride *= new[k]
        oi, ni = oj, nj + 1
    if oi != len(old):
        return None
    return tuple(new_strides)


class Lowering:
    def __init__(self, graph: G.Graph, donate: dict[int, int] | None = None, deterministic: bool = True,
                 bucket_bytes: int = 64 << 20, horizontal: bool = True):
        self.g = graph
        self.donate = donate or {}
        self.deterministic = deterministic
        self.bucket_bytes = bucket_bytes
        self.horizontal = horizontal
        self.bodies: dict[int, tuple] = {}  # module index -> (body graph, inplace)
        self.views: dict[int, View] = {}
        self.buffers: list[Buffer] = []
        self.steps: list[tuple] = []  # (kind, label, payload)
        self.modules: list[str] = []
        self.module_index: dict[str, int] = {}
        self.comms: list[Comm] = []
        self.zeros: set[int] = set()
        self.uses: dict[int, list[G.Node]] = {}
        for n in graph.nodes:
            for v in n.inputs:
                self.uses.setdefault(v, []).append(n)
        self.out_target: dict[int, Buffer] = {}
        self.placed: dict[int, tuple] = {}  # value -> (concat value, column offset in elements, row width)
        self.concat_buffers: dict[int, Buffer] = {}

    # ---- buffers ----------------------------------------------------------------------------------------------
    def new_buffer(self, nbytes, arena=False) -> Buffer:
        b = Buffer("w", 0, nbytes, first=len(self.steps), last=len(self.steps), arena=arena)
        self.buffers.append(b)
        return b

    def touch(self, view: View, step=None):
        step = len(self.steps) if step is None else step
        view.buffer.first = min(view.buffer.first, step)
        view.buffer.last = max(view.buffer.last, step)

    def fresh(self, v: int) -> View:
        """Dense storage for value `v`: the graph output / donor buffer when it is an output, its slot in a
        concatenation when placed there, else a new workspace buffer (in the arena when it is all-reduced)."""
        t = self.g.types[v]
        if v in self.placed:
            cat, col, width = self.placed[v]
            ct = self.g.types[cat]
            if cat not in self.concat_buffers:
                self.concat_buffers[cat] = self.out_target.get(cat) or self.new_buffer(ct.nbytes, self.is_reduced(cat))
            buf = self.concat_buffers[cat]
            # value shape [.., width] laid out as rows of the concatenation
            rows = t.numel // width
            inner = reshape_view((rows, width), (ct.shape[-1], 1), t.shape)
            return View(buf, col * SIZE_OF[t.dtype], t.dtype, t.shape, inner)
        buf = self.out_target.get(v) or self.new_buffer(t.nbytes, self.is_reduced(v))
        return View(buf, 0, t.dtype, t.shape, dense_strides(t.shape))

    def is_reduced(self, v: int) -> bool:
        return any(n.op == "all_reduce" for n in self.uses.get(v, []))

    # ---- the walk ---------------------------------------------------------------------------------------------
    def run(self) -> CompiledPlan:
        g = self.g
        for k, v in enumerate(g.inputs):
            t = g.types[v]
            self.views[v] = View(Buffer("i", k, t.nbytes), 0, t.dtype, t.shape, dense_strides(t.shape))
        out_buffers = []
        for k, v in enumerate(g.outputs):
            out_buffers.append(self.views[g.inputs[self.donate[k]]].buffer if k in self.donate else Buffer("o", k, g.types[v].nbytes))
            self.out_target.setdefault(v, out_buffers[k])  # a value returned twice is produced in its first place and copied to the others
        self.find_concat_placements()
        for n in g.nodes:
            self.lower(n)
        for k, v in enumerate(g.outputs):
            view = self.views[v]
            want = out_buffers[k]
            if view.buffer is not want or view.offset != 0 or not view.dense:
                # an output that ended up a view of something else is copied out
                if not view.dense:
                    # a 2-d transpose (a weight gradient returned as the transposed view of the product that made it)
                    # is written into the output by the transpose kernel, any other view by the copy step below
                    live = [(n, s) for n, s in zip(view.shape, view.strides) if n != 1]
                    if len(live) == 2 and live[0][1] == 1 and live[1][1] == live[0][0] and SIZE_OF[view.dtype] in (2, 4):
                        rows, cols = live[1][0], live[0][0]  # the memory is a dense [rows, cols]; the output is its transpose
                        src = View(view.buffer, view.offset, view.dtype, (rows, cols), (cols, 1))
                        dst = View(want, 0, view.dtype, (cols, rows), (rows, 1))
                        self.touch(src)
                        self.steps.append(("transpose", "output_transpose", (src, dst)))
                        continue
                dst = View(want, 0, view.dtype, view.shape, dense_strides(view.shape))
                self.touch(view)
                self.steps.append(("copy", "output_copy", (view, dst)))
        return self.emit()

    def find_concat_placements(self):
        """Operands of a last-axis concatenation that are (reshapes of) attention-backward gradients used nowhere else
        are produced directly inside the concatenation's buffer; other operands are copied into place."""
        g = self.g
        for n in g.nodes:
            if n.op != "concatenate":
                continue
            ct = g.types[n.output]
            if n.params["dimension"] != len(ct.shape) - 1:
                continue
            sources, col, ok = [], 0, True
            for v in n.inputs:
                src = v
                prod = g.producer(src)
                if prod is not None and prod.op == "reshape" and len(self.uses.get(src, [])) == 1:
                    src = prod.inputs[0]
                    prod = g.producer(src)
                real_uses = [u for u in self.uses.get(src, []) if u.op != "fusion_output"]
                maker = g.producer(prod.inputs[0]) if prod is not None and prod.op == "fusion_output" else prod
                # attention-backward gradients only: those kernels write strided rows, generated kernels do not
                if maker is None or maker.op != "fusion" or maker.params.get("name") != "flash_attention_backward" or len(real_uses) != 1:
                    ok = False
                    break
                sources.append((src, col, g.types[v].shape[-1]))
                col += g.types[v].shape[-1]
            if ok:
                for src, c, w in sources:
                    if g.types[src].shape[-1] and w % g.types[src].shape[-1] == 0:
                        self.placed[src] = (n.output, c, w)
                    else:
                        ok = False
                if not ok:
                    for src, _, _ in sources:
                        self.placed.pop(src, None)

    def module(self, body: G.Graph, inplace=False) -> int:
        text = ("option inplace\n" if inplace else "") + body.to_text()
        if text not in self.module_index:
            self.module_index[text] = len(self.modules)
            self.modules.append(text)
            self.bodies[self.module_index[text]] = (body, inplace)
        return self.module_index[text]

    def lower(self, n: G.Node):
        g, v = self.g, n.output
        op = n.op
        if op in ("reshape",):
            src = self.views[n.inputs[0]]
            strides = reshape_view(src.shape, src.strides, g.types[v].shape)
            if strides is None:  # the view's elements are not evenly spaced in the new shape: a dense copy first
                src = self.dense_operand(n.inputs[0], "reshape")
                strides = dense_strides(g.types[v].shape)
            self.views[v] = View(src.buffer, src.offset, src.dtype, g.types[v].shape, strides)
        elif op == "slice":
            src = self.views[n.inputs[0]]
            start = n.params["start_indices"]
            off = sum(s * st for s, st in zip(start, src.strides)) * SIZE_OF[src.dtype]
            self.views[v] = View(src.buffer, src.offset + off, src.dtype, g.types[v].shape, src.strides)
        elif op == "transpose":
            # a view: shape and strides permuted. Products and attention read strided operands in place; a fused kernel
            # that needs the value dense gets a copy (`dense_operand`).
            src = self.views[n.inputs[0]]
            perm = n.params["permutation"]
            self.views[v] = View(src.buffer, src.offset, src.dtype, tuple(src.shape[d] for d in perm), tuple(src.strides[d] for d in perm))
        elif op in ("device_wait", "host_wait"):
            self.views[v] = self.views[n.inputs[0]]
        elif op == "all_reduce":
            src = self.views[n.inputs[0]]
            if not src.dense:
                raise NotImplementedError("all_reduce of a strided view")
            src.buffer.pinned_end = True
            # ready once the last step that touched the operand (its producer) has been queued
            self.comms.append(Comm(src.buffer.last + 1, src, n.params["op"]))
            self.views[v] = src
        elif op == "full":
            if n.params["fill_value"] == 0 and all(u.op == "scatter_add" and u.inputs[0] == v for u in self.uses.get(v, [])):
                self.zeros.add(v)
            elif n.params["fill_value"] == 0:
                view = self.fresh(v)
                self.steps.append(("fill", "zeros", (view, 0)))
                self.views[v] = view
            else:
                # any other constant (a padding value beside a concatenation): a generated kernel that has no operands
                view = self.fresh(v)
                self.views[v] = view
                if g.types[v].numel:
                    body = G.Graph()
                    body.set_outputs([body.apply("full", (), **n.params)])
                    self.touch(view)
                    self.steps.append(("fusion", "constant", (self.module(body), None, [view])))
        elif op == "fusion_output":
            pass  # bound when its fusion was lowered
        elif op == "concatenate":
            t = g.types[v]
            if v in self.concat_buffers:  # its operands were produced in place
                self.views[v] = View(self.concat_buffers[v], 0, t.dtype, t.shape, dense_strides(t.shape))
                return
            # each operand is copied to its place: [outer, part] rows of the operand into rows `pitch` apart of the result
            axis = n.params["dimension"]
            out = self.fresh(v)
            self.views[v] = out
            outer, inner = math.prod(t.shape[:axis]), math.prod(t.shape[axis + 1 :])
            pitch, at = t.shape[axis] * inner, 0
            for operand in n.inputs:
                src = self.dense_operand(operand, "concatenate")
                part = src.shape[axis] * inner
                origin = View(src.buffer, src.offset, src.dtype, (outer, part), (part, 1))
                place = View(out.buffer, out.offset + at * SIZE_OF[t.dtype], t.dtype, (outer, part), (pitch, 1))
                self.touch(origin)
                self.touch(place)
                self.steps.append(("copy", "concatenate", (origin, place)))
                at += part
        elif op == "dot_general":
            self.lower_dot(n, n, v, relu=False)
        elif op == "scatter_add":
            x, ids, upd = n.inputs
            out = self.fresh(v)
            rows, width = g.types[v].shape
            picks = g.types[ids].numel
            # sorted form: counts, cursor, starts, order, sorted (int32 each); atomic form: float32 rows
            nbytes = (3 * rows + 1 + 2 * picks) * 4 if self.deterministic else rows * width * 4
            scratch = View(self.new_buffer(nbytes), 0, "uint8", (nbytes,), (1,))
            xin = None if x in self.zeros else self.views[x]
            args = (xin, self.views[ids], self.views[upd], out, scratch)
            for a in args:
                if a is not None:
                    self.touch(a)
            self.steps.append(("scatter_add", "scatter_add", (*args, int(self.deterministic))))
            self.views[v] = out
        elif op == "fusion":
            self.lower_fusion(n)
        else:
            raise NotImplementedError(f"no plan step for primitive {op} outside a fusion")

    def fusion_outputs(self, n: G.Node):
        """Values of a fusion's outputs: the node's own and its fusion_output nodes', by body output index."""
        body: G.Graph = n.params["body"]
        outs = [n.output] + [None] * (len(body.outputs) - 1)
        for u in self.uses.get(n.output, []):
            if u.op == "fusion_output":
                outs[u.params["index"]] = u.output
        return outs

    @staticmethod
    def dot_fusion_epilogue(body: G.Graph):
        """The tail of a `dot_general` fusion body as a GEMM epilogue: `(code, body input of the epilogue operand or
        None)`. 1: `max(product, 0)`; 2: `other + product`; 3: `select(0 < other, product, 0)` (a relu's backward
        with `other` the relu's output). Anything else has no kernel."""
        dots = [b for b in body.nodes if b.op == "dot_general"]
        if len(dots) != 1 or len(body.outputs) != 1:
            raise NotImplementedError("dot_general fusions are lowered for one product and one output")
        product = dots[0].output
        by_output = {b.output: b for b in body.nodes}
        def is_zero(value):  # a number in a traced body, "i:.." / "f:.." text in a parsed one
            if isinstance(value, str):
                kind, _, text = value.partition(":")
                return (float.fromhex(text) if kind == "f" else int(text)) == 0
            return value == 0

        fills = {b.output for b in body.nodes if b.op == "full" and is_zero(b.params.get("fill_value"))}
        zeros = {b.output for b in body.nodes if b.op == "broadcast_in_dim" and b.inputs[0] in fills}
        tail = by_output.get(body.outputs[0])
        used = {dots[0].output: dots[0]}
        if tail is not None and tail.op == "max" and product in tail.inputs and any(i in zeros for i in tail.inputs):
            code, other = 1, None
        elif tail is not None and tail.op == "add" and product in tail.inputs:
            (other,) = [i for i in tail.inputs if i != product] or [None]
            code = 2
        elif tail is not None and tail.op == "select" and tail.inputs[1] == product and tail.inputs[2] in zeros:
            cond = by_output.get(tail.inputs[0])
            if cond is None or cond.op != "lt" or cond.inputs[0] not in zeros:
                raise NotImplementedError("dot_general fusion: the select's condition is not `0 < operand`")
            code, other = 3, cond.inputs[1]
            used[cond.output] = cond
        else:
            raise NotImplementedError("dot_general fusions are lowered for a relu, an add or a relu-backward select after the product")
        used[tail.output] = tail
        for b in body.nodes:
            if b.output not in used and b.op not in ("full", "broadcast_in_dim"):
                raise NotImplementedError(f"dot_general fusion: no epilogue for primitive {b.op}")
        if other is not None and other not in body.inputs:
            raise NotImplementedError("dot_general fusion: the epilogue operand must be an input of the fusion")
        return dots[0], code, other

    def lower_dot(self, dot: G.Node, holder: G.Node, out_value: int, relu, operands=None, aux_value=None):
        g = self.g
        lhs_v, rhs_v = operands if operands else dot.inputs
        lhs, rhs = self.views[lhs_v], self.views[rhs_v]
        p = dot.params
        if p["lhs_batch"] or p["rhs_batch"] or len(lhs.shape) != 2 or len(rhs.shape) != 2:
            raise NotImplementedError("dot_general outside attention is lowered for 2-d operands without batch dimensions")
        (lc,), (rc,) = p["lhs_contracting"], p["rhs_contracting"]
        a = lhs if lc == 1 else View(lhs.buffer, lhs.offset, lhs.dtype, lhs.shape[::-1], lhs.strides[::-1])
        b = rhs if rc == 0 else View(rhs.buffer, rhs.offset, rhs.dtype, rhs.shape[::-1], rhs.strides[::-1])
        b = self.k_major_copy(b, a.shape[0])
        out = self.fresh(out_value)
        nbytes = gemm_scratch_bytes(a.shape[0], b.shape[1], a.shape[1])
        scratch = View(self.new_buffer(nbytes), 0, "uint8", (nbytes,), (1,)) if nbytes else None
        code = int(relu)
        aux = self.views[aux_value] if aux_value is not None else None
        if aux is not None and (aux.shape != out.shape or aux.dtype != out.dtype or aux.strides[-1] != 1):
            raise NotImplementedError("dot_general fusion: the epilogue operand must be row-major and shaped like the product")
        for x in (a, b, out, *([scratch] if scratch else []), *([aux] if aux else [])):
            self.touch(x)
        label = {0: "dot_general", 1: "dot_general_relu", 2: "dot_general_add", 3: "dot_general_relu_backward"}[code]
        self.steps.append(("gemm", label, (a, b, out, code, scratch, aux)))
        self.views[out_value] = out

    def dense_operand(self, value: int, label: str) -> View:
        """The view of `value` if it is dense, else a dense copy made once: by a `transpose` step for 2-d views whose two
        dimensions are swapped (which is what transposed weights and cotangents are), by a `copy` step for any other."""
        view = self.views[value]
        if view.dense and view.offset % 16 == 0:
            return view
        live = [(n, s) for n, s in zip(view.shape, view.strides) if n != 1]
        # (a dense slice that starts inside a 16-byte line - rows of 24 bytes, from row 1 - is copied to an aligned place
        # like any other view: generated kernels load whole lines)
        if not view.dense and len(live) == 2 and live[0][1] == 1 and live[1][1] == live[0][0] and SIZE_OF[view.dtype] in (2, 4):
            rows, cols = live[1][0], live[0][0]  # the memory is a dense [rows, cols]; the value is its transpose [cols, rows]
            src = View(view.buffer, view.offset, view.dtype, (rows, cols), (cols, 1))
            copy = View(self.new_buffer(rows * cols * SIZE_OF[view.dtype]), 0, view.dtype, (cols, rows), (rows, 1))
            self.touch(src)
            self.touch(copy)
            self.steps.append(("transpose", "materialize_transpose", (src, copy)))
            dense = View(copy.buffer, 0, view.dtype, view.shape, dense_strides(view.shape))
            self.views[value] = dense  # later readers use the copy too
            return dense
        # any other view (a slice, a permutation of more axes): a dense copy made by the copy step's strided kernel
        copy = View(self.new_buffer(math.prod(view.shape) * SIZE_OF[view.dtype]), 0, view.dtype, view.shape, dense_strides(view.shape))
        self.touch(view)
        self.touch(copy)
        self.steps.append(("copy", "materialize_view", (view, copy)))
        self.views[value] = copy
        return copy

    def k_major_copy(self, b: View, m: int) -> View:
        """`b` [K, N], or a transposed copy of it. A weight whose K rows lie 8 KB or more apart (N contiguous, N >= 4096
        16-bit elements) is a slow TMA operand: every 128-byte row of a tile comes from a different DRAM page and the
        power-of-two stride camps on few L2 slices (measured: [131072, 4096, 1024] runs at 900 TFLOP/s with such a B
        against 1280 with a K-major one). Transposing the weight once per step costs microseconds."""
        k, n = b.shape
        size = G.SIZE_OF[b.dtype]
        if not (b.strides == (n, 1) and size == 2 and n * size >= 8192 and k * n * size <= (64 << 20) and m >= 8 * k):
            return b
        copy = View(self.new_buffer(k * n * size), 0, b.dtype, (n, k), (k, 1))
        self.touch(b)
        self.touch(copy)
        self.steps.append(("transpose", "weight_transpose", (b, copy)))
        return View(copy.buffer, 0, b.dtype, (k, n), (1, k))

    def lower_fusion(self, n: G.Node):
        g = self.g
        name = n.params["name"]
        body: G.Graph = n.params["body"]
        label = n.params.get("label", name)
        outs = self.fusion_outputs(n)
        if name == "dot_general":
            dot, code, other = self.dot_fusion_epilogue(body)
            operands = [n.inputs[body.inputs.index(i)] for i in dot.inputs]
            aux_value = n.inputs[body.inputs.index(other)] if other is not None else None
            self.lower_dot(dot, n, n.output, code, operands=operands, aux_value=aux_value)
            return
        found = n.params.get("attention")  # set by the attention pass: roles of every operand's dimensions, scale, mask
        if name == "flash_attention" and found:
            def as_bsnh(view: View, roles: str) -> View:
                order = [roles.index(r) for r in "BSNH"]
                return View(view.buffer, view.offset, view.dtype, tuple(view.shape[d] for d in order), tuple(view.strides[d] for d in order))

            q, k, v = (as_bsnh(self.views[x], found[r]) for x, r in zip(n.inputs, "qkv"))
            if q.strides[3] != 1 or k.strides[3] != 1 or v.strides[3] != 1:
                raise NotImplementedError("flash_attention: the head dimension of q, k and v must be contiguous in memory")
            o_dense = self.fresh(outs[0])
            o = as_bsnh(o_dense, found["o"])
            b, sq, nh, _ = q.shape
            lse_value = outs[1] if len(outs) > 1 else None
            lse = View((self.out_target.get(lse_value) if lse_value is not None else None) or self.new_buffer(b * nh * sq * 4), 0,
                       "float32", (b, nh, sq), dense_strides((b, nh, sq)))
            for x in (q, k, v, o, lse):
                self.touch(x)
            self.steps.append(("attn_fwd", "flash_attention", (q, k, v, o, lse, found["scale"], found["causal"], found["offset"])))
            self.views[outs[0]] = o_dense
            if lse_value is not None:
                t = g.types[lse_value]
                self.views[lse_value] = View(lse.buffer, 0, "float32", t.shape, dense_strides(t.shape))
            return
        if name == "flash_attention":
            q, k, v = (self.views[x] for x in n.inputs)
            o = self.fresh(outs[0])
            lse_t = g.types[outs[1]] if outs[1] is not None else None
            b, sq, nh, _ = q.shape
            lse_shape = (b, nh, sq)
            lse = View((self.out_target.get(outs[1]) if outs[1] is not None else None) or self.new_buffer(b * nh * sq * 4), 0, "float32",
                       lse_shape, dense_strides(lse_shape))
            scale, causal, offset = attention_params(body)
            for x in (q, k, v, o, lse):
                self.touch(x)
            self.steps.append(("attn_fwd", "flash_attention", (q, k, v, o, lse, scale, causal, offset)))
            self.views[outs[0]] = o
            if outs[1] is not None:
                self.views[outs[1]] = View(lse.buffer, 0, "float32", lse_t.shape, dense_strides(lse_t.shape))
            return
        if name == "flash_attention_backward":
            q, k, v, o, lse, do = (self.views[x] for x in n.inputs)
            b, sq, nh, _ = q.shape
            lse3 = View(lse.buffer, lse.offset, "float32", (b, nh, sq), dense_strides((b, nh, sq)))
            delta = View(self.new_buffer(b * nh * sq * 4), 0, "float32", (b, nh, sq), dense_strides((b, nh, sq)))
            grads = [self.fresh(x) for x in outs]
            scale, causal, offset = (found["scale"], found["causal"], found["offset"]) if found else attention_params(body)
            args = (q, k, v, o, do, lse3, delta, *grads)
            if not self.deterministic and q.dtype == "bfloat16" and q.shape[3] == 64:
                # the single-kernel backward: dQ summed atomically over the key blocks in a float32 accumulator
                acc_shape = tuple(q.shape)
                args += (View(self.new_buffer(b * sq * nh * 64 * 4), 0, "float32", acc_shape, dense_strides(acc_shape)),)
            for x in args:
                self.touch(x)
            self.steps.append(("attn_bwd", "flash_attention_backward", (*args, scale, causal, offset)))
            for x, view in zip(outs, grads):
                self.views[x] = view
            return
        if name not in ROW_FUSIONS:
            raise NotImplementedError(f"no kernel for fusion {name}")
        ins = [self.dense_operand(x, label) for x in n.inputs]
        out_views = []
        inplace = False
        for x in outs:
            if x is None:
                raise NotImplementedError(f"fusion {label}: an unused fusion output")
            view = self.fresh(x)
            if not view.dense:
                raise NotImplementedError(f"fusion {label}: output placed in a strided slot")
            inplace |= any(view.buffer is i.buffer for i in ins)
            out_views.append(view)
        if all(math.prod(v.shape) == 0 for v in out_views):
            # nothing to compute (an empty batch): no kernel is generated and no step queued, as the reference skips a
            # zero-size grid (lumen/runtime/kernel/cuda/mod.rs:131-133)
            for x, view in zip(outs, out_views):
                self.views[x] = view
            return
        module = self.module(body, inplace)
        scratch = None
        nbytes = fusion_scratch_bytes(self.modules[module])
        if nbytes:
            scratch = View(self.new_buffer(nbytes), 0, "uint8", (nbytes,), (1,))
        for x in (*ins, *out_views, *([scratch] if scratch else [])):
            self.touch(x)
        self.steps.append(("fusion", label, (module, scratch, [*ins, *out_views])))
        for x, view in zip(outs, out_views):
            self.views[x] = view

    # ---- placement and text -------------------------------------------------------------------------------------
    def place(self) -> tuple[int, int]:
        end = len(self.steps)
        work = [b for b in self.buffers if b.kind == "w"]
        for b in work:
            if b.pinned_end or b.arena:
                b.last = end
        offset = 0
        arena = [b for b in work if b.arena]
        for b in arena:  # in order of creation = order of production in the backward pass
            b.offset = offset
            offset += -(-b.nbytes // ALIGN) * ALIGN
        arena_bytes = offset
        placed: list[Buffer] = []
        top = arena_bytes
        for b in sorted((b for b in work if not b.arena), key=lambda b: -b.nbytes):
            size = -(-b.nbytes // ALIGN) * ALIGN
            spans = sorted((p.offset, p.offset + -(-p.nbytes // ALIGN) * ALIGN) for p in placed if not (p.last < b.first or b.last < p.first))
            at = arena_bytes
            for lo, hi in spans:
                if at + size <= lo:
                    break
                at = max(at, hi)
            b.offset = at
            placed.append(b)
            top = max(top, at + size)
        return top, arena_bytes

    # ---- collectives as steps ---------------------------------------------------------------------------------------
    @staticmethod
    def step_views(payload):
        """Every View a step's payload holds."""
        if isinstance(payload, View):
            yield payload
        elif isinstance(payload, (tuple, list)):
            for item in payload:
                yield from Lowering.step_views(item)

    def insert_collectives(self):
        """Cuts the all-reduced gradients (contiguous in the arena, in order of production) into buckets of at least
        `bucket_bytes` and turns each into two steps: `all_reduce` of the bucket as one flat tensor, queued right after
        the step that produces its last gradient, and `wait`, placed before the first later step that touches one of
        its gradients (alignment padding between gradients is reduced along with them and never read). Every rank
        compiles the same plan, so every rank queues the same collectives in the same order."""
        buckets, current = [], None
        for c in sorted(self.comms, key=lambda c: c.view.buffer.offset):
            start = c.view.buffer.offset + c.view.offset
            end = start + -(-c.view.buffer.nbytes // ALIGN) * ALIGN
            same = current is not None and current["end"] == start and current["dtype"] == c.view.dtype and current["op"] == c.op
            if not same or current["end"] - current["start"] >= self.bucket_bytes:
                current = {"start": start, "end": end, "ready": c.ready_step, "dtype": c.view.dtype, "op": c.op, "buffers": [c.view.buffer]}
                buckets.append(current)
            else:
                current["end"], current["ready"] = end, max(current["ready"], c.ready_step)
                current["buffers"].append(c.view.buffer)
        buckets.sort(key=lambda b: b["ready"])
        touched = [{id(v.buffer) for v in self.step_views(payload)} for _, _, payload in self.steps]
        before: dict[int, list] = {}
        ops = {"sum": 0, "prod": 1, "max": 2, "min": 3}
        for k, b in enumerate(buckets):
            mine = {id(buf) for buf in b["buffers"]}
            first_use = next((i for i in range(b["ready"], len(self.steps)) if touched[i] & mine), len(self.steps))
            flat = View(Buffer("w", 0, b["end"] - b["start"], offset=b["start"]), 0, b["dtype"],
                        ((b["end"] - b["start"]) // SIZE_OF[b["dtype"]],), (1,))
            before.setdefault(b["ready"], []).append((0, k, ("all_reduce", "all_reduce", (flat, ops[b["op"]]))))
            before.setdefault(first_use, []).append((1, k, ("wait", "device_wait", (k,))))
        steps = []
        for i in range(len(self.steps) + 1):
            steps += [step for _, _, step in sorted(before.get(i, []), key=lambda t: (t[0], t[1]))]
            if i < len(self.steps):
                steps.append(self.steps[i])
        self.steps = steps
        return [{k: v for k, v in b.items() if k != "buffers"} for b in buckets]

    # ---- horizontal fusion ------------------------------------------------------------------------------------------
    ELEMENTWISE = {"add", "sub", "mul", "div", "max", "min", "neg", "abs", "sign", "exp", "log", "sqrt", "rsqrt", "tanh", "logistic",
                   "cast", "select", "eq", "lt", "not", "and", "or"}

    @staticmethod
    def flat_signature(body: G.Graph):
        """`(signature, shape)` of a body that is elementwise over ONE shape (every other value a scalar - a constant
        or a 0-d operand such as a run-time learning rate or step count - broadcast to it), else None: bodies with
        equal signatures are the same kernel up to that shape."""
        shape = None
        for v in body.inputs:
            if body.types[v].shape == ():
                continue
            if shape is None:
                shape = body.types[v].shape
            if body.types[v].shape != shape:
                return None
        if shape is None or shape == ():
            return None
        for n in body.nodes:
            t = body.types[n.output]
            if n.op == "full":
                if t.shape != ():
                    return None
            elif n.op == "broadcast_in_dim":
                if body.types[n.inputs[0]].shape != () or t.shape != shape:
                    return None
            elif n.op in Lowering.ELEMENTWISE:
                if t.shape != shape and t.shape != ():  # scalar arithmetic on 0-d operands stays scalar
                    return None
            else:
                return None
        if any(body.types[v].shape != shape for v in body.outputs):
            return None
        # the body over a placeholder shape no real tensor has: equal texts = the same program up to its shape
        text = Lowering.reshaped_body(body, shape, (1, 7919)).to_text()
        return text, shape

    @staticmethod
    def reshaped_body(body: G.Graph, shape, new_shape) -> G.Graph:
        """The elementwise `body` over `new_shape` instead of `shape` (same primitives, same constants)."""
        out = G.Graph()
        out.types = [G.TensorType(t.dtype, new_shape) if t.shape == shape else t for t in body.types]
        out.inputs, out.outputs = list(body.inputs), list(body.outputs)
        for n in body.nodes:
            params = dict(n.params)
            if "shape" in params and tuple(params["shape"]) == tuple(shape):
                params["shape"] = tuple(new_shape)
            out.nodes.append(G.Node(n.op, n.inputs, n.output, params))
        return out

    def fuse_horizontally(self):
        """Replaces every run of two or more consecutive, mutually independent `fusion` steps whose bodies are the same
        elementwise program up to its shape by ONE `multi` step: a kernel generated once for rows of `C` elements (`C`
        the greatest common divisor of the members' sizes, at most 4096) that takes every member's tensors and row
        count from a table. The training step's per-parameter optimizer updates become one launch per gradient
        bucket."""
        steps, i = [], 0
        while i < len(self.steps):
            kind, label, payload = self.steps[i]
            sig = None
            if kind == "fusion" and payload[1] is None:
                body, inplace = self.bodies[payload[0]]
                found = self.flat_signature(body)
                sig = (found[0], inplace) if found else None
            if sig is None:
                steps.append(self.steps[i])
                i += 1
                continue
            run, written, seen = [], set(), set()
            j = i
            while j < len(self.steps):
                k2, _, p2 = self.steps[j]
                if k2 != "fusion" or p2[1] is not None:
                    break
                b2, inplace2 = self.bodies[p2[0]]
                f2 = self.flat_signature(b2)
                if not f2 or (f2[0], inplace2) != sig:
                    break
                tensors = p2[2]
                n_in = len(b2.inputs)
                ins = {id(t.buffer) for t in tensors[:n_in]}
                outs = {id(t.buffer) for t in tensors[n_in:]}
                if (ins | outs) & written or outs & seen:  # depends on, or overwrites something of, an earlier member
                    break
                written |= outs
                seen |= ins | outs
                run.append((b2, tensors))
                j += 1
            if len(run) < 2:
                steps.append(self.steps[i])
                i += 1
                continue
            body0, _ = self.bodies[payload[0]]
            full = next(k for k, v in enumerate(body0.inputs) if body0.types[v].shape != ())  # the first full-shape operand
            cols = math.gcd(*[math.prod(tensors[full].shape) for _, tensors in run])
            while cols > 4096 and cols % 2 == 0:
                cols //= 2
            shape0 = body0.types[body0.inputs[full]].shape
            flat = self.reshaped_body(body0, shape0, (2, cols))  # two rows: one row would read as a row-constant operand
            text = ("option inplace\n" if sig[1] else "") + "option multi\n" + flat.to_text()
            if text not in self.module_index:
                self.module_index[text] = len(self.modules)
                self.modules.append(text)
            groups = [tensors for _, tensors in run]
            steps.append(("multi", f"{label}_x{len(run)}", (self.module_index[text], groups)))
            i = j
        self.steps = steps

    def emit(self) -> CompiledPlan:
        workspace, arena_bytes = self.place()
        buckets = self.insert_collectives() if self.comms else []
        if self.horizontal:
            self.fuse_horizontally()
        lines = []
        for k, text in enumerate(self.modules):
            lines.append(f"module {k}\n{text}endmodule\n")
        lines.append(f"plan {len(self.g.inputs)} {len(self.g.outputs)} {workspace}\n")
        ids: dict[int, int] = {}
        tensor_lines = []

        def tid(view: View) -> int:
            key = id(view)
            if key not in ids:
                ids[key] = len(ids)
                base = "w" if view.buffer.kind == "w" else f"{view.buffer.kind}{view.buffer.index}"
                off = view.offset + (view.buffer.offset if view.buffer.kind == "w" else 0)
                dims = " ".join(map(str, view.shape))
                strides = " ".join(map(str, view.strides))
                tensor_lines.append(f"t {ids[key]} {view.dtype} {base} {off} {len(view.shape)} {dims} {strides}".rstrip() + "\n")
            return ids[key]

        step_lines, labels = [], []
        launches = 0
        for kind, label, payload in self.steps:
            labels.append(label)
            if kind == "fusion":
                launches += 2 if payload[1] else 1  # scratch: partial sums + finalize
            elif kind == "multi":
                launches += 1  # one horizontally fused launch (tables of up to ~100 groups)
            elif kind == "gemm":
                launches += 2 if payload[4] else 1  # scratch: split-K partial tiles + reduction
            elif kind == "attn_bwd":
                launches += 3  # delta, dK/dV, dQ
            elif kind in ("attn_fwd",):
                launches += 1
            elif kind == "scatter_add":
                launches += 4 if payload[5] else 2  # count, starts, place, rows | float32 atomics, then one rounding
            elif kind == "transpose":
                launches += 1
            if kind == "fusion":
                module, scratch, tensors = payload
                args = " ".join(str(tid(t)) for t in tensors)
                step_lines.append(f"s fusion {label} {module} {tid(scratch) if scratch else -1} {len(tensors)} {args}\n")
            elif kind == "multi":
                module, groups = payload
                args = " ".join(str(tid(t)) for tensors in groups for t in tensors)
                step_lines.append(f"s multi {label} {module} {len(groups)} {args}\n")
            elif kind == "all_reduce":
                view, op = payload
                step_lines.append(f"s all_reduce {label} {tid(view)} {op}\n")
            elif kind == "wait":
                step_lines.append(f"s wait {label} {payload[0]}\n")
            elif kind == "gemm":
                a, b, d, epi, scratch, aux = payload
                step_lines.append(f"s gemm {label} {tid(a)} {tid(b)} {tid(d)} {epi} {tid(scratch) if scratch else -1} {tid(aux) if aux else -1}\n")
            elif kind in ("attn_fwd", "attn_bwd"):
                *tensors, scale, causal, offset = payload
                args = " ".join(str(tid(t)) for t in tensors)
                step_lines.append(f"s {kind} {label} {args} {float(scale).hex()} {int(causal)} {offset}\n")
            elif kind == "scatter_add":
                x, idx, upd, out, scratch, det = payload
                step_lines.append(f"s scatter_add {label} {tid(x) if x else -1} {tid(idx)} {tid(upd)} {tid(out)} {tid(scratch)} {det}\n")
            elif kind == "copy":
                src, dst = payload
                step_lines.append(f"s copy {label} {tid(src)} {tid(dst)}\n")
            elif kind == "transpose":
                src, dst = payload
                step_lines.append(f"s transpose {label} {tid(src)} {tid(dst)}\n")
            elif kind == "fill":
                view, byte = payload
                step_lines.append(f"s fill {label} {tid(view)} {byte}\n")
        text = "".join(lines) + "".join(tensor_lines) + "".join(step_lines) + "end\n"
        return CompiledPlan(text, workspace, len(self.g.inputs), len(self.g.outputs), self.comms, arena_bytes, labels, launches, buckets)


def attention_params(body: G.Graph):
    """Scale, causal flag and causal offset of a traced attention body: the constant multiplying the scores
    (`Score::Mul`, lumen/codegen/attention/cuda/mod.rs:45-60) and the iota comparison's shift."""
    scale, causal, offset = 1.0, False, 0
    dot_outputs = {n.output for n in body.nodes if n.op == "dot_general"}
    consts = {n.output: n.params["fill_value"] for n in body.nodes if n.op == "full"}
    bcast = {n.output: n.inputs[0] for n in body.nodes if n.op == "broadcast_in_dim"}

    def const_of(v):
        v = bcast.get(v, v)
        return consts.get(v)

    for n in body.nodes:
        if n.op == "mul" and scale == 1.0 and any(i in dot_outputs for i in n.inputs):
            c = [const_of(i) for i in n.inputs if i not in dot_outputs]
            if c and c[0] is not None:
                scale = float(c[0])
        if n.op == "iota":
            causal = True
        if n.op == "add" and causal:
            c = [const_of(i) for i in n.inputs]
            ints = [x for x in c if isinstance(x, int) and not isinstance(x, bool)]
            if ints and body.types[n.output].dtype == "int64":
                offset = ints[0]
    return scale, causal, offset


def gemm_scratch_bytes(m: int, n: int, k: int) -> int:
    """Split-K scratch the backend wants for an [m, k] x [k, n] product (0 when it does not split)."""
    from lumen_b200 import _lib

    return _lib.lib().lb_gemm_scratch_bytes(m, n, k, 1)


_SCRATCH_CACHE: dict[str, int] = {}


def fusion_scratch_bytes(module_text: str) -> int:
    """Scratch bytes the generated kernel for this body needs (asks the backend, which also compiles it)."""
    if module_text not in _SCRATCH_CACHE:
        import ctypes

        from lumen_b200 import _lib

        handle = ctypes.c_void_p()
        _lib.check(_lib.lib().lb_fusion_compile(module_text.encode(), ctypes.byref(handle)))
        _SCRATCH_CACHE[module_text] = _lib.lib().lb_fusion_scratch_bytes(handle)
    return _SCRATCH_CACHE[module_text]


def compile_graph(graph: G.Graph, donate: dict[int, int] | None = None, fuse: bool = True, deterministic: bool = True,
                  bucket_bytes: int = 64 << 20, horizontal: bool = True) -> CompiledPlan:
    """`graph` lowered to plan text. `donate[k] = j` writes output `k` into input `j`'s buffer. Bare elementwise and
    reduction prims are first grouped into fusions by the fusion pass (`lumen_b200.fusion_pass`). `deterministic`
    (the reference's config flag of that name, lumen/graph_compiler/config/mod.rs:117) picks the sorted scatter-add,
    which adds colliding rows in update order like the interpreter; without it they are added with atomics.
    All-reduced gradients are reduced in buckets of at least `bucket_bytes`; `horizontal` merges runs of same-bodied
    elementwise fusions (the optimizer updates) into single launches."""
    if fuse:
        from lumen_b200.attention_pass import match_attention
        from lumen_b200.fusion_pass import fuse as run_fusion_pass
        from lumen_b200.simplify import clean

        # dce / cse / simplify, then the attention passes, then fusion (the reference's pipeline order for its CUDA
        # device, lumen/graph_compiler/mod.rs:101-118)
        graph = run_fusion_pass(match_attention(clean(graph)))
    return Lowering(graph, donate, deterministic, bucket_bytes, horizontal).run()


def gradient_buckets(compiled: CompiledPlan, bucket_bytes: int = 64 << 20) -> list[dict]:
    """Groups the all-reduced gradients (contiguous in the arena, in order of production) into buckets of at least
    `bucket_bytes`: `{"start", "end"}` byte range of the workspace and `"ready"`, the step index after which the
    whole bucket has been produced. Sorted by readiness, the order in which the host reduces them. Every rank
    compiles the same plan, so every rank issues the same collectives in the same order
    (lumen/graph_compiler/schedule.rs:17-41)."""
    buckets, current = [], None
    for c in sorted(compiled.comms, key=lambda c: c.view.buffer.offset):
        start = c.view.buffer.offset + c.view.offset
        end = start + -(-c.view.buffer.nbytes // ALIGN) * ALIGN
        if current is None or current["end"] != start or current["end"] - current["start"] >= bucket_bytes:
            current = {"start": start, "end": end, "ready": c.ready_step}
            buckets.append(current)
        else:
            current["end"], current["ready"] = end, max(current["ready"], c.ready_step)
    return sorted(buckets, key=lambda b: b["ready"])
