"""The clean-up passes that run before fusion: dead-code elimination, common-subexpression elimination and a few
value-preserving simplifications - the counterparts of the reference's `cse` and `simplify` passes
(lumen/graph_compiler/passes/cse.rs, simplify.rs:163-179), which every device pipeline (the CPU's included) runs.

Every rewrite here leaves each remaining value bit-identical when the graph is evaluated primitive by primitive
(the reference requires that of every pass, lumen/reference/README.md:15):

* `dce`: nodes whose value reaches no output are dropped (autograd traces cotangents nobody asked for);
* `cse`: a node equal to an earlier one - same primitive, operands and parameters - reuses that value (the backward
  pass re-traces broadcasts, iotas and constants the forward already has);
* `simplify`: `reshape` to the operand's own shape, `transpose` by the identity, `cast` to the operand's own dtype and
  `broadcast_in_dim` to the same shape are removed; a transpose of a transpose becomes one; a reshape of a reshape
  becomes one; `cast(dot_general(..), t)` with the product used nowhere else becomes the product's `output_dtype`
  (the accumulator is rounded once either way).
"""

from __future__ import annotations

from lumen_b200 import graph as G


def _copy(graph: G.Graph) -> G.Graph:
    out = G.Graph()
    out.types, out.inputs, out.outputs, out.nodes = list(graph.types), list(graph.inputs), list(graph.outputs), list(graph.nodes)
    return out


def dce(graph: G.Graph) -> G.Graph:
    """`graph` without the nodes no output depends on. `fusion_output` nodes keep their fusion alive."""
    live = set(graph.outputs)
    keep = []
    for n in reversed(graph.nodes):
        if n.output in live:
            keep.append(n)
            live.update(n.inputs)
    # a fusion whose first output is dead but whose other outputs live: the fusion node itself carries output 0
    out = _copy(graph)
    out.nodes = keep[::-1]
    return out


def _key(n: G.Node, rename):
    def freeze(v):
        if isinstance(v, G.Graph):
            return ("graph", v.to_text())
        if isinstance(v, dict):
            return tuple(sorted((k, freeze(x)) for k, x in v.items()))
        if isinstance(v, (list, tuple)):
            return tuple(freeze(x) for x in v)
        if isinstance(v, float):
            return ("f", v.hex()) if v == v else ("f", "nan")
        return (type(v).__name__, v)

    return (n.op, tuple(rename.get(v, v) for v in n.inputs), tuple(sorted((k, freeze(v)) for k, v in n.params.items())))


def cse(graph: G.Graph) -> G.Graph:
    """Later nodes equal to an earlier one read the earlier value instead. Collectives are never merged."""
    rename: dict[int, int] = {}
    seen: dict = {}
    nodes = []
    for n in graph.nodes:
        inputs = tuple(rename.get(v, v) for v in n.inputs)
        if n.op in ("all_reduce", "device_wait", "host_wait"):
            nodes.append(G.Node(n.op, inputs, n.output, n.params))
            continue
        key = _key(n, rename)
        first = seen.get(key)
        if first is not None and graph.types[first] == graph.types[n.output] and n.output not in graph.outputs:
            rename[n.output] = first
            continue
        seen.setdefault(key, n.output)
        nodes.append(G.Node(n.op, inputs, n.output, n.params))
    out = _copy(graph)
    out.nodes = nodes
    out.outputs = [rename.get(v, v) for v in graph.outputs]
    return out


def simplify(graph: G.Graph) -> G.Graph:
    types = graph.types
    producer = {n.output: n for n in graph.nodes}
    uses: dict[int, int] = {}
    for n in graph.nodes:
        for v in n.inputs:
            uses[v] = uses.get(v, 0) + 1
    for v in graph.outputs:
        uses[v] = uses.get(v, 0) + 1
    rename: dict[int, int] = {}
    nodes = []
    dropped = set()

    def src(v):
        while v in rename:
            v = rename[v]
        return v

    for n in graph.nodes:
        inputs = tuple(src(v) for v in n.inputs)
        n = G.Node(n.op, inputs, n.output, dict(n.params))
        out_t = types[n.output]
        is_output = n.output in graph.outputs
        if not is_output and n.op in ("reshape", "broadcast_in_dim") and types[inputs[0]].shape == out_t.shape and (
                n.op == "reshape" or tuple(n.params["broadcast_dimensions"]) == tuple(range(len(out_t.shape)))):
            rename[n.output] = inputs[0]
            continue
        if not is_output and n.op == "transpose" and tuple(n.params["permutation"]) == tuple(range(len(out_t.shape))):
            rename[n.output] = inputs[0]
            continue
        if not is_output and n.op == "cast" and types[inputs[0]].dtype == out_t.dtype:
            rename[n.output] = inputs[0]
            continue
        inner = producer.get(inputs[0]) if inputs else None
        if n.op == "transpose" and inner is not None and inner.op == "transpose" and inner.output not in dropped:
            first = tuple(inner.params["permutation"])
            second = tuple(n.params["permutation"])
            n = G.Node("transpose", (src(inner.inputs[0]),), n.output, {"permutation": tuple(first[p] for p in second)})
        elif n.op == "reshape" and inner is not None and inner.op == "reshape" and inner.output not in dropped:
            n = G.Node("reshape", (src(inner.inputs[0]),), n.output, dict(n.params))
        elif (n.op == "cast" and inner is not None and inner.op == "dot_general" and uses.get(inner.output, 0) == 1
              and inner.params.get("output_dtype", inner.params["accum_dtype"]) == inner.params["accum_dtype"]
              and out_t.dtype == types[inner.inputs[0]].dtype and inner in nodes):
            # the product's accumulator rounded once to the operands' dtype: the cast becomes the product's output dtype
            at = nodes.index(inner)
            params = dict(inner.params)
            params["output_dtype"] = out_t.dtype
            nodes[at] = G.Node("dot_general", inner.inputs, n.output, params)
            producer[n.output] = nodes[at]
            dropped.add(inner.output)
            continue
        producer[n.output] = n
        nodes.append(n)
    out = _copy(graph)
    out.nodes = nodes
    out.outputs = [src(v) for v in graph.outputs]
    return out


LONGEST_ROW = 1 << 18  # elements one block of the row kernels reduces (64 chunks of 1024 threads x 4 elements)


def split_long_reductions(graph: G.Graph, limit: int = LONGEST_ROW) -> G.Graph:
    """A sum or maximum over every axis of a tensor of more than `limit` elements (a loss over many tokens, the square
    norm of a large gradient) becomes two reductions: the tensor seen as [N / C, C] is reduced over its rows - the
    column kernels spread that over the whole GPU - and the C partial results are reduced by one block. C is the
    largest divisor of N from 4096 down. Reductions over the trailing axes of a tensor that has leading axes too, with
    rows longer than `limit`, are cut into pieces per row likewise (C up to 16384). A length without a divisor of a
    useful size (a prime, twice a prime) is cut into a head of whole pieces of 4096 and a tail, reduced apart and
    combined. Unlike the passes above this changes the order in which a float sum adds its terms (to a shallower tree:
    the rounding error shrinks); the reference's reduction kernels split long reductions the same way
    (lumen/codegen/reduction/triton.rs)."""
    if not any(n.op in ("reduce_sum", "reduce_max") for n in graph.nodes):
        return graph
    out = _copy(graph)
    nodes = []

    def emit(op, inputs, dtype, shape, result=None, **params):
        if result is None:
            out.types.append(G.TensorType(dtype, tuple(shape)))
            result = len(out.types) - 1
        nodes.append(G.Node(op, tuple(inputs), result, params))
        return result

    for n in graph.nodes:
        if n.op not in ("reduce_sum", "reduce_max"):
            nodes.append(n)
            continue
        t, result_t = graph.types[n.inputs[0]], graph.types[n.output]
        rank = len(t.shape)
        axes = tuple(sorted(a % rank for a in n.params["axes"])) if rank else ()
        kept = rank - len(axes)
        length = 1
        for a in axes:
            length *= t.shape[a]
        if not axes or axes != tuple(range(kept, rank)) or length <= limit:
            nodes.append(n)  # short rows, or axes the row kernels do not take anyway
            continue
        outer = t.numel // length
        combine = "add" if n.op == "reduce_sum" else "max"

        def reduce(value, shape, axis, result=None):
            params = dict(n.params)
            params["axes"] = (axis,)
            return emit(n.op, (value,), result_t.dtype, tuple(d for k, d in enumerate(shape) if k != axis), result, **params)

        if outer == 1:
            cols = next(c for c in range(min(4096, length), 0, -1) if length % c == 0)
            if cols >= 64:
                rows_view = emit("reshape", (n.inputs[0],), t.dtype, (length // cols, cols), new_sizes=(length // cols, cols))
                reduce(reduce(rows_view, (length // cols, cols), 0), (cols,), 0, n.output)
                continue
            whole, rest = length // 4096, length % 4096
            flat = emit("reshape", (n.inputs[0],), t.dtype, (length,), new_sizes=(length,))
            head = emit("slice", (flat,), t.dtype, (whole * 4096,), start_indices=(0,), limit_indices=(whole * 4096,))
            head = emit("reshape", (head,), t.dtype, (whole, 4096), new_sizes=(whole, 4096))
            first = reduce(reduce(head, (whole, 4096), 0), (4096,), 0)
            tail = emit("slice", (flat,), t.dtype, (rest,), start_indices=(whole * 4096,), limit_indices=(length,))
            emit(combine, (first, reduce(tail, (rest,), 0)), result_t.dtype, (), n.output)
            continue
        piece = next(c for c in range(min(16384, length), 0, -1) if length % c == 0)
        if piece >= 64 and length // piece <= limit:
            count = length // piece
            pieces = emit("reshape", (n.inputs[0],), t.dtype, (outer * count, piece), new_sizes=(outer * count, piece))
            partial = reduce(pieces, (outer * count, piece), 1)
            per_row = emit("reshape", (partial,), result_t.dtype, (outer, count), new_sizes=(outer, count))
            flat = reduce(per_row, (outer, count), 1)
            emit("reshape", (flat,), result_t.dtype, result_t.shape, n.output, new_sizes=tuple(result_t.shape))
            continue
        whole, rest = length // 4096, length % 4096
        if whole > limit:
            nodes.append(n)  # rows of more than 2^30 elements: left to the kernel's own message
            continue
        rows = emit("reshape", (n.inputs[0],), t.dtype, (outer, length), new_sizes=(outer, length))
        head = emit("slice", (rows,), t.dtype, (outer, whole * 4096), start_indices=(0, 0), limit_indices=(outer, whole * 4096))
        head = emit("reshape", (head,), t.dtype, (outer * whole, 4096), new_sizes=(outer * whole, 4096))  # a copy: rows lie `length` apart
        partial = reduce(head, (outer * whole, 4096), 1)
        per_row = emit("reshape", (partial,), result_t.dtype, (outer, whole), new_sizes=(outer, whole))
        first = reduce(per_row, (outer, whole), 1)
        tail = emit("slice", (rows,), t.dtype, (outer, rest), start_indices=(0, whole * 4096), limit_indices=(outer, length))
        both = emit(combine, (first, reduce(tail, (outer, rest), 1)), result_t.dtype, (outer,))
        emit("reshape", (both,), result_t.dtype, result_t.shape, n.output, new_sizes=tuple(result_t.shape))
    out.nodes = nodes
    return out


def clean(graph: G.Graph) -> G.Graph:
    """dce, cse and simplify to a fixed point (a few rounds at most), then dce again; whole-tensor reductions too long for
    one block are split last."""
    g = graph
    for _ in range(4):
        before = len(g.nodes)
        g = dce(simplify(cse(dce(g))))
        if len(g.nodes) == before:
            break
    return split_long_reductions(g)
