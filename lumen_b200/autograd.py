"""Reverse-mode differentiation of traced programs: `vjp`, `grad`, `value_and_grad` and `backward`, the transforms of
`lumen.autograd` (lumen/autograd/transforms.py:156-267) for the primitives this backend runs.

The reference differentiates by forward mode plus transposition; here the recorded nodes are walked once in reverse
and every primitive's vector-Jacobian product is traced as new strict prims into the same graph, so the derivative is
an ordinary traced program: the fusion pass groups it, the attention pass finds the FlashAttention-2 backward in it,
the oracle evaluates it. The rules that decide numerics follow the reference's (lumen/autograd/rules.py):

* `dot_general`: the cotangent is narrowed to the other operand's dtype - re-using the value a widening cast was made
  from - the gradient product accumulates in the forward product's accumulator and is written in the differentiated
  operand's dtype (rules.py:425-489);
* `cast`: the cotangent is cast back, except that a gradient which only exists as the narrowing of a wider product (the
  weight gradient of `x @ w.bfloat16()` with float32 `w`) hands over the wider value: one rounding fewer (rules.py:28-60);
* `max` splits a tie evenly (0.5 each), `reduce_max` averages over the positions equal to the maximum (rules.py:398-421).

`flash_attention` fusions (`F.flash_attention`) differentiate to the traced FlashAttention-2 backward
(lumen/functional/attention/flash.py:51-85) as one `flash_attention_backward` fusion.
"""

from __future__ import annotations

from lumen_b200 import functional as F
from lumen_b200 import graph as G
from lumen_b200 import prims
from lumen_b200.prims import TracedTensor
from lumen_b200.tracer import accum_dtype, broadcast_to, is_float


def _tensor(graph, var):
    return TracedTensor(graph, var)


def _full_like(x, value):
    prims.push_graph(x.graph)
    try:
        return broadcast_to(prims.full((), value, x.dtype), x.shape)
    finally:
        prims.pop_graph()


def _producer(graph, var):
    for n in reversed(graph.nodes):
        if n.output == var:
            return n
    return None


def _narrowed(ct, dtype):
    """`ct` in `dtype`: the value a widening cast made it from, else `ct` cast to it (rules.py:431-439)."""
    if ct.dtype == dtype:
        return ct
    n = _producer(ct.graph, ct.var)
    if n is not None and n.op == "cast" and ct.graph.types[n.inputs[0]].dtype == dtype:
        return _tensor(ct.graph, n.inputs[0])
    return prims.cast(ct, dtype)


def _widened(graph, var, dtype):
    """The `dtype` value that `var` is only the narrowing of (possibly transposed or summed), else None
    (rules.py:28-45)."""
    n = _producer(graph, var)
    if n is None:
        return None
    if n.op == "transpose":
        inner = _widened(graph, n.inputs[0], dtype)
        return None if inner is None else prims.transpose(inner, n.params["permutation"])
    if n.op == "add":
        x, y = (_widened(graph, i, dtype) for i in n.inputs)
        return None if x is None or y is None else prims.add(x, y)
    if n.op == "cast" and graph.types[n.inputs[0]].dtype == dtype:
        return _tensor(graph, n.inputs[0])
    return None


def _sum_to(ct, shape, dims_kept):
    """`ct` summed over the dimensions a broadcast added: back to `shape`, whose dimension k is `ct`'s `dims_kept[k]`."""
    axes = tuple(d for d in range(ct.ndim) if d not in dims_kept)
    acc = accum_dtype(ct.dtype)
    out = ct
    if axes:
        out = prims.reduce_sum(out if out.dtype == acc else out.to(acc), axes, acc)
        out = out if out.dtype == ct.dtype else out.to(ct.dtype)
    # dimensions of size 1 that were stretched
    kept_shape = tuple(ct.shape[d] for d in dims_kept)
    stretched = tuple(k for k, (have, want) in enumerate(zip(kept_shape, shape)) if want == 1 and have != 1)
    if stretched:
        wide = out if out.dtype == acc else out.to(acc)
        wide = prims.reduce_sum(wide, stretched, acc)
        out = (wide if wide.dtype == ct.dtype else wide.to(ct.dtype)).reshape(shape)
    return out


def _dot_operand_grad(ct, x, y, x_contract, y_contract, x_batch, y_batch, params, x_is_lhs):
    """The cotangent of operand `x` of `dot_general(x, y)` (or of `dot_general(y, x)` when not `x_is_lhs`): a product of the
    cotangent with the other operand, its dimensions put back in `x`'s order (rules.py:463-486)."""
    x_kept = [d for d in range(x.ndim) if d not in x_contract and d not in x_batch]
    y_kept = [d for d in range(y.ndim) if d not in y_contract and d not in y_batch]
    nb = len(x_batch)
    ans_batch = list(range(nb))
    if x_is_lhs:  # answer dims: batch, x kept, y kept
        ans_y = list(range(nb + len(x_kept), nb + len(x_kept) + len(y_kept)))
    else:  # answer dims: batch, y kept, x kept
        ans_y = list(range(nb, nb + len(y_kept)))
    ct = _narrowed(ct, y.dtype)
    dims = ((tuple(ans_y), tuple(y_kept)), (tuple(ans_batch), tuple(y_batch)))
    x_bar = F.dot(ct, y, dims, params["accum_dtype"], x.dtype)
    # x_bar's dims: batch, ct's remaining dims (= x kept), y's remaining dims (= y contracting, in y's order)
    order = sorted(range(len(y_contract)), key=lambda i: y_contract[i])
    have = list(x_batch) + x_kept + [x_contract[i] for i in order]
    perm = sorted(range(len(have)), key=have.__getitem__)
    return x_bar if perm == list(range(len(perm))) else prims.transpose(x_bar, perm)


class _Reverse:
    """One reverse sweep over the nodes a function recorded."""

    def __init__(self, graph: G.Graph, first_node: int, last_node: int):
        self.g = graph
        self.nodes = list(graph.nodes[first_node:last_node])
        self.ct: dict[int, TracedTensor] = {}
        self.pieces: dict[int, list] = {}  # var -> [(start indices, cotangent of that slice)], until the var is visited

    def add_slice(self, var, start, value):
        """The cotangent of `slice(var, start, ..)`: kept as a piece. Pieces that tile `var` along one dimension become
        ONE concatenation when `var` is visited (three slices of a packed q/k/v projection -> concat(dq, dk, dv)),
        anything else zeros-padded sums."""
        if is_float(self.g.types[var].dtype):
            self.pieces.setdefault(var, []).append((tuple(start), value))

    def flush(self, var):
        pieces = self.pieces.pop(var, None)
        if not pieces:
            return
        shape = self.g.types[var].shape
        for d in range(len(shape)):
            ordered = sorted(pieces, key=lambda piece: piece[0][d])
            at, ok = 0, True
            for start, value in ordered:
                same_elsewhere = all(start[k] == 0 and value.shape[k] == shape[k] for k in range(len(shape)) if k != d)
                if start[d] != at or not same_elsewhere:
                    ok = False
                    break
                at += value.shape[d]
            if ok and at == shape[d] and len(ordered) > 1:
                self.add(var, prims.concatenate([value for _, value in ordered], d))
                return
        x = _tensor(self.g, var)
        for start, value in pieces:
            self.add(var, self.pad_back(value, x, start))

    def add(self, var, value):
        if value is None or not is_float(self.g.types[var].dtype):
            return
        t = self.g.types[var]
        if value.dtype != t.dtype or value.shape != t.shape:
            raise RuntimeError(f"autograd: cotangent {value.type} for a value of type {t}")
        self.ct[var] = value if var not in self.ct else self.ct[var] + value

    def run(self, seeds: dict[int, TracedTensor]):
        for v, c in seeds.items():
            self.add(v, c)
        consumed = {}
        for n in self.nodes:  # fusion_output nodes hand their cotangent to their fusion
            if n.op == "fusion_output":
                consumed.setdefault(n.inputs[0], {})[n.params["index"]] = n.output
        for n in reversed(self.nodes):
            if n.op == "fusion_output":
                continue
            self.flush(n.output)
            extra = consumed.get(n.output, {}) if n.op == "fusion" else {}
            if n.output not in self.ct and not any(v in self.ct for v in extra.values()):
                continue
            self.node(n, extra)
        for var in list(self.pieces):  # slices of the primals themselves
            self.flush(var)
        return self.ct

    def node(self, n: G.Node, extra):
        g = self.g
        ct = self.ct.get(n.output)
        x = [_tensor(g, v) for v in n.inputs]
        out = _tensor(g, n.output)
        op, p = n.op, n.params
        give = lambda k, value: self.add(n.inputs[k], value)  # noqa: E731
        if op == "add":
            give(0, ct), give(1, ct)
        elif op == "sub":
            give(0, ct), give(1, prims.neg(ct))
        elif op == "neg":
            give(0, prims.neg(ct))
        elif op == "mul":
            give(0, prims.mul(ct, x[1])), give(1, prims.mul(x[0], ct))
        elif op == "div":
            give(0, prims.div(ct, x[1]))
            give(1, prims.mul(ct, prims.neg(prims.div(out, x[1]))))
        elif op == "max":
            for k in (0, 1):
                a, b = x[k], x[1 - k]
                share = prims.select(prims.lt(b, a), _full_like(a, 1.0), prims.select(prims.eq(a, b), _full_like(a, 0.5), _full_like(a, 0.0)))
                give(k, prims.mul(ct, share))
        elif op == "exp":
            give(0, prims.mul(ct, out))
        elif op == "log":
            give(0, prims.div(ct, x[0]))
        elif op == "sqrt":
            give(0, prims.div(ct, prims.add(out, out)))
        elif op == "rsqrt":  # d/dx x^-1/2 = -1/2 out / x
            give(0, prims.mul(ct, prims.mul(_full_like(out, -0.5), prims.div(out, x[0]))))
        elif op == "tanh":
            give(0, prims.mul(ct, prims.sub(_full_like(out, 1.0), prims.mul(out, out))))
        elif op == "logistic":
            give(0, prims.mul(ct, prims.mul(out, prims.sub(_full_like(out, 1.0), out))))
        elif op == "abs":
            give(0, prims.mul(ct, prims.sign(x[0])))
        elif op == "cast":
            if is_float(x[0].dtype):
                wide = _widened(g, ct.var, x[0].dtype) if x[0].dtype != ct.dtype else None
                give(0, wide if wide is not None else (ct if ct.dtype == x[0].dtype else prims.cast(ct, x[0].dtype)))
        elif op == "select":
            zero = _full_like(ct, 0.0)
            give(1, prims.select(x[0], ct, zero)), give(2, prims.select(x[0], zero, ct))
        elif op == "broadcast_in_dim":
            give(0, _sum_to(ct, x[0].shape, tuple(p["broadcast_dimensions"])))
        elif op == "reshape":
            give(0, prims.reshape(ct, x[0].shape))
        elif op == "transpose":
            perm = list(p["permutation"])
            give(0, prims.transpose(ct, sorted(range(len(perm)), key=perm.__getitem__)))
        elif op == "reduce_sum":
            kept = [d for d in range(x[0].ndim) if d not in p["axes"]]
            back = prims.broadcast_in_dim(ct, x[0].shape, kept)
            give(0, back if back.dtype == x[0].dtype else back.to(x[0].dtype))
        elif op == "reduce_max":
            kept = [d for d in range(x[0].ndim) if d not in p["axes"]]
            where = prims.cast(prims.eq(x[0], prims.broadcast_in_dim(out, x[0].shape, kept)), x[0].dtype)
            acc = accum_dtype(x[0].dtype)
            count = prims.reduce_sum(where if acc == x[0].dtype else where.to(acc), tuple(p["axes"]), acc)
            count = count if count.dtype == x[0].dtype else count.to(x[0].dtype)
            give(0, prims.mul(prims.broadcast_in_dim(prims.div(ct, count), x[0].shape, kept), where))
        elif op == "dot_general":
            lc, rc, lb, rb = (tuple(p[k]) for k in ("lhs_contracting", "rhs_contracting", "lhs_batch", "rhs_batch"))
            ctw = ct
            give(0, _dot_operand_grad(ctw, x[0], x[1], lc, rc, lb, rb, p, True))
            give(1, _dot_operand_grad(ctw, x[1], x[0], rc, lc, rb, lb, p, False))
        elif op == "gather":
            if p["axis"] != 0:
                raise NotImplementedError("autograd: gather is differentiated along axis 0 (rows of a table)")
            prims.push_graph(g)
            try:
                zeros = prims.full(x[0].shape, 0.0, x[0].dtype)
            finally:
                prims.pop_graph()
            give(0, prims.scatter_add(zeros, x[1], ct, 0))
        elif op == "scatter_add":
            give(0, ct)
            give(2, prims.gather(ct, x[1], p["axis"]))
        elif op == "slice":
            self.add_slice(n.inputs[0], p["start_indices"], ct)
        elif op == "concatenate":
            d, at = p["dimension"], 0
            for k, operand in enumerate(x):
                start = [0] * ct.ndim
                limit = list(ct.shape)
                start[d], limit[d] = at, at + operand.shape[d]
                give(k, prims.slice(ct, start, limit))
                at += operand.shape[d]
        elif op == "fusion" and p.get("name") == "flash_attention":
            self.attention(n, x, extra)
        elif op in ("full", "iota", "eq", "lt", "sign", "not", "and", "or", "is_finite", "floor", "ceil"):
            pass  # constants and piecewise-constant functions: no gradient flows
        else:
            raise NotImplementedError(f"autograd: no rule for primitive {op}" + (f" (fusion {p.get('name')})" if op == "fusion" else ""))

    def pad_back(self, ct, x, start):
        """The cotangent of a slice: `ct` placed at `start` in zeros of `x`'s shape (concatenations of zeros)."""
        g = self.g
        out = ct
        for d in range(x.ndim):
            before, after = start[d], x.shape[d] - start[d] - ct.shape[d]
            parts = []
            prims.push_graph(g)
            try:
                if before:
                    parts.append(prims.full(out.shape[:d] + (before,) + out.shape[d + 1:], 0.0, ct.dtype))
                parts.append(out)
                if after:
                    parts.append(prims.full(out.shape[:d] + (after,) + out.shape[d + 1:], 0.0, ct.dtype))
            finally:
                prims.pop_graph()
            if len(parts) > 1:
                out = prims.concatenate(parts, d)
        return out

    def attention(self, n, x, extra):
        """`F.flash_attention`'s backward: the traced FlashAttention-2 program as one fusion (flash.py:51-85)."""
        from lumen_b200.compiler import attention_params
        from lumen_b200.nn import fused

        g = self.g
        if any(v in self.ct for v in extra.values()):
            raise NotImplementedError("autograd: the log-sum-exp output of flash_attention is not differentiated")
        scale, causal, _ = attention_params(n.params["body"])
        lse_var = extra.get(1)
        if lse_var is None:
            raise NotImplementedError("autograd: flash_attention's backward needs its log-sum-exp output")
        q, k, v = x
        o, lse, do = _tensor(g, n.output), _tensor(g, lse_var), self.ct[n.output]
        dq, dk, dv = fused(lambda a, b, c, oo, ll, gg: F.attention_backward_prims(a, b, c, oo, ll, gg, scale, causal),
                           q, k, v, o, lse, do, name="flash_attention_backward")
        self.add(n.inputs[0], dq), self.add(n.inputs[1], dk), self.add(n.inputs[2], dv)


def _trace_inside(fn, args):
    graph = next(a.graph for a in args if isinstance(a, TracedTensor))
    first = len(graph.nodes)
    prims.push_graph(graph)
    try:
        out = fn(*args)
    finally:
        prims.pop_graph()
    return graph, first, len(graph.nodes), out


def vjp(fn, *primals):
    """`(fn(*primals), pull)` where `pull(cotangent)` returns the cotangents of the tensor `primals` (None for
    non-float ones), traced into the same graph (lumen/autograd/transforms.py:206-237)."""
    graph, first, last, out = _trace_inside(fn, primals)
    outs = out if isinstance(out, (tuple, list)) else (out,)

    def pull(*cotangents):
        if len(cotangents) != len(outs):
            raise TypeError(f"vjp: {len(outs)} outputs, {len(cotangents)} cotangents")
        prims.push_graph(graph)
        try:
            ct = _Reverse(graph, first, last).run({o.var: c for o, c in zip(outs, cotangents)})
        finally:
            prims.pop_graph()
        return tuple(ct.get(p.var) if isinstance(p, TracedTensor) else None for p in primals)

    return out, pull


def backward(out: TracedTensor, wrt, cotangent: TracedTensor | None = None):
    """The gradients of the scalar (or seeded) `out` with respect to the traced tensors `wrt`, differentiating every
    node recorded in `out`'s graph so far (lumen/autograd/transforms.py:156-168)."""
    graph = out.graph
    prims.push_graph(graph)
    try:
        if cotangent is None:
            if out.shape != ():
                raise RuntimeError("backward() of a tensor that is not a scalar needs a cotangent")
            cotangent = prims.full((), 1.0, out.dtype)
        ct = _Reverse(graph, 0, len(graph.nodes)).run({out.var: cotangent})
    finally:
        prims.pop_graph()
    return [ct.get(w.var) for w in wrt]


def value_and_grad(fn, argnums=0):
    """`fn` returning a floating-point scalar -> a function returning `(value, gradient(s))` with respect to the
    argument(s) `argnums` (lumen/autograd/transforms.py:240-264)."""
    many = isinstance(argnums, (tuple, list))
    which = tuple(argnums) if many else (argnums,)

    def wrapped(*args):
        value, pull = vjp(fn, *args)
        if not isinstance(value, TracedTensor) or value.shape != () or not is_float(value.dtype):
            raise RuntimeError("grad: the function must return one floating-point scalar")
        prims.push_graph(value.graph)
        try:
            seed = prims.full((), 1.0, value.dtype)
        finally:
            prims.pop_graph()
        cts = pull(seed)
        for k in which:
            if cts[k] is None:
                raise RuntimeError(f"grad: the value does not depend on argument {k} (or it is not a float tensor)")
        grads = tuple(cts[k] for k in which)
        return value, (grads if many else grads[0])

    return wrapped


def grad(fn, argnums=0):
    """`fn` returning a scalar -> a function returning its gradient(s) (lumen/autograd/transforms.py:267-275)."""
    vg = value_and_grad(fn, argnums)

    def wrapped(*args):
        return vg(*args)[1]

    return wrapped
