"""Differentiable building blocks of the transformer training step, traced as lumen graphs.

Every op below records prims: either directly in the outer graph (`dot_general`, `reshape`, `slice`,
`concatenate`, `scatter_add`) or inside a `fusion` node whose body is the op spelled in strict prims, named as the
reference's passes name their fusions (`elementwise`, `row`, `reduction`, `dot_general`, `flash_attention`,
`flash_attention_backward`; lumen/codegen/fusion/triton.rs:56-74, lumen/graph_compiler/passes/attention/mod.rs:29).
The reference reaches the same shape of graph by tracing prims and running its fusion / attention / diamond
passes; here the boundaries are drawn at trace time. Either way the CPU oracle evaluates the bodies primitive by
primitive, so the traced graph is its own specification.

Gradients are hand-derived per op and recorded on a tape, as the reference's `autograd.Function`s for attention,
cross entropy and norms are (lumen/functional/attention/flash.py:21-85, lumen/functional/cross_entropy/logits.py,
lumen/functional/functions.py `_RMSNorm`); the dot rule follows lumen/autograd/rules.py:425-489: the cotangent is
narrowed to the operands' dtype, the gradient accumulates in float32 and is written in the operand's dtype.
"""

from __future__ import annotations

import math

from lumen_b200 import functional as F
from lumen_b200 import graph as G
from lumen_b200 import prims
from lumen_b200.prims import TracedTensor


# ---- fusions ------------------------------------------------------------------------------------------------
def fused(fn, *inputs: TracedTensor, name: str = "elementwise", label: str = ""):
    """Traces `fn` on fresh inputs typed like `inputs` into a fusion body and applies it; returns the body's
    outputs as traced tensors of the outer graph (a list if `fn` returns several)."""
    body = G.Graph()
    prims.push_graph(body)
    try:
        args = [TracedTensor(body, body.add_input(t.dtype, t.shape)) for t in inputs]
        out = fn(*args)
    finally:
        prims.pop_graph()
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    body.set_outputs([o.var for o in outs])
    prims.push_graph(inputs[0].graph)
    try:
        result = prims.fusion(list(inputs), body, name, label or name)
    finally:
        prims.pop_graph()
    return result if isinstance(out, (tuple, list)) else result[0]


class Tape:
    """Backward closures in program order; `backward` walks them in reverse accumulating cotangents."""

    def __init__(self):
        self.entries = []  # (outputs, inputs, vjp)

    def record(self, outputs, inputs, vjp):
        self.entries.append((list(outputs), list(inputs), vjp))

    def backward(self, loss: TracedTensor, seed: TracedTensor | None = None):
        grads: dict[int, TracedTensor] = {}
        if seed is not None:
            grads[loss.var] = seed
        for outputs, inputs, vjp in reversed(self.entries):
            cots = [grads.get(o.var) for o in outputs]
            if all(c is None for c in cots) and not (len(outputs) == 1 and outputs[0].var == loss.var and seed is None):
                continue
            # A vjp marked `adds_into = k` takes the cotangent already accumulated for input k and returns the SUM:
            # the addition runs inside its own fusion (same primitives, same roundings) instead of a separate pass.
            k_fused = getattr(vjp, "adds_into", None)
            pending = None
            if k_fused is not None and inputs[k_fused] is not None and inputs[k_fused].var in grads:
                pending = grads.pop(inputs[k_fused].var)
            results = vjp(*cots, pending=pending) if k_fused is not None else vjp(*cots)
            for x, g in zip(inputs, results):
                if g is None or x is None:
                    continue
                if x.var in grads:
                    grads[x.var] = fused(lambda a, b: a + b, grads[x.var], g, label="grad_add")
                else:
                    grads[x.var] = g
        return grads


# ---- ops ------------------------------------------------------------------------------------------------------
def embedding(tape: Tape, tokens: TracedTensor, positions: TracedTensor, ids: TracedTensor) -> TracedTensor:
    """`tokens[ids] + positions` flattened to `[batch * seq, dim]` (examples/transformer.py:88-100); the gradient
    of `tokens` is a scatter-add, of `positions` a sum over the batch."""
    b, s = ids.shape
    d = tokens.shape[1]
    x = fused(lambda tok, pos, i: (tok[i] + pos).reshape(b * s, d), tokens, positions, ids, label="embedding")

    def vjp(dx):
        dx3 = dx.reshape(b, s, d)
        prims.push_graph(dx.graph)
        try:
            zeros = prims.full(tokens.shape, 0.0, tokens.dtype)
        finally:
            prims.pop_graph()
        dtok = prims.scatter_add(zeros, ids, dx3, 0)
        dpos = fused(lambda g: F.sum(g.float(), 0).to(g.dtype) if g.dtype != "float32" else F.sum(g, 0), dx3,
                     name="reduction", label="positions_grad")
        return dtok, dpos, None

    tape.record([x], [tokens, positions, ids], vjp)
    return x


def _ln_forward(x, w, b, eps):
    a, ww, bb = x.float(), w.float(), b.float()
    mean = F.mean(a, -1, keepdim=True)
    xc = a - mean
    var = F.mean(xc * xc, -1, keepdim=True)
    std = F.sqrt(var + eps)
    y = (xc / std * ww + bb).to(x.dtype)  # the reference tests' spelling of layer norm, in float32
    rows = x.shape[0]
    return y, mean.reshape(rows), (1.0 / std).reshape(rows)


def layer_norm(tape: Tape, x: TracedTensor, w: TracedTensor, b: TracedTensor, eps: float = 1e-5) -> TracedTensor:
    """Pre-LayerNorm with scale and bias over the last dimension, statistics in float32; one `row` fusion that also
    saves each row's mean and 1/std for the backward (a row fusion for dx, a column reduction for dw, db)."""
    rows, _ = x.shape
    y, mean, rstd = fused(lambda a, ww, bb: _ln_forward(a, ww, bb, eps), x, w, b, name="row", label="layer_norm")

    def vjp(dy, *_, pending=None):
        def dx_body(g, a, ww, mu, rs, *acc):
            gf = g.float() * ww.float()
            xhat = (a.float() - mu.reshape(rows, 1)) * rs.reshape(rows, 1)
            c1 = F.mean(gf, -1, keepdim=True)
            c2 = F.mean(gf * xhat, -1, keepdim=True)
            dx = ((gf - c1 - xhat * c2) * rs.reshape(rows, 1)).to(a.dtype)
            return acc[0] + dx if acc else dx  # the residual stream's cotangent, added as `grad_add` would

        def dwb_body(g, a, mu, rs):
            gf = g.float()
            xhat = (a.float() - mu.reshape(rows, 1)) * rs.reshape(rows, 1)
            return (prims.reduce_sum(gf * xhat, (0,), "float32").to(a.dtype), prims.reduce_sum(gf, (0,), "float32").to(a.dtype))

        extra = [pending] if pending is not None else []
        dx = fused(dx_body, dy, x, w, mean, rstd, *extra, name="row", label="layer_norm_backward")
        dw, db = fused(dwb_body, dy, x, mean, rstd, name="reduction", label="layer_norm_weight_grads")
        return dx, dw, db

    vjp.adds_into = 0
    tape.record([y], [x, w, b], vjp)
    return y


def linear(tape: Tape, x: TracedTensor, w: TracedTensor, output_dtype: str | None = None, relu: bool = False,
           residual: TracedTensor | None = None) -> TracedTensor:
    """`x @ w.t()` for `x` `[rows, in]` and `w` `[out, in]`, accumulated in float32, written as `output_dtype`
    (the operands' by default): `F.matmul(x, w.t(), "float32", dtype)` (examples/transformer.py:116-121). A
    `dot_general` fusion carries an elementwise tail into the GEMM's epilogue, as the reference's fusion pass does
    (lumen/codegen/fusion/triton.rs:56-74): `relu`, and `residual + product` for 16-bit models. In the backward of a
    16-bit model, the product that yields the cotangent of a relu output is masked by that output in its epilogue
    (the relu's own backward), instead of in a separate pass over the activations."""
    out_dtype = output_dtype or x.dtype
    if residual is not None and out_dtype == "float32":
        return add(tape, residual, linear(tape, x, w, output_dtype, relu))
    dims = (((1,), (1,)), ((), ()))

    def product(a, ww, *res):
        y = prims.dot_general(a, ww, dims, "float32", out_dtype) if a.dtype != "float32" else prims.dot_general(a, ww, dims, "float32")
        if relu:
            y = F.relu(y)
        return res[0] + y if res else y

    extra = [residual] if residual is not None else []
    if relu or extra:
        y = fused(product, x, w, *extra, name="dot_general", label="linear_relu" if relu else "linear_add")
    else:
        y = product(x, w)
    y.relu_output = relu and not extra  # python-side note for the consumer's backward

    def vjp(dy):
        if relu and not getattr(dy, "relu_masked", False):
            dy = fused(lambda g, out: F.where(F.gt(out, 0), g, 0), dy, y, label="relu_backward")
        if dy.dtype != x.dtype:  # the cotangent is narrowed to the operands' dtype (lumen/autograd/rules.py:431-439)
            dy = fused(lambda g: g.to(x.dtype), dy, label="narrow_cotangent")
        acc = "float32"
        dx_dims = (((1,), (0,)), ((), ()))
        if getattr(x, "relu_output", False) and x.dtype != "float32":
            # x = relu(..): its cotangent passes where x > 0. Fused into this product's epilogue.
            dx = fused(lambda g, ww, out: F.where(F.gt(out, 0), prims.dot_general(g, ww, dx_dims, acc, x.dtype), 0), dy, w, x,
                       name="dot_general", label="linear_backward_relu")
            dx.relu_masked = True
        else:
            dx = prims.dot_general(dy, w, dx_dims, acc, x.dtype)
        dw = prims.dot_general(dy, x, (((0,), (0,)), ((), ())), acc, w.dtype)
        return (dx, dw, dy) if extra else (dx, dw)

    tape.record([y], [x, w, *extra], vjp)
    return y


def add(tape: Tape, x: TracedTensor, y: TracedTensor) -> TracedTensor:
    out = fused(lambda a, b: a + b, x, y, label="residual_add")
    tape.record([out], [x, y], lambda g: (g, g))
    return out


def attention(tape: Tape, qkv: TracedTensor, batch: int, heads: int) -> TracedTensor:
    """Causal multi-head self-attention over a packed projection `[batch * seq, 3 * dim]`: q, k, v are strided
    views of it read in place by the kernels (the merged q/k/v GEMM of the reference's merge_dots pass), the
    forward is one `flash_attention` fusion (lumen/functional/attention/flash.py:30-49) and the backward one
    `flash_attention_backward` fusion (flash.py:51-85) whose three gradients are concatenated back into the packed
    layout."""
    tokens, width = qkv.shape
    dim = width // 3
    seq, hd = tokens // batch, dim // heads
    scale = 1.0 / math.sqrt(hd)
    q, k, v = (prims.slice(qkv, (0, i * dim), (tokens, (i + 1) * dim)).reshape(batch, seq, heads, hd) for i in range(3))
    o, lse = fused(lambda a, b, c: F.attention_forward_prims(a, b, c, scale, True), q, k, v, name="flash_attention")
    out = o.reshape(tokens, dim)

    def vjp(dout):
        do = dout.reshape(batch, seq, heads, hd)
        dq, dk, dv = fused(lambda a, b, c, oo, ll, g: F.attention_backward_prims(a, b, c, oo, ll, g, scale, True),
                           q, k, v, o, lse, do, name="flash_attention_backward")
        return (prims.concatenate([t.reshape(tokens, dim) for t in (dq, dk, dv)], 1),)

    tape.record([out], [qkv], vjp)
    return out


def cross_entropy_mean(tape: Tape, logits: TracedTensor, targets: TracedTensor, grad_dtype: str) -> TracedTensor:
    """Mean next-token cross entropy of `logits` `[rows, classes]`, computed in float32 (a `row` fusion saving each row's
    log-sum-exp, then a `reduction` for the mean); its gradient `(softmax - one_hot) / rows` is written directly in
    `grad_dtype`, the narrowing the following dot transposes need."""
    rows = logits.shape[0]
    wide = (lambda x: x) if logits.dtype == "float32" else (lambda x: x.float())  # 16-bit logits are widened in registers
    losses, lse = fused(lambda x, t: F.cross_entropy_forward_prims(wide(x), t), logits, targets, name="row", label="cross_entropy")
    loss = fused(lambda l: F.mean(l), losses, name="reduction", label="mean_loss")

    def vjp(dloss):
        def body(x, t, ll):
            prims.push_graph(x.graph)
            try:
                g = prims.full((rows,), 1.0 / rows, "float32")
            finally:
                prims.pop_graph()
            return F.cross_entropy_backward_prims(wide(x), t, ll, g).to(grad_dtype)

        return fused(body, logits, targets, lse, name="row", label="cross_entropy_backward"), None

    tape.record([loss], [logits, targets], vjp)
    return loss


def sgd_update(param: TracedTensor, grad: TracedTensor, lr, grad_scale: float = 1.0) -> TracedTensor:
    """`p - lr * g` (examples/optim.py:18-24), with the gradient first scaled by `grad_scale` (1 / world size after
    a summing all-reduce). The result is donated into the parameter's buffer. `lr` is a Python number (a constant of
    the generated kernel) or a traced 0-d float32 tensor: a run-time scalar the kernel reads from device memory, as the
    reference passes an optimizer's float fields on CUDA (lumen/codegen/devices/cuda/mod.rs:197-200), so that a
    schedule changes it without a new plan. Either way it is rounded to the parameter's dtype before the product."""
    if isinstance(lr, TracedTensor):
        def body_rt(p, g, rate):
            if grad_scale != 1.0:
                g = g * grad_scale
            return p - g * rate.to(p.dtype)

        return fused(body_rt, param, grad, lr, label="sgd_update")

    def body(p, g):
        if grad_scale != 1.0:
            g = g * grad_scale
        return p - g * lr

    return fused(body, param, grad, label="sgd_update")


def adamw_update(param: TracedTensor, m: TracedTensor, v: TracedTensor, grad: TracedTensor, step, lr: float = 1e-3,
                 betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 grad_scale: float = 1.0):
    """One AdamW step with decoupled weight decay as examples/optim.py:63-80 spells it: float32 moments,
    `m = b1 m + (1 - b1) g`, `v = b2 v + (1 - b2) g g`, bias corrections `1 / (1 - exp(step * log(b)))` (`step` counts
    from 1), `w (1 - lr wd) - lr (m c1) / (sqrt(v c2) + eps)` rounded once to the parameter's dtype. One generated
    kernel with three outputs `(param, m, v)`, each donated into its operand's buffer by the caller. `step` is a
    Python number (the corrections become constants) or a traced 0-d float32 tensor (one traced program serves every
    step, as the reference's spelling with exp / log intends)."""
    import numpy as np

    b1, b2 = betas
    log_b1, log_b2 = float(np.log(np.float32(b1))), float(np.log(np.float32(b2)))
    traced_step = isinstance(step, TracedTensor)

    def body(p, mm, vv, g, *t):
        if traced_step:
            c1 = 1.0 / (1.0 - F.exp(t[0] * log_b1))
            c2 = 1.0 / (1.0 - F.exp(t[0] * log_b2))
        else:
            one = np.float32(1.0)
            c1 = float(one / (one - np.exp(np.float32(step) * np.float32(log_b1))))
            c2 = float(one / (one - np.exp(np.float32(step) * np.float32(log_b2))))
        g, w = g.float(), p.float()
        if grad_scale != 1.0:
            g = g * grad_scale
        m_new = mm * b1 + g * (1.0 - b1)
        v_new = vv * b2 + g * g * (1.0 - b2)
        new = w * (1.0 - lr * weight_decay) - (m_new * c1) * lr / (F.sqrt(v_new * c2) + eps)
        return new.to(p.dtype), m_new, v_new

    extra = [step] if traced_step else []
    return fused(body, param, m, v, grad, *extra, label="adamw_update")
