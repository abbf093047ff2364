"""torch-style functions that trace strict prims, mirroring `lumen.functional`
(lumen/functional/functions.py:137-470, lumen/functional/attention/flash.py:30-49,
lumen/functional/cross_entropy/logits.py:14-40). Every function spells its computation with explicit prims so
that the traced graph, evaluated primitive by primitive, defines the expected result."""

from __future__ import annotations

import builtins
import math

from lumen_b200 import prims
from lumen_b200.prims import TracedTensor
from lumen_b200.tracer import (
    _ge,
    _gt,
    _le,
    _min,
    _ne,
    accum_dtype,
    broadcast_shapes,
    broadcast_to,
    common_dtype,
    elementwise,
    is_float,
    norm_dim,
    norm_dims,
    operands,
)


def _require_float(x, op):
    if not is_float(x.dtype):
        raise TypeError(f"{op} needs a floating-point tensor, got {x.dtype}: convert it with .to(dtype)")
    return x


def add(a, b):
    return elementwise(prims.add, a, b)


def sub(a, b):
    return elementwise(prims.sub, a, b)


def mul(a, b):
    return elementwise(prims.mul, a, b)


def eq(a, b):
    return elementwise(prims.eq, a, b)


def ne(a, b):
    return elementwise(_ne, a, b)


def lt(a, b):
    return elementwise(prims.lt, a, b)


def le(a, b):
    return elementwise(_le, a, b)


def gt(a, b):
    return elementwise(_gt, a, b)


def ge(a, b):
    return elementwise(_ge, a, b)


def maximum(a, b):
    return elementwise(prims.max, a, b)


def minimum(a, b):
    return elementwise(_min, a, b)


def neg(x):
    return prims.neg(x)


def where(condition, input, other):  # noqa: A002
    if not isinstance(condition, TracedTensor) or condition.dtype != "bool":
        raise TypeError("where expected condition to be a bool tensor")
    g = condition.graph
    if not isinstance(input, TracedTensor) and not isinstance(other, TracedTensor):
        kind = "bool" if isinstance(input, bool) and isinstance(other, bool) else None
        ints = builtins.all(isinstance(v, int) for v in (input, other))
        prims.push_graph(g)
        try:
            input = prims.full(condition.shape, input, kind or ("int64" if ints else "float32"))
        finally:
            prims.pop_graph()
    x, y = operands("where", input, other)
    shape = broadcast_shapes(condition.shape, x.shape)
    return prims.select(broadcast_to(condition, shape), broadcast_to(x, shape), broadcast_to(y, shape))


def _float_fn(prim, name):
    def f(x):
        return prim(_require_float(x, name))

    f.__name__ = name
    return f


exp = _float_fn(prims.exp, "exp")
log = _float_fn(prims.log, "log")
sqrt = _float_fn(prims.sqrt, "sqrt")
rsqrt = _float_fn(prims.rsqrt, "rsqrt")
tanh = _float_fn(prims.tanh, "tanh")
sigmoid = _float_fn(prims.logistic, "sigmoid")


def relu(x):
    """`max(x, 0)` (lumen/functional/functions.py:224-226)."""
    return elementwise(prims.max, x, 0)


def _keep(x, out, dims, keepdim):
    if not keepdim:
        return out
    return out.reshape(tuple(1 if d in dims else n for d, n in enumerate(x.shape)))


def sum(x, dim=None, keepdim=False):  # noqa: A001
    """Sum over `dim`, accumulated in the tensor's own dtype (lumen/functional/functions.py:265-271)."""
    dims = norm_dims(dim, x.ndim)
    return _keep(x, prims.reduce_sum(x, dims, x.dtype), dims, keepdim)


def mean(x, dim=None, keepdim=False):
    """`sum * (1/count)` (lumen/functional/functions.py:274-281)."""
    _require_float(x, "mean")
    dims = norm_dims(dim, x.ndim)
    count = math.prod(x.shape[d] for d in dims)
    return sum(x, dims, keepdim) / count


def amax(x, dim=(), keepdim=False):
    dims = norm_dims(dim if dim != () else None, x.ndim)
    return _keep(x, prims.reduce_max(x, dims), dims, keepdim)


def softmax(x, dim):
    """`exp(x - max) / sum(exp(x - max))` as separate prims (lumen/functional/functions.py:315-323)."""
    _require_float(x, "softmax")
    e = exp(x - amax(x, dim, keepdim=True))
    return e / sum(e, dim, keepdim=True)


def log_softmax(x, dim):
    """`log(softmax(x))` from the max-shifted input (lumen/functional/functions.py:326-331)."""
    _require_float(x, "log_softmax")
    shifted = x - amax(x, dim, keepdim=True)
    return shifted - log(sum(exp(shifted), dim, keepdim=True))


def rms_norm(x, weight=None, eps=None):
    """`x * rsqrt(mean(x^2) + eps)` over the last dimension in `x`'s accumulation dtype, rounded to `x`'s, times
    `weight` if given; `eps` defaults to the dtype's machine epsilon (lumen/functional/functions.py:334-347,
    376-407)."""
    _require_float(x, "rms_norm")
    if weight is not None and (weight.dtype != x.dtype or tuple(weight.shape) != tuple(x.shape[-1:])):
        raise TypeError(f"rms_norm: weight must be {x.dtype}{list(x.shape[-1:])}, got {weight.dtype}{list(weight.shape)}")
    if eps is None:
        eps = {"float16": 2.0**-10, "bfloat16": 2.0**-7, "float64": 2.0**-52}.get(x.dtype, 2.0**-23)
    h = x.to(accum_dtype(x.dtype))
    inv = rsqrt(mean(h * h, -1, keepdim=True) + eps)
    y = (h * inv).to(x.dtype)
    return y if weight is None else y * weight


def div(a, b):
    """True division (lumen/functional/functions.py:131-134)."""
    return a / b


def square(x):
    """`x * x` (lumen/functional/functions.py:509-512)."""
    return x * x


def reciprocal(x):
    """`1 / x` as true division (lumen/functional/functions.py:515-517)."""
    return 1.0 / x


def abs(x):  # noqa: A001
    return prims.abs(x)


def sign(x):
    """-1, 0 or 1 by the sign; a float's zero and NaN stay as they are (lumen/functional/functions.py:504-506)."""
    return prims.sign(x)


def pow(x, exponent):  # noqa: A001
    """`x ** exponent`, elementwise (lumen/functional/functions.py:520-522)."""
    return elementwise(prims.pow, x, exponent)


def silu(x):
    """`x * sigmoid(x)`."""
    return _require_float(x, "silu") * sigmoid(x)


def swiglu(gate, up):
    """`silu(gate) * up`: the gated unit of a SwiGLU MLP, `gate` and `up` being the two projections of the input."""
    return silu(gate) * up


def gelu(x):
    """The tanh form of GELU: `0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3)))`."""
    _require_float(x, "gelu")
    inner = (x + (x * x * x) * 0.044715) * math.sqrt(2.0 / math.pi)
    return (x * 0.5) * (tanh(inner) + 1.0)


def _zeros_like(x, value=0, dtype=None):
    prims.push_graph(x.graph)
    try:
        return prims.full(x.shape, value, dtype or x.dtype)
    finally:
        prims.pop_graph()


def isfinite(x):
    """Neither infinite nor NaN; always true for a non-float tensor (lumen/functional/functions.py:530-535)."""
    return prims.is_finite(x) if is_float(x.dtype) else _zeros_like(x, True, "bool")


def isnan(x):
    """NaN is the one value not equal to itself; always false for a non-float tensor
    (lumen/functional/functions.py:538-544)."""
    return _ne(x, x) if is_float(x.dtype) else _zeros_like(x, False, "bool")


def _truth(x):
    """`x` as bools: its nonzero elements (lumen/functional/functions.py:547-552)."""
    if not isinstance(x, TracedTensor):
        return bool(x)
    return x if x.dtype == "bool" else _ne(x, _zeros_like(x))


def logical_and(a, b):
    return elementwise(prims.and_, _truth(a), _truth(b))


def logical_or(a, b):
    return elementwise(prims.or_, _truth(a), _truth(b))


def logical_not(x):
    return prims.not_(_truth(x))


def _flip(x):
    """An order-reversing bijection of the values: the negation, or the bitwise not of unsigned integers and bools
    (lumen/functional/functions.py:581-586)."""
    return prims.not_(x) if x.dtype == "bool" or x.dtype.startswith("uint") else prims.neg(x)


def amin(x, dim=(), keepdim=False):
    """Minimum over `dim` (every dimension when empty), as the flipped maximum of the flipped values
    (lumen/functional/functions.py:589-592)."""
    return _flip(amax(_flip(x), dim, keepdim))


def max(x, other=None):  # noqa: A001
    """`max(x)` over every element, or the elementwise `max(x, other)`."""
    return amax(x) if other is None else maximum(x, other)


def min(x, other=None):  # noqa: A001
    """`min(x)` over every element, or the elementwise `min(x, other)` (lumen/functional/functions.py:595-600)."""
    return amin(x) if other is None else minimum(x, other)


def any(x, dim=None, keepdim=False):  # noqa: A001
    """Whether any element over `dim` (all when None) is nonzero (lumen/functional/functions.py:603-605)."""
    return amax(_truth(x), () if dim is None else dim, keepdim)


def all(x, dim=None, keepdim=False):  # noqa: A001
    """Whether every element over `dim` is nonzero (lumen/functional/functions.py:608-610)."""
    return logical_not(any(logical_not(x), dim, keepdim))


def _arg(x, dim, keepdim, best):
    """The first index along `dim` at which `x` attains `best` (amax or amin), as int32; over the flattened tensor when
    `dim` is None: matching positions keep their index, the others get the dimension's size, and the smallest wins
    (lumen/functional/functions.py:613-627)."""
    if dim is None:
        return _arg(x.reshape(-1), 0, False, best)
    d = norm_dim(dim, x.ndim)
    target = best(x, d, True)
    prims.push_graph(x.graph)
    try:
        index = prims.iota("int32", x.shape, d)
        big = prims.full(x.shape, x.shape[d], "int32")
    finally:
        prims.pop_graph()
    hit = prims.eq(x, broadcast_to(target, x.shape))
    return amin(prims.select(hit, index, big), d, keepdim)


def argmax(x, dim=None, keepdim=False):
    return _arg(x, dim, keepdim, amax)


def argmin(x, dim=None, keepdim=False):
    return _arg(x, dim, keepdim, amin)


def cat(tensors, dim=0):
    """`tensors` one after another along `dim` (lumen/functional/functions.py:654-659)."""
    tensors = list(tensors)
    return prims.concatenate(tensors, norm_dim(dim, tensors[0].ndim))


def stack(tensors, dim=0):
    """`tensors` of one shape stacked along a new dimension `dim` (lumen/functional/functions.py:662-674)."""
    tensors = list(tensors)
    d = norm_dim(dim, tensors[0].ndim + 1)
    return cat([t.unsqueeze(d) for t in tensors], d)


def triu(x, diagonal=0):
    """The upper triangle of the last two dimensions: elements on and above diagonal `diagonal`, the others zero
    (lumen/functional/functions.py:677-685)."""
    prims.push_graph(x.graph)
    try:
        rows = prims.iota("int32", x.shape, x.ndim - 2)
        cols = prims.iota("int32", x.shape, x.ndim - 1)
        shift = prims.full(x.shape, diagonal, "int32")
        zero = prims.full(x.shape, 0, x.dtype)
    finally:
        prims.pop_graph()
    return prims.select(_le(prims.add(rows, shift), cols), x, zero)


def pad(x, pads, value=0):
    """`x` padded with `value`: `pads` lists (before, after) amounts from the LAST dimension backwards, like
    `torch.nn.functional.pad` (lumen/functional/functions.py: `pad`); written as concatenations with constant blocks."""
    pads = list(pads)
    if len(pads) % 2 or len(pads) // 2 > x.ndim or builtins.any(p < 0 for p in pads):
        raise ValueError(f"pad takes non-negative (before, after) pairs for at most {x.ndim} dimensions, got {pads}")
    out = x
    for k in range(len(pads) // 2):
        d = x.ndim - 1 - k
        before, after = pads[2 * k], pads[2 * k + 1]
        parts = []
        prims.push_graph(x.graph)
        try:
            if before:
                parts.append(prims.full(out.shape[:d] + (before,) + out.shape[d + 1 :], value, x.dtype))
            parts.append(out)
            if after:
                parts.append(prims.full(out.shape[:d] + (after,) + out.shape[d + 1 :], value, x.dtype))
        finally:
            prims.pop_graph()
        if len(parts) > 1:
            out = prims.concatenate(parts, d)
    return out


def clamp(x, min=None, max=None):  # noqa: A002
    """`x` clamped to `[min, max]`; either bound may be None, a scalar or a tensor
    (lumen/functional/functions.py:570-578)."""
    out = x
    if min is not None:
        out = maximum(out, min)
    if max is not None:
        out = minimum(out, max)
    return out


def layer_norm(a, w, b=None, eps=1e-5):
    """Layer norm over the last dimension, spelled as the reference's tests spell it
    (tests/graph_compiler/test_normalizations.py:103-106): `xc / sqrt(mean(xc*xc) + eps) * w (+ b)`."""
    xc = a - mean(a, -1, keepdim=True)
    y = xc / sqrt(mean(xc * xc, -1, keepdim=True) + eps) * w
    return y if b is None else y + b


def dot(x, y, dimension_numbers, accum, output):
    """`dot_general` accumulating in `accum`, cast to `output` when narrower (lumen/graph/tracer.py `_dot`)."""
    out = prims.dot_general(x, y, dimension_numbers, accum)
    return out if output == accum else prims.cast(out, output)


def matmul(input, other, accum_dtype, output_dtype):  # noqa: A002
    """`input @ other` with torch's shape rules and explicit accumulation/output dtypes
    (lumen/functional/functions.py:410-452)."""
    common_dtype("matmul", (input, other))
    if input.ndim == 0 or other.ndim == 0:
        raise RuntimeError("both arguments to matmul need to be at least 1D")
    if input.ndim > 2 and other.ndim == 2:
        k = input.shape[-1]
        rows = input.reshape(math.prod(input.shape[:-1]), k)
        out = dot(rows, other, (((1,), (0,)), ((), ())), accum_dtype, output_dtype)
        return out.reshape(*input.shape[:-1], other.shape[-1])
    x = input.unsqueeze(0) if input.ndim == 1 else input
    y = other.unsqueeze(-1) if other.ndim == 1 else other
    batch = broadcast_shapes(x.shape[:-2], y.shape[:-2])
    x, y = broadcast_to(x, batch + x.shape[-2:]), broadcast_to(y, batch + y.shape[-2:])
    b = tuple(range(len(batch)))
    out = dot(x, y, (((len(b) + 1,), (len(b),)), (b, b)), accum_dtype, output_dtype)
    if input.ndim == 1:
        out = out.squeeze(-2)
    if other.ndim == 1:
        out = out.squeeze(-1)
    return out


def one_hot(target, n, dtype):
    """`[..., n]` of `dtype`: 1 at each row's class (lumen/functional/cross_entropy/utils.py)."""
    shape = tuple(target.shape) + (n,)
    prims.push_graph(target.graph)
    try:
        classes = prims.iota(target.dtype, shape, len(shape) - 1)
    finally:
        prims.pop_graph()
    hit = prims.eq(classes, broadcast_to(target.reshape(*target.shape, 1), shape))
    return prims.cast(hit, dtype)


def scores(q, k, scale, causal):
    """`q k^T * scale` `[B, N, Sq, Sk]` in the accumulation dtype, masked keys -inf
    (lumen/functional/attention/utils.py:19-30)."""
    accum = accum_dtype(q.dtype)
    s = prims.dot_general(q, k, (((3,), (3,)), ((0, 2), (0, 2))), accum) * scale
    if causal:
        sq, sk = s.shape[2], s.shape[3]
        prims.push_graph(q.graph)
        try:
            rows = prims.iota("int64", s.shape, 2)
            cols = prims.iota("int64", s.shape, 3)
        finally:
            prims.pop_graph()
        s = where(le(cols, rows + (sk - sq)), s, float("-inf"))
    return s


def expand_heads(x, n):
    b, s, nkv, h = x.shape
    return x if nkv == n else x.unsqueeze(3).expand(b, s, nkv, n // nkv, h).reshape(b, s, n, h)


def attention_forward_prims(q, k, v, scale, causal):
    """The forward trace of flash attention (lumen/functional/attention/flash.py:30-49): returns `(o, lse)` with
    `o` `[B, Sq, N, Hv]` in the inputs' dtype and `lse` `[B, N, Sq, 1]` in the accumulation dtype."""
    n = q.shape[2]
    accum = accum_dtype(q.dtype)
    s = scores(q, expand_heads(k, n), scale, causal)
    m = amax(s, -1, keepdim=True)
    e = exp(s - m)
    total = sum(e, -1, keepdim=True)
    p = (e / total).to(q.dtype)
    o = dot(p, expand_heads(v, n), (((3,), (1,)), ((0, 1), (0, 2))), accum, q.dtype)
    return o.permute(0, 2, 1, 3), m + log(total)


def attention_backward_prims(q, k, v, o, lse, do, scale, causal):
    """FlashAttention-2's backward as traced by the reference (lumen/functional/attention/flash.py:51-85):
    transposed probabilities recomputed from the saved log-sum-exp; returns `(dq, dk, dv)` in the inputs' dtype."""
    b, sq, n, _ = q.shape
    sk, nkv = k.shape[1], k.shape[2]
    dtype, accum = q.dtype, accum_dtype(q.dtype)
    ke, ve = expand_heads(k, n), expand_heads(v, n)
    st = prims.dot_general(ke, q, (((3,), (3,)), ((0, 2), (0, 2))), accum) * scale
    if causal:
        prims.push_graph(q.graph)
        try:
            keys = prims.iota("int64", st.shape, 2)
            queries = prims.iota("int64", st.shape, 3)
        finally:
            prims.pop_graph()
        st = where(le(keys, queries + (sk - sq)), st, float("-inf"))
    pt = exp(st - lse.reshape(b, n, 1, sq))
    d = prims.dot_general(do, o, (((3,), (3,)), ((0, 1, 2), (0, 1, 2))), accum)
    d = d.permute(0, 2, 1).reshape(b, n, 1, sq)
    dpt = prims.dot_general(ve, do, (((3,), (3,)), ((0, 2), (0, 2))), accum)
    dst = (pt * (dpt - d) * scale).to(dtype)
    pt = pt.to(dtype)
    dv = prims.dot_general(pt, do, (((3,), (1,)), ((0, 1), (0, 2))), accum)
    dk = prims.dot_general(dst, q, (((3,), (1,)), ((0, 1), (0, 2))), accum)
    dq = prims.dot_general(dst, ke, (((2,), (1,)), ((0, 1), (0, 2))), accum)
    dq, dk, dv = (t.permute(0, 2, 1, 3) for t in (dq, dk, dv))
    if nkv != n:
        dk = sum(dk.reshape(b, sk, nkv, n // nkv, k.shape[3]), 3)
        dv = sum(dv.reshape(b, sk, nkv, n // nkv, v.shape[3]), 3)
    return dq.to(dtype), dk.to(dtype), dv.to(dtype)


def flash_attention(q, k, v, scale=None, causal=False):
    """Scaled dot-product attention of `[B, S, N, H]` operands as ONE `flash_attention` fusion: `(output, log-sum-exp)`
    with the output `[B, Sq, N, H]` and the float32 log-sum-exp `[B, N, Sq]` (lumen/functional/attention/flash.py:
    21-49, whose traced forward the reference's attention pass turns into the same fusion). The fusion's body is the
    spelled-out program (`attention_forward_prims`), which is what the oracle evaluates; the backend runs its
    tcgen05 kernel."""
    from lumen_b200.nn import fused

    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return fused(lambda a, b, c: attention_forward_prims(a, b, c, scale, bool(causal)), q, k, v, name="flash_attention")


def cross_entropy_forward_prims(x, target):
    """Per-row `logsumexp(x) - x[target]` and the saved logsumexp
    (lumen/functional/cross_entropy/logits.py:19-28)."""
    m = amax(x, -1, keepdim=True)
    lse = m.reshape(*target.shape) + log(sum(exp(x - m), -1))
    rows, n = math.prod(target.shape), x.shape[-1]
    prims.push_graph(x.graph)
    try:
        base = prims.iota(target.dtype, [rows], 0)
    finally:
        prims.pop_graph()
    at = base * n + target.reshape(rows)
    return lse - prims.gather(x.reshape(rows * n), at, 0).reshape(*target.shape), lse


def cross_entropy(x, target):
    """Per-row cross entropy `logsumexp(x) - x[target]` of `[rows, classes]` logits against integer class ids, spelled
    with a one-hot product instead of a gather (`sum(x * one_hot)` adds one value and zeros: the same number), so that
    autograd's elementwise and reduction rules differentiate it to `softmax(x) - one_hot` and the fusion pass keeps it
    in row kernels (lumen/functional/cross_entropy/logits.py:14-40 computes the same rows)."""
    _require_float(x, "cross_entropy")
    m = amax(x, -1, keepdim=True)
    lse = m.reshape(*target.shape) + log(sum(exp(x - m), -1))
    return lse - sum(x * one_hot(target, x.shape[-1], x.dtype), -1)


def cross_entropy_backward_prims(x, target, lse, g):
    """`(softmax(x) - one_hot(target)) * g` (lumen/functional/cross_entropy/logits.py:30-34)."""
    p = exp(x - lse.reshape(*target.shape, 1))
    return (p - one_hot(target, x.shape[-1], x.dtype)) * g.reshape(*target.shape, 1)


__all__ = [n for n in dir() if not n.startswith("_")]
_ = norm_dim
