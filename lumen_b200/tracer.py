"""Tracing: torch-style operators on traced tensors that record strict prims, with lumen's rules
(lumen/graph/tracer.py:1190-1328, 1352-1446): one dtype per op and no promotion, Python scalars lifted with
`full((), x, dtype)`, NumPy trailing-aligned broadcasting through `broadcast_in_dim`, and `x / c` for a static
`c` traced as `x * (1/c)`."""

from __future__ import annotations

import builtins
import math

from lumen_b200 import graph as G
from lumen_b200 import prims
from lumen_b200.prims import TracedTensor


def is_float(dtype):
    return G.is_float(dtype)


def accum_dtype(dtype):
    """float32 for floats narrower than 4 bytes, else the dtype itself (lumen/graph/tracer.py `_accum_dtype`)."""
    return "float32" if dtype in ("float16", "bfloat16") else dtype


def lift(x):
    return x


def common_dtype(op, operands):
    tensors = [x for x in operands if isinstance(x, TracedTensor)]
    if not tensors:
        raise TypeError(f"{op} needs a tensor operand")
    dtypes = sorted({x.dtype for x in tensors if not x.weak} or {x.dtype for x in tensors})
    if len(dtypes) > 1:
        raise TypeError(f"{op} got tensors of dtypes {' and '.join(dtypes)}: convert them to one with .to(dtype)")
    return dtypes[0]


def _scalar_fits(x, dtype):
    if isinstance(x, bool):
        return dtype == "bool"
    if isinstance(x, int):
        return dtype != "bool"
    return is_float(dtype)


def as_tensor(x, dtype, op, graph):
    if isinstance(x, TracedTensor):
        if x.weak and x.dtype != dtype:
            return x.to(dtype)
        return x
    if not isinstance(x, (bool, int, float)):
        raise TypeError(f"expected a tensor or a Python scalar, got {type(x).__name__}")
    if not _scalar_fits(x, dtype):
        raise TypeError(f"{op} of a {dtype} tensor and the {type(x).__name__} {x!r}: convert the tensor with .to(dtype)")
    prims.push_graph(graph)
    try:
        return prims.full((), x, dtype)
    finally:
        prims.pop_graph()


def broadcast_shapes(*shapes):
    ndim = builtins.max(len(s) for s in shapes)
    out = []
    for d in range(-ndim, 0):
        sizes = {s[d] for s in shapes if len(s) >= -d} - {1}
        if len(sizes) > 1:
            raise RuntimeError(f"shapes {', '.join(str(list(s)) for s in shapes)} are not broadcastable at dimension {d}")
        out.append(sizes.pop() if sizes else 1)
    return tuple(out)


def broadcast_to(x, shape):
    shape = tuple(shape)
    if x.shape == shape:
        return x
    lead = len(shape) - x.ndim
    return prims.broadcast_in_dim(x, shape, range(lead, len(shape)))


def operands(op, *xs):
    dtype = common_dtype(op, xs)
    graph = next(x.graph for x in xs if isinstance(x, TracedTensor))
    tensors = [as_tensor(x, dtype, op, graph) for x in xs]
    shape = broadcast_shapes(*(t.shape for t in tensors))
    return [broadcast_to(t, shape) for t in tensors]


def elementwise(prim, *xs):
    out = prim(*operands(getattr(prim, "__name__", "op").lstrip("_"), *xs))
    tensors = [x for x in xs if isinstance(x, TracedTensor)]
    out.weak = bool(tensors) and all(x.weak for x in tensors)
    return out


def _min(x, y):
    if is_float(x.dtype):
        return prims.neg(prims.max(prims.neg(x), prims.neg(y)))
    return prims.select(prims.lt(y, x), y, x)


def _le(x, y):
    less = prims.lt(x, y)
    return prims.select(less, less, prims.eq(x, y))


def _gt(x, y):
    return prims.lt(y, x)


def _ge(x, y):
    return _le(y, x)


def _ne(x, y):
    g = x.graph
    prims.push_graph(g)
    try:
        return prims.eq(prims.eq(x, y), prims.full(x.shape, False, "bool"))
    finally:
        prims.pop_graph()


def norm_dim(dim, ndim):
    if not -ndim <= dim < builtins.max(ndim, 1):
        raise IndexError(f"dimension {dim} out of range for a rank-{ndim} tensor")
    return dim % ndim if ndim else 0


def norm_dims(dim, ndim):
    if dim is None:
        return tuple(range(ndim))
    if isinstance(dim, int):
        dim = (dim,)
    return tuple(sorted(norm_dim(d, ndim) for d in dim))


# ---- TracedTensor methods -----------------------------------------------------------------------------------
def _binary_method(prim, reflected=False):
    def op(self, other):
        if not isinstance(other, (TracedTensor, bool, int, float)):
            return NotImplemented
        return elementwise(prim, other, self) if reflected else elementwise(prim, self, other)

    return op


def _truediv(self, other):
    # A static divisor is traced as a multiplication by its reciprocal (lumen/graph/tracer.py:1442-1446).
    if isinstance(other, (int, float)) and not isinstance(other, bool):
        return elementwise(prims.mul, self, 1.0 / other)
    return elementwise(prims.div, self, other)


def _rtruediv(self, other):
    return elementwise(prims.div, other, self)


def _to(self, dtype):
    return self if dtype == self.dtype else prims.cast(self, dtype)


def _reshape(self, *shape):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    if -1 in shape:
        known = -math.prod(shape)
        shape = tuple(self.numel // known if n == -1 else n for n in shape)
    return self if tuple(shape) == self.shape else prims.reshape(self, shape)


def _permute(self, *perm):
    if len(perm) == 1 and isinstance(perm[0], (tuple, list)):
        perm = tuple(perm[0])
    perm = tuple(norm_dim(d, self.ndim) for d in perm)
    return self if perm == tuple(range(self.ndim)) else prims.transpose(self, perm)


def _transpose(self, a, b):
    a, b = norm_dim(a, self.ndim), norm_dim(b, self.ndim)
    perm = list(range(self.ndim))
    perm[a], perm[b] = perm[b], perm[a]
    return _permute(self, perm)


def _t(self):
    if self.ndim != 2:
        raise RuntimeError(f"t() expects a 2-d tensor, got {self.ndim}-d")
    return _transpose(self, 0, 1)


def _unsqueeze(self, dim):
    dim = dim % (self.ndim + 1)
    return _reshape(self, self.shape[:dim] + (1,) + self.shape[dim:])


def _squeeze(self, dim):
    dim = norm_dim(dim, self.ndim)
    return _reshape(self, self.shape[:dim] + self.shape[dim + 1 :]) if self.shape[dim] == 1 else self


def _expand(self, *shape):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    shape = tuple(self.shape[d - (len(shape) - self.ndim)] if n == -1 else n for d, n in enumerate(shape))
    return broadcast_to(self, shape)


def _getitem(self, index):
    """`table[ids]` with an integer tensor: a gather of rows (lumen/reference/mod.rs:731-749)."""
    if isinstance(index, TracedTensor):
        return prims.gather(self, index, 0)
    raise NotImplementedError("only tensor[int_tensor] (a row gather) is traced")


TracedTensor.__add__ = _binary_method(prims.add)
TracedTensor.__radd__ = _binary_method(prims.add, True)
TracedTensor.__sub__ = _binary_method(prims.sub)
TracedTensor.__rsub__ = _binary_method(prims.sub, True)
TracedTensor.__mul__ = _binary_method(prims.mul)
TracedTensor.__rmul__ = _binary_method(prims.mul, True)
TracedTensor.__truediv__ = _truediv
TracedTensor.__rtruediv__ = _rtruediv
TracedTensor.__neg__ = lambda self: prims.neg(self)
TracedTensor.__lt__ = _binary_method(prims.lt)
TracedTensor.__le__ = _binary_method(_le)
TracedTensor.__gt__ = _binary_method(_gt)
TracedTensor.__ge__ = _binary_method(_ge)
TracedTensor.__getitem__ = _getitem
TracedTensor.to = _to
TracedTensor.float = lambda self: _to(self, "float32")
TracedTensor.bfloat16 = lambda self: _to(self, "bfloat16")
TracedTensor.reshape = _reshape
TracedTensor.permute = _permute
TracedTensor.transpose = _transpose
TracedTensor.t = _t
TracedTensor.unsqueeze = _unsqueeze
TracedTensor.squeeze = _squeeze
TracedTensor.expand = _expand
TracedTensor.__hash__ = lambda self: hash((id(self.graph), self.var))


def trace(fn, *types, names=None):
    """Runs `fn` on traced inputs of `types` ((dtype, shape) pairs) and returns the graph; `fn` returns a traced
    tensor or a tuple of them, the graph's outputs."""
    g = G.Graph()
    prims.push_graph(g)
    try:
        args = [TracedTensor(g, g.add_input(dtype, shape)) for dtype, shape in types]
        out = fn(*args)
    finally:
        prims.pop_graph()
    outs = out if isinstance(out, (tuple, list)) else (out,)
    g.set_outputs([o.var for o in outs])
    return g
