"""The strict primitives as functions of traced tensors, mirroring `lumen.graph.prims`
(lumen/graph/prims.py:103-648): each call type-checks its operands and appends one node to the traced graph.
Nothing here promotes, broadcasts or casts: that is `lumen_b200.functional`'s job, done with explicit prims."""

from __future__ import annotations

from lumen_b200 import graph as G


class TracedTensor:
    """A value of the graph being traced. Operators are attached by `lumen_b200.tracer`."""

    # relu_output / relu_masked: trace-time notes of lumen_b200.nn (this value is a relu's output / a cotangent that
    # already went through a relu's backward mask); they do not exist in the graph
    __slots__ = ("graph", "var", "weak", "relu_output", "relu_masked")

    def __init__(self, graph: G.Graph, var: int, weak: bool = False):
        self.graph, self.var, self.weak = graph, var, weak
        self.relu_output = self.relu_masked = False

    @property
    def type(self) -> G.TensorType:
        return self.graph.types[self.var]

    @property
    def dtype(self) -> str:
        return self.type.dtype

    @property
    def shape(self) -> tuple[int, ...]:
        return self.type.shape

    @property
    def ndim(self) -> int:
        return len(self.type.shape)

    @property
    def numel(self) -> int:
        return self.type.numel

    def __repr__(self) -> str:
        return f"%{self.var}: {self.type}"


_GRAPHS: list[G.Graph] = []


def current_graph() -> G.Graph:
    if not _GRAPHS:
        raise RuntimeError("no graph is being traced")
    return _GRAPHS[-1]


def push_graph(g: G.Graph) -> None:
    _GRAPHS.append(g)


def pop_graph() -> G.Graph:
    return _GRAPHS.pop()


def bind(prim, /, *operands, **params) -> TracedTensor:
    """Appends primitive `prim` on `operands` to their graph (lumen/graph/prims.py:103)."""
    name = prim
    g = operands[0].graph if operands else current_graph()
    for x in operands:
        if not isinstance(x, TracedTensor):
            raise TypeError(f"{name}: operands are traced tensors, got {type(x).__name__}")
        if x.graph is not g:
            raise RuntimeError(f"{name}: operands of different graphs")
    return TracedTensor(g, g.apply(name, [x.var for x in operands], **params))


def _binary(name):
    def f(x, y):
        return bind(name, x, y)

    f.__name__ = name
    return f


def _unary(name):
    def f(x):
        return bind(name, x)

    f.__name__ = name
    return f


add, sub, mul, div = _binary("add"), _binary("sub"), _binary("mul"), _binary("div")
max, eq, lt = _binary("max"), _binary("eq"), _binary("lt")  # noqa: A001
min, pow, rem = _binary("min"), _binary("pow"), _binary("rem")  # noqa: A001
and_, or_, xor = _binary("and"), _binary("or"), _binary("xor")
neg, exp, log, sqrt, tanh, logistic = (_unary(n) for n in ("neg", "exp", "log", "sqrt", "tanh", "logistic"))
rsqrt, floor, ceil, exp2, log2, sin, cos = (_unary(n) for n in ("rsqrt", "floor", "ceil", "exp2", "log2", "sin", "cos"))
abs, sign, not_, is_finite = _unary("abs"), _unary("sign"), _unary("not"), _unary("is_finite")  # noqa: A001


def cast(x, new_dtype):
    return bind("cast", x, new_dtype=new_dtype)


def select(pred, on_true, on_false):
    return bind("select", pred, on_true, on_false)


def reduce_sum(x, axes, accum_dtype):
    return bind("reduce_sum", x, axes=tuple(axes), accum_dtype=accum_dtype)


def reduce_max(x, axes):
    return bind("reduce_max", x, axes=tuple(axes))


def dot_general(lhs, rhs, dimension_numbers, accum_dtype, output_dtype=None):
    """`dimension_numbers` = ((lhs_contracting, rhs_contracting), (lhs_batch, rhs_batch)); the result is
    `accum_dtype` as traced (lumen/graph/prims.py:233-250); `output_dtype` is what the late simplify pass folds a
    following narrowing cast into (lumen/graph/primitive.rs:248-250)."""
    (lc, rc), (lb, rb) = dimension_numbers
    return bind(
        "dot_general", lhs, rhs,
        lhs_contracting=tuple(lc), rhs_contracting=tuple(rc), lhs_batch=tuple(lb), rhs_batch=tuple(rb),
        accum_dtype=accum_dtype, output_dtype=output_dtype or accum_dtype,
    )  # fmt: skip


def reshape(x, new_sizes):
    return bind("reshape", x, new_sizes=tuple(new_sizes))


def broadcast_in_dim(x, shape, broadcast_dimensions):
    return bind("broadcast_in_dim", x, shape=tuple(shape), broadcast_dimensions=tuple(broadcast_dimensions))


def transpose(x, permutation):
    return bind("transpose", x, permutation=tuple(permutation))


def slice(x, start_indices, limit_indices):  # noqa: A001
    return bind("slice", x, start_indices=tuple(start_indices), limit_indices=tuple(limit_indices))


def concatenate(operands, dimension):
    return bind("concatenate", *operands, dimension=dimension)


def gather(x, indices, axis):
    return bind("gather", x, indices, axis=axis)


def scatter_add(x, indices, updates, axis):
    return bind("scatter_add", x, indices, updates, axis=axis)


def full(shape, fill_value, dtype):
    return bind("full", shape=tuple(shape), fill_value=fill_value, dtype=dtype)


def iota(dtype, shape, dimension):
    return bind("iota", dtype=dtype, shape=tuple(shape), dimension=dimension)


def device_wait(x):
    return bind("device_wait", x)


def all_reduce(x, op, ranks):
    return bind("all_reduce", x, op=op, ranks=tuple(ranks))


def fusion(operands, body: G.Graph, name: str, label: str = ""):
    """A fusion node over `operands` running `body`; returns one traced tensor per body output (the extra ones
    through `fusion_output` nodes, lumen/reference/mod.rs:71-79)."""
    first = bind("fusion", *operands, name=name, label=label or name, body=body)
    g = first.graph
    return [first] + [TracedTensor(g, G.fusion_output(g, first.var, k)) for k in range(1, len(body.outputs))]
