"""Graph IR with lumen's strict primitives and their type rules.

A `Graph` is a list of typed values: inputs, then one value per node. `Graph.apply` adds a node after checking
the primitive's operand types, as the reference's `Graph.apply -> Primitive::infer` does
(lumen/graph/primitive.rs:535-1075): operands of one elementwise op share a dtype (no promotion),
`reduce_sum`/`dot_general` carry an explicit `accum_dtype` (lumen/graph/primitive.rs:1163-1176), and
`dot_general` outputs `output_dtype`, the accumulator's as traced.

`Graph.to_text` writes the line format both the CUDA backend (lumen_b200/csrc/graph_text.cpp) and the CPU oracle
(oracle/oracle.cpp) parse:

    graph <index>
    in <id> <dtype> <d0,d1,...|->
    node <id> <op> <dtype> <shape|-> <operand ids|-> [key=value ...]
    out <ids>
    end

Fusion bodies are graphs of their own, written before the graph that uses them and named by `body=<index>`.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

FLOATS = ("float16", "bfloat16", "float32", "float64")
SIGNED = ("int8", "int16", "int32", "int64")
UNSIGNED = ("uint8", "uint16", "uint32", "uint64")
DTYPES = ("bool",) + SIGNED + UNSIGNED + FLOATS

SIZE_OF = {
    "bool": 1, "int8": 1, "uint8": 1, "int16": 2, "uint16": 2, "float16": 2, "bfloat16": 2,
    "int32": 4, "uint32": 4, "float32": 4, "int64": 8, "uint64": 8, "float64": 8,
}  # fmt: skip

ELEMENTWISE_BINARY = ("add", "sub", "mul", "div", "max", "eq", "lt", "min", "pow", "rem", "and", "or", "xor")
FLOAT_UNARY = ("exp", "log", "sqrt", "tanh", "logistic", "rsqrt", "floor", "ceil", "exp2", "log2", "sin", "cos")
ANY_UNARY = ("neg", "abs", "sign", "not")
COLLECTIVES = ("all_reduce",)


def is_float(dtype: str) -> bool:
    return dtype in FLOATS


def is_int(dtype: str) -> bool:
    return dtype in SIGNED or dtype in UNSIGNED


@dataclass(frozen=True)
class TensorType:
    dtype: str
    shape: tuple[int, ...]

    def __post_init__(self):
        if self.dtype not in DTYPES:
            raise TypeError(f"unknown dtype {self.dtype!r}")
        object.__setattr__(self, "shape", tuple(int(n) for n in self.shape))

    @property
    def numel(self) -> int:
        return math.prod(self.shape)

    @property
    def nbytes(self) -> int:
        return self.numel * SIZE_OF[self.dtype]

    def __str__(self) -> str:
        return f"{self.dtype}[{','.join(map(str, self.shape))}]"


@dataclass
class Node:
    op: str
    inputs: tuple[int, ...]
    output: int
    params: dict = field(default_factory=dict)


def check_accum(x: TensorType, accum: str, op: str) -> None:
    """The operand's dtype, or float32 (int32) for floats (integers) narrower than 4 bytes
    (lumen/graph/primitive.rs:1163-1176)."""
    narrower = SIZE_OF[x.dtype] < 4
    widened = narrower and ((is_float(x.dtype) and accum == "float32") or (is_int(x.dtype) and accum == "int32"))
    if accum != x.dtype and not widened:
        raise TypeError(
            f"{op}: accumulates in the operand's dtype, or float32 (int32) for narrower floats (integers): "
            f"got accum_dtype {accum} for {x}"
        )


def _check_dims(dims, rank, what, op):
    if len(set(dims)) != len(dims) or any(not 0 <= d < rank for d in dims):
        raise TypeError(f"{op}: {what} {list(dims)} must be distinct dimensions of a rank-{rank} tensor")


def free_dims(rank, taken):
    return [d for d in range(rank) if d not in taken]


class Graph:
    """Typed values and the nodes computing them, in program order."""

    def __init__(self):
        self.types: list[TensorType] = []
        self.inputs: list[int] = []
        self.nodes: list[Node] = []
        self.outputs: list[int] = []

    # ---- construction -------------------------------------------------------------------------------------
    def add_input(self, dtype: str, shape) -> int:
        self.types.append(TensorType(dtype, tuple(shape)))
        self.inputs.append(len(self.types) - 1)
        return self.inputs[-1]

    def set_outputs(self, outputs) -> None:
        self.outputs = [int(v) for v in outputs]

    def type_of(self, v: int) -> TensorType:
        return self.types[v]

    def apply(self, prim: str, operands=(), /, **params) -> int:
        op = prim
        operands = tuple(int(v) for v in operands)
        out = infer(op, [self.types[v] for v in operands], params)
        self.types.append(out)
        v = len(self.types) - 1
        self.nodes.append(Node(op, operands, v, params))
        return v

    def producer(self, v: int) -> Node | None:
        for n in self.nodes:
            if n.output == v:
                return n
        return None

    # ---- text ---------------------------------------------------------------------------------------------
    def to_text(self) -> str:
        graphs: list[str] = []
        _write(self, graphs)
        return "".join(graphs)

    def __str__(self) -> str:
        return self.to_text()


def _fmt_shape(shape) -> str:
    return ",".join(map(str, shape)) if len(shape) else "-"


def _fmt_value(v) -> str:
    if isinstance(v, bool):
        return f"b:{int(v)}"
    if isinstance(v, int):
        return f"i:{v}"
    return f"f:{float(v).hex()}"


def _fmt_param(key, value, graphs) -> str:
    if isinstance(value, Graph):
        return f"{key}={_write(value, graphs)}"
    if key == "fill_value":
        return f"{key}={_fmt_value(value)}"
    if isinstance(value, dict):  # e.g. what the attention pass found: scale=..;causal=..;q=BSNH
        inner = ";".join(f"{k}:{float(v).hex() if isinstance(v, float) else (int(v) if isinstance(v, bool) else v)}" for k, v in value.items())
        return f"{key}={inner}"
    if isinstance(value, (list, tuple)):
        return f"{key}={','.join(map(str, value))}"
    if isinstance(value, bool):
        return f"{key}={int(value)}"
    text = str(value)
    if any(c.isspace() for c in text):
        raise ValueError(f"parameter {key}={value!r} has whitespace")
    return f"{key}={text}"


def _write(g: Graph, graphs: list[str]) -> int:
    """Appends `g` (after its fusion bodies) to `graphs` and returns its index."""
    lines = []
    for v in g.inputs:
        t = g.types[v]
        lines.append(f"in {v} {t.dtype} {_fmt_shape(t.shape)}\n")
    for n in g.nodes:
        t = g.types[n.output]
        ops = ",".join(map(str, n.inputs)) if n.inputs else "-"
        attrs = "".join(" " + _fmt_param(k, v, graphs) for k, v in n.params.items())
        lines.append(f"node {n.output} {n.op} {t.dtype} {_fmt_shape(t.shape)} {ops}{attrs}\n")
    lines.append(f"out {','.join(map(str, g.outputs)) if g.outputs else '-'}\nend\n")
    index = len(graphs)
    graphs.append(f"graph {index}\n" + "".join(lines))
    return index


# ---- type rules -------------------------------------------------------------------------------------------
def _same(op, args):
    first = args[0]
    for a in args[1:]:
        if a.dtype != first.dtype or a.shape != first.shape:
            raise TypeError(f"{op}: operands must share a type, got {', '.join(map(str, args))}")
    return first


def _arity(op, args, n):
    if len(args) != n:
        raise TypeError(f"{op} takes {n} operands, got {len(args)}")


def infer(op: str, args: list[TensorType], params: dict) -> TensorType:
    """The result type of `op` on `args`, or a TypeError naming the rule broken."""
    if op in ELEMENTWISE_BINARY:
        _arity(op, args, 2)
        x = _same(op, args)
        if op in ("eq", "lt"):
            return TensorType("bool", x.shape)
        if op in ("and", "or", "xor") and is_float(x.dtype):
            raise TypeError(f"{op}: takes integer or bool operands, got {x}")
        if op == "pow" and not is_float(x.dtype):
            raise TypeError(f"{op}: takes float operands, got {x}")
        if op in ("add", "sub", "mul", "div", "max", "min", "rem") and x.dtype == "bool":
            raise TypeError(f"{op}: does not take bool operands")
        return x
    if op in FLOAT_UNARY:
        _arity(op, args, 1)
        if not is_float(args[0].dtype):
            raise TypeError(f"{op}: takes a float operand, got {args[0]}")
        return args[0]
    if op in ANY_UNARY:
        _arity(op, args, 1)
        x = args[0]
        if op == "not" and is_float(x.dtype):
            raise TypeError(f"not: takes an integer or bool operand, got {x}")
        if op in ("neg", "abs", "sign") and x.dtype == "bool":
            raise TypeError(f"{op}: does not take bool operands")
        return x
    if op == "is_finite":
        _arity(op, args, 1)
        return TensorType("bool", args[0].shape)
    if op == "cast":
        _arity(op, args, 1)
        x, new = args[0], params["new_dtype"]
        # A wide integer to a float narrower than float32 would round twice: rejected as ambiguous.
        if is_int(x.dtype) and SIZE_OF[x.dtype] > 2 and new in ("float16", "bfloat16"):
            raise TypeError(f"cast: {x.dtype} to {new} is ambiguous, cast to float32 first")
        return TensorType(new, x.shape)
    if op == "select":
        _arity(op, args, 3)
        pred, x, y = args
        if pred.dtype != "bool" or pred.shape != x.shape:
            raise TypeError(f"select: the predicate must be bool{list(x.shape)}, got {pred}")
        return _same(op, [x, y])
    if op in ("reduce_sum", "reduce_max"):
        _arity(op, args, 1)
        x, axes = args[0], list(params["axes"])
        _check_dims(axes, len(x.shape), "axes", op)
        dtype = x.dtype
        if op == "reduce_sum":
            if x.dtype == "bool":
                raise TypeError("reduce_sum: does not take bool operands")
            check_accum(x, params["accum_dtype"], op)
            dtype = params["accum_dtype"]
        return TensorType(dtype, tuple(n for d, n in enumerate(x.shape) if d not in axes))
    if op == "dot_general":
        _arity(op, args, 2)
        lhs, rhs = args
        lc, rc = list(params["lhs_contracting"]), list(params["rhs_contracting"])
        lb, rb = list(params["lhs_batch"]), list(params["rhs_batch"])
        accum, output = params["accum_dtype"], params["output_dtype"]
        floats = is_float(lhs.dtype) and is_float(rhs.dtype)
        if (lhs.dtype != rhs.dtype and not floats) or lhs.dtype == "bool":
            raise TypeError(f"dot_general: operands must share a non-bool dtype (or be floats), got {lhs} and {rhs}")
        check_accum(lhs, accum, op)
        check_accum(rhs, accum, op)
        if output not in (lhs.dtype, rhs.dtype, accum):
            raise TypeError(
                f"dot_general: outputs the operands' dtype or accum_dtype ({accum}): got output_dtype {output} for {lhs}"
            )
        _check_dims(lb + lc, len(lhs.shape), "lhs dimensions", op)
        _check_dims(rb + rc, len(rhs.shape), "rhs dimensions", op)
        if (
            len(lb) != len(rb)
            or len(lc) != len(rc)
            or any(lhs.shape[l] != rhs.shape[r] for l, r in zip(lb + lc, rb + rc))
        ):
            raise TypeError(f"dot_general: batch and contracting dimensions of {lhs} and {rhs} do not match")
        shape = (
            [lhs.shape[d] for d in lb]
            + [lhs.shape[d] for d in free_dims(len(lhs.shape), lb + lc)]
            + [rhs.shape[d] for d in free_dims(len(rhs.shape), rb + rc)]
        )
        return TensorType(output, tuple(shape))
    if op == "reshape":
        _arity(op, args, 1)
        new = tuple(params["new_sizes"])
        if math.prod(new) != args[0].numel:
            raise TypeError(f"reshape: cannot reshape {args[0]} to {list(new)}")
        return TensorType(args[0].dtype, new)
    if op == "broadcast_in_dim":
        _arity(op, args, 1)
        x, shape, dims = args[0], tuple(params["shape"]), list(params["broadcast_dimensions"])
        if len(dims) != len(x.shape) or any(not 0 <= d < len(shape) for d in dims) or sorted(set(dims)) != dims:
            raise TypeError(f"broadcast_in_dim: dimensions {dims} must map {x} into {list(shape)} in order")
        for d, n in zip(dims, x.shape):
            if n != 1 and n != shape[d]:
                raise TypeError(f"broadcast_in_dim: cannot broadcast {x} to {list(shape)} along {dims}")
        return TensorType(x.dtype, shape)
    if op == "transpose":
        _arity(op, args, 1)
        x, perm = args[0], list(params["permutation"])
        if sorted(perm) != list(range(len(x.shape))):
            raise TypeError(f"transpose: {perm} is not a permutation of {x}'s dimensions")
        return TensorType(x.dtype, tuple(x.shape[d] for d in perm))
    if op == "slice":
        _arity(op, args, 1)
        x, lo, hi = args[0], list(params["start_indices"]), list(params["limit_indices"])
        if len(lo) != len(x.shape) or len(hi) != len(x.shape) or any(
            not 0 <= a <= b <= n for a, b, n in zip(lo, hi, x.shape)
        ):
            raise TypeError(f"slice: [{lo}, {hi}) is not a box inside {x}")
        return TensorType(x.dtype, tuple(b - a for a, b in zip(lo, hi)))
    if op == "concatenate":
        if not args:
            raise TypeError("concatenate takes at least 1 operand")
        d = params["dimension"]
        first = args[0]
        for a in args[1:]:
            if a.dtype != first.dtype or len(a.shape) != len(first.shape) or any(
                i != d and m != n for i, (m, n) in enumerate(zip(a.shape, first.shape))
            ):
                raise TypeError(f"concatenate: operands must agree outside dimension {d}")
        shape = list(first.shape)
        shape[d] = sum(a.shape[d] for a in args)
        return TensorType(first.dtype, tuple(shape))
    if op == "full":
        _arity(op, args, 0)
        return TensorType(params["dtype"], tuple(params["shape"]))
    if op == "iota":
        _arity(op, args, 0)
        shape = tuple(params["shape"])
        if not 0 <= params["dimension"] < len(shape) or params["dtype"] == "bool":
            raise TypeError(f"iota: dimension {params['dimension']} of {list(shape)}")
        return TensorType(params["dtype"], shape)
    if op == "gather":
        _arity(op, args, 2)
        x, idx, axis = args[0], args[1], params["axis"]
        if idx.dtype not in ("int32", "int64") or not 0 <= axis < len(x.shape):
            raise TypeError(f"gather: int32 or int64 indices into an axis of {x}, got {idx} and axis {axis}")
        return TensorType(x.dtype, x.shape[:axis] + idx.shape + x.shape[axis + 1 :])
    if op == "scatter_add":
        _arity(op, args, 3)
        x, idx, u, axis = args[0], args[1], args[2], params["axis"]
        want = x.shape[:axis] + idx.shape + x.shape[axis + 1 :]
        if idx.dtype not in ("int32", "int64") or u.dtype != x.dtype or u.shape != want or x.dtype == "bool":
            raise TypeError(f"scatter_add: updates must be {x.dtype}{list(want)}, got {u}")
        return x
    if op in ("device_wait", "host_wait"):
        _arity(op, args, 1)
        return args[0]
    if op == "all_reduce":
        _arity(op, args, 1)
        if params["op"] not in ("sum", "max", "min"):
            raise TypeError(f"all_reduce: op must be sum, max or min, got {params['op']}")
        return args[0]
    if op == "fusion":
        body: Graph = params["body"]
        _arity(op, args, len(body.inputs))
        for a, v in zip(args, body.inputs):
            if a != body.types[v]:
                raise TypeError(f"fusion: operand {a} for body input {body.types[v]}")
        return body.types[body.outputs[0]]
    if op == "fusion_output":
        raise TypeError("fusion_output is added with Graph.fusion_output")
    raise TypeError(f"unknown primitive {op!r}")


def fusion_output(g: Graph, fusion: int, index: int) -> int:
    """The `index`-th (≥1) output of the multi-output fusion producing `fusion`
    (lumen/reference/mod.rs:71-79)."""
    node = g.producer(fusion)
    if node is None or node.op != "fusion":
        raise TypeError("fusion_output: the operand must be a fusion")
    body: Graph = node.params["body"]
    if not 1 <= index < len(body.outputs):
        raise TypeError(f"fusion_output: index {index} of a fusion with {len(body.outputs)} outputs")
    g.types.append(body.types[body.outputs[index]])
    v = len(g.types) - 1
    g.nodes.append(Node("fusion_output", (fusion,), v, {"index": index}))
    return v
