"""Seeded random programs over the element-wise, comparison, cast and reduction functions, for the tests that run the
same program through the oracle and through the backend. A program is a recipe (a list of steps over a pool of values)
drawn once per seed, so tracing it twice builds the same graph twice.

`exact` programs use only functions whose float32 / bfloat16 results are defined bit for bit (IEEE add, sub, mul, div,
sqrt, min / max, rounding to integers, comparisons, selects, casts): the backend must reproduce the oracle's bits.
Other programs end in transcendental functions, which the backend computes with CUDA's single-precision library
(1 - 2 ulp), and are compared within a tolerance."""

import numpy as np

from lumen_b200 import functional as F
from lumen_b200 import prims

SHAPES = [(37, 129), (64, 256), (5, 7, 64), (1000,), (3, 1), (130, 33), (16, 1024), (2, 3, 4, 8)]

FLOAT_BINARY = ["add", "sub", "mul", "div", "maximum", "minimum"]
FLOAT_UNARY = ["neg", "abs", "sign", "relu", "floor", "ceil", "sqrt_abs", "half", "recast"]
BOOL_MAKERS = ["lt", "le", "gt", "eq_floor", "isfinite"]
SMOOTH_UNARY = ["exp_capped", "tanh", "logistic", "log1p_abs", "sin", "cos", "rsqrt_shift", "silu", "gelu", "exp2_capped", "log2_shift"]


def draw_recipe(seed: int, exact: bool):
    """(shape, dtype, input kinds, steps, outputs). Input kinds: "full", "row" (the last axis only) or "col" (ones in the
    last axis). A step is (name, operand indices); value k of the pool is input k for k < len(inputs), else the result of
    step k - len(inputs). Outputs: (kind, value index) with kind "value", "sum_last", "max_last" or "sum_first"."""
    rng = np.random.default_rng(seed)
    shape = SHAPES[int(rng.integers(len(SHAPES)))]
    dtype = ["float32", "bfloat16"][int(rng.integers(2))]
    n_inputs = int(rng.integers(2, 5))
    kinds = ["full"] + [["full", "full", "row", "col"][int(rng.integers(4))] for _ in range(n_inputs - 1)]
    floats, bools, steps = list(range(n_inputs)), [], []
    for _ in range(int(rng.integers(5, 13))):
        k = n_inputs + len(steps)
        choice = rng.random()
        if choice < 0.45:
            steps.append((FLOAT_BINARY[int(rng.integers(len(FLOAT_BINARY)))], (int(rng.choice(floats)), int(rng.choice(floats)))))
            floats.append(k)
        elif choice < 0.7:
            steps.append((FLOAT_UNARY[int(rng.integers(len(FLOAT_UNARY)))], (int(rng.choice(floats)),)))
            floats.append(k)
        elif choice < 0.85 or not bools:
            name = BOOL_MAKERS[int(rng.integers(len(BOOL_MAKERS)))]
            steps.append((name, (int(rng.choice(floats)), int(rng.choice(floats)))))
            bools.append(k)
        elif choice < 0.93:
            steps.append(("where", (int(rng.choice(bools)), int(rng.choice(floats)), int(rng.choice(floats)))))
            floats.append(k)
        else:
            steps.append((["logical_and", "logical_or", "logical_not"][int(rng.integers(3))], (int(rng.choice(bools)), int(rng.choice(bools)))))
            bools.append(k)
    made = [v for v in floats if v >= n_inputs] or floats
    outputs = [("value", int(v)) for v in rng.choice(made, size=min(len(made), int(rng.integers(1, 4))), replace=False)]
    if not exact:
        # a smooth function of each result, then one more product or sum: nothing discontinuous reads an approximate value
        finished = []
        for _, v in outputs:
            k = n_inputs + len(steps)
            steps.append((SMOOTH_UNARY[int(rng.integers(len(SMOOTH_UNARY)))], (v,)))
            steps.append((["add", "mul"][int(rng.integers(2))], (k, int(rng.integers(n_inputs)))))
            finished.append(("value", k + 1))
        outputs = finished
    if len(shape) >= 2 and rng.random() < 0.6:
        outputs.append((["sum_last", "max_last", "sum_first"][int(rng.integers(3))], outputs[0][1]))
    if bools and rng.random() < 0.3:
        outputs.append(("value", int(rng.choice(bools))))
    return shape, dtype, kinds, steps, outputs


def input_types(recipe):
    shape, dtype, kinds, _, _ = recipe
    return [(dtype, {"full": shape, "row": shape[-1:], "col": shape[:-1] + (1,)}[kind]) for kind in kinds]


def draw_inputs(recipe, seed: int):
    """Standard-normal samples in the program's dtype, with a few exact integers, zeros of both signs and repeats among
    them, so that comparisons for equality, `sign` and the rounding functions see their special cases."""
    rng = np.random.default_rng(seed + 10_000)
    arrays = []
    for dtype, shape in input_types(recipe):
        a = rng.standard_normal(shape).astype(np.float32) * np.float32(2.0)
        flat = a.reshape(-1)
        picks = rng.integers(0, flat.size, size=max(flat.size // 16, 1))
        flat[picks] = rng.choice(np.array([0.0, -0.0, 1.0, -1.0, 2.0, 0.5, -3.0], np.float32), size=picks.size)
        if dtype == "bfloat16":
            from tests.helpers import bf16

            a = bf16(a)
        elif dtype in ("float16", "float64"):
            a = a.astype(dtype)
        arrays.append(a)
    return arrays


def in_dtype(recipe, dtype):
    """The same element-wise recipe with float16 or float64 values (the generated kernels' other float types)."""
    shape, _, kinds, steps, outputs = recipe
    return shape, dtype, kinds, steps, outputs


def build(recipe):
    """The program as a function of its inputs, for `tracer.trace` and `lumen_b200.compile`."""
    shape, dtype, kinds, steps, outputs = recipe
    other = "bfloat16" if dtype == "float32" else "float32"

    def program(*inputs):
        pool = list(inputs)
        for name, args in steps:
            x = [pool[a] for a in args]
            if name in ("add", "sub", "mul", "div", "maximum", "minimum", "lt", "le", "gt", "logical_and", "logical_or"):
                y = getattr(F, name)(x[0], x[1])
            elif name in ("neg", "abs", "sign", "relu", "silu", "gelu", "isfinite"):
                y = getattr(F, name)(x[0])
            elif name == "logical_not":
                y = F.logical_not(x[0])
            elif name in ("floor", "ceil", "tanh", "logistic", "sin", "cos"):
                y = getattr(prims, name)(x[0])
            elif name == "sqrt_abs":
                y = prims.sqrt(F.abs(x[0]))
            elif name == "half":
                y = F.mul(x[0], 0.5)
            elif name == "recast":  # through the other float type and back: a rounding to bfloat16 in a float32 program
                y = prims.cast(prims.cast(x[0], other), dtype)
            elif name == "eq_floor":
                y = F.eq(prims.floor(x[0]), prims.floor(x[1]))
            elif name == "where":
                y = F.where(x[0], x[1], x[2])
            elif name == "exp_capped":
                y = prims.exp(F.minimum(x[0], 4.0))
            elif name == "exp2_capped":
                y = prims.exp2(F.minimum(x[0], 6.0))
            elif name == "log1p_abs":
                y = prims.log(F.add(F.abs(x[0]), 1.0))
            elif name == "log2_shift":
                y = prims.log2(F.add(F.abs(x[0]), 0.5))
            elif name == "rsqrt_shift":
                y = prims.rsqrt(F.add(F.abs(x[0]), 0.5))
            else:
                raise AssertionError(name)
            pool.append(y)
        results = []
        for kind, v in outputs:
            value = pool[v]
            if kind == "value":
                results.append(value)
            else:
                wide = value if value.dtype in ("float32", "float64") else prims.cast(value, "float32")
                results.append({"sum_last": lambda t: F.sum(t, -1), "max_last": lambda t: F.amax(t, -1), "sum_first": lambda t: F.sum(t, 0)}[kind](wide))
        return tuple(results)

    return program


# ---- programs of views: reshapes, transposes, slices and concatenations between element-wise steps ----------------------

LAYOUT_SHAPES = [(8, 12), (16, 6, 4), (32, 64), (4, 8, 16), (64, 48), (2, 6, 8, 4)]


def draw_layout_recipe(seed: int):
    """(dtype, input shapes, steps, outputs). Steps are (name, operands, parameters) over a pool of values whose shapes
    are tracked here, so that every step is well formed: "unary" / "binary" (same-shaped operands), "transpose" (a
    permutation), "merge" (two neighbouring axes into one), "split" (an axis into two factors), "slice" (a range of one
    axis) and "concat" (two values along an axis)."""
    rng = np.random.default_rng(seed + 77_000)
    dtype = ["float32", "bfloat16"][int(rng.integers(2))]
    shape = LAYOUT_SHAPES[int(rng.integers(len(LAYOUT_SHAPES)))]
    shapes = [shape, shape]
    steps = []
    for _ in range(int(rng.integers(4, 10))):
        a = int(rng.integers(len(shapes)))
        s = shapes[a]
        choice = rng.random()
        if choice < 0.3:
            same = [k for k, t in enumerate(shapes) if t == s]
            b = int(rng.choice(same))
            steps.append(("binary", (a, b), ["add", "sub", "mul", "maximum"][int(rng.integers(4))]))
            shapes.append(s)
        elif choice < 0.4:
            steps.append(("unary", (a,), ["neg", "abs", "relu", "half"][int(rng.integers(4))]))
            shapes.append(s)
        elif choice < 0.6 and len(s) >= 2:
            perm = tuple(int(p) for p in rng.permutation(len(s)))
            steps.append(("transpose", (a,), perm))
            shapes.append(tuple(s[p] for p in perm))
        elif choice < 0.7 and len(s) >= 2:
            d = int(rng.integers(len(s) - 1))
            steps.append(("reshape", (a,), s[:d] + (s[d] * s[d + 1],) + s[d + 2 :]))
            shapes.append(steps[-1][2])
        elif choice < 0.8:
            d = int(rng.integers(len(s)))
            factors = [f for f in (2, 3, 4) if s[d] % f == 0 and s[d] > f]
            if not factors or len(s) >= 4:
                continue
            f = int(rng.choice(factors))
            steps.append(("reshape", (a,), s[:d] + (f, s[d] // f) + s[d + 1 :]))
            shapes.append(steps[-1][2])
        elif choice < 0.9:
            d = int(rng.integers(len(s)))
            if s[d] < 2:
                continue
            lo = int(rng.integers(0, s[d] // 2))
            hi = int(rng.integers(lo + 1, s[d] + 1))
            start = tuple(lo if k == d else 0 for k in range(len(s)))
            limit = tuple(hi if k == d else s[k] for k in range(len(s)))
            steps.append(("slice", (a,), (start, limit)))
            shapes.append(tuple(hi - lo if k == d else s[k] for k in range(len(s))))
        else:
            same = [k for k, t in enumerate(shapes) if t == s]
            b = int(rng.choice(same))
            d = int(rng.integers(len(s)))
            steps.append(("concat", (a, b), d))
            shapes.append(tuple(2 * s[k] if k == d else s[k] for k in range(len(s))))
    made = list(range(2, len(shapes))) or [0]
    picks = rng.choice(made, size=min(len(made), int(rng.integers(1, 3))), replace=False)
    # a result is returned as it is (a view is then copied out) or through one more element-wise step (the kernel reads the view)
    outputs = [(int(v), bool(rng.random() < 0.6)) for v in picks]
    return dtype, [shape, shape], steps, outputs


def build_layout(recipe):
    dtype, _, steps, outputs = recipe

    def program(x, y):
        pool = [x, y]
        for name, args, param in steps:
            v = [pool[a] for a in args]
            if name == "binary":
                out = getattr(F, param)(v[0], v[1])
            elif name == "unary":
                out = F.mul(v[0], 0.5) if param == "half" else getattr(F, param)(v[0])
            elif name == "transpose":
                out = prims.transpose(v[0], param)
            elif name == "reshape":
                out = prims.reshape(v[0], param)
            elif name == "slice":
                out = prims.slice(v[0], param[0], param[1])
            else:
                out = prims.concatenate([v[0], v[1]], param)
            pool.append(out)
        return tuple(F.mul(pool[v], 1.5) if finish else pool[v] for v, finish in outputs)

    return program


def draw_layout_inputs(recipe, seed: int):
    dtype, shapes, _, _ = recipe
    rng = np.random.default_rng(seed + 78_000)
    arrays = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    if dtype == "bfloat16":
        from tests.helpers import bf16

        arrays = [bf16(a) for a in arrays]
    return arrays


# ---- integer programs: wrapping arithmetic, division rules, bit operations, saturating casts, exact reductions ----------

INT_DTYPES = ["int32", "int64", "uint8", "int8", "int16", "uint32"]
INT_BINARY = ["add", "sub", "mul", "div", "rem", "max", "min", "and_", "or_", "xor"]
INT_UNARY = ["neg", "abs", "sign", "not_", "through_float", "through_other"]


def draw_integer_recipe(seed: int):
    """(shape, dtype, other dtype, steps, outputs): every value has the program's shape; integers of `dtype`, or truth
    values from comparisons. Outputs: (kind, value) with kind "value", "sum_last", "max_last", "min_last" or "sum_first"."""
    rng = np.random.default_rng(seed + 91_000)
    shape = [(33, 65), (128, 64), (7, 5, 32), (1000,), (40, 257)][int(rng.integers(5))]
    dtype = INT_DTYPES[int(rng.integers(len(INT_DTYPES)))]
    other = [d for d in INT_DTYPES if d != dtype][int(rng.integers(len(INT_DTYPES) - 1))]
    n_inputs = int(rng.integers(2, 4))
    ints, bools, steps = list(range(n_inputs)), [], []
    for _ in range(int(rng.integers(4, 11))):
        k = n_inputs + len(steps)
        choice = rng.random()
        if choice < 0.55:
            steps.append((INT_BINARY[int(rng.integers(len(INT_BINARY)))], (int(rng.choice(ints)), int(rng.choice(ints)))))
            ints.append(k)
        elif choice < 0.75:
            steps.append((INT_UNARY[int(rng.integers(len(INT_UNARY)))], (int(rng.choice(ints)),)))
            ints.append(k)
        elif choice < 0.9 or not bools:
            steps.append((["lt", "eq", "le", "gt"][int(rng.integers(4))], (int(rng.choice(ints)), int(rng.choice(ints)))))
            bools.append(k)
        else:
            steps.append(("where", (int(rng.choice(bools)), int(rng.choice(ints)), int(rng.choice(ints)))))
            ints.append(k)
    made = [v for v in ints if v >= n_inputs] or ints
    outputs = [("value", int(v)) for v in rng.choice(made, size=min(len(made), int(rng.integers(1, 3))), replace=False)]
    if len(shape) >= 2 and rng.random() < 0.7:
        outputs.append((["sum_last", "max_last", "min_last", "sum_first"][int(rng.integers(4))], outputs[0][1]))
    if bools and rng.random() < 0.3:
        outputs.append(("value", int(rng.choice(bools))))
    return shape, dtype, other, n_inputs, steps, outputs


def draw_integer_inputs(recipe, seed: int):
    """Full-range draws mixed with small values, zeros (divisors), the type's limits and minus one."""
    shape, dtype, _, n_inputs, _, _ = recipe
    rng = np.random.default_rng(seed + 92_000)
    info = np.iinfo(dtype)
    arrays = []
    for _ in range(n_inputs):
        a = rng.integers(info.min, info.max, size=shape, dtype=dtype, endpoint=True)
        flat = a.reshape(-1)
        small = rng.integers(0, flat.size, size=flat.size // 3)
        flat[small] = rng.integers(max(info.min, -6), 7, size=small.size).astype(dtype)
        edge = rng.integers(0, flat.size, size=max(flat.size // 20, 1))
        flat[edge] = rng.choice(np.array([info.min, info.max, 0, 1, info.max - 1], dtype=np.int64 if info.max < 2**63 - 1 else object), size=edge.size).astype(dtype)
        arrays.append(a)
    return arrays


def build_integer(recipe):
    shape, dtype, other, n_inputs, steps, outputs = recipe

    def program(*inputs):
        pool = list(inputs)
        for name, args in steps:
            x = [pool[a] for a in args]
            if name in INT_BINARY:
                y = getattr(prims, name)(x[0], x[1])
            elif name in ("neg", "abs", "sign", "not_"):
                y = getattr(prims, name)(x[0])
            elif name == "through_float":  # to float32 (round to nearest even) and back (saturating)
                y = prims.cast(prims.cast(x[0], "float32"), dtype)
            elif name == "through_other":
                y = prims.cast(prims.cast(x[0], other), dtype)
            elif name in ("lt", "eq", "le", "gt"):
                y = getattr(F, name)(x[0], x[1])
            else:
                y = F.where(x[0], x[1], x[2])
            pool.append(y)
        reduce = {"sum_last": lambda t: F.sum(t, -1), "max_last": lambda t: F.amax(t, -1), "min_last": lambda t: F.amin(t, -1), "sum_first": lambda t: F.sum(t, 0)}
        return tuple(pool[v] if kind == "value" else reduce[kind](pool[v]) for kind, v in outputs)

    return program


# ---- programs with reductions whose results are used again: normalisation-like rows, column and whole-tensor sums -------

REDUCING_SHAPES = [(37, 129), (64, 256), (5, 7, 64), (130, 33), (16, 1024), (9, 2048), (3, 5000), (2, 3, 4, 40), (257, 8),
                   (20000, 96), (4096, 1536), (70000, 8), (12, 300, 40)]  # the last four: column sums over many row slices


def draw_reducing_recipe(seed: int):
    """(shape, dtype, steps, outputs): float programs in which sums, means and maxima over the last axis (kept as a
    length-one axis) are combined again with the full tensor, once or twice in a row as a layer normalisation does; the
    outputs add reductions over the first axis, over all but the last axis and over everything. Only smooth functions
    follow a sum, so that results can be compared within a tolerance. With dtype "float64" in the recipe the same program
    is the ground truth the float32 / bfloat16 results are measured against."""
    rng = np.random.default_rng(seed + 55_000)
    shape = REDUCING_SHAPES[int(rng.integers(len(REDUCING_SHAPES)))]
    dtype = ["float32", "float32", "bfloat16"][int(rng.integers(3))]
    steps = []  # (name, operands) over pool = [x, y, w(row vector)] + results; "full" and "stat" values tracked apart
    full, stats = [0, 1], []
    n_in = 3
    for _ in range(int(rng.integers(1, 4))):
        k = n_in + len(steps)
        steps.append((["add", "mul", "sub"][int(rng.integers(3))], (int(rng.choice(full)), int(rng.choice(full + [2])))))
        full.append(k)
    for _ in range(int(rng.integers(1, 3))):  # one or two rounds of: statistic of a full value, then full (op) statistic
        k = n_in + len(steps)
        steps.append((["row_sum", "row_mean", "row_max", "row_sumsq"][int(rng.integers(4))], (int(rng.choice(full)),)))
        stats.append(k)
        steps.append((["sub", "mul", "div_shift", "add"][int(rng.integers(4))], (int(rng.choice(full)), k)))
        full.append(k + 1)
        if rng.random() < 0.5:
            steps.append((["tanh", "exp_capped", "half", "mul_w"][int(rng.integers(4))], (k + 1,)))
            full.append(k + 2)
    outputs = [("value", full[-1])]
    for _ in range(int(rng.integers(0, 3))):
        kind = ["sum_first", "sum_leading", "sum_all", "sum_last", "max_last", "stat"][int(rng.integers(6))]
        outputs.append((kind, int(rng.choice(stats)) if kind == "stat" else int(rng.choice(full[2:]))))
    return shape, dtype, steps, outputs


def reducing_input_types(recipe):
    shape, dtype, _, _ = recipe
    return [(dtype, shape), (dtype, shape), (dtype, shape[-1:])]


def draw_reducing_inputs(recipe, seed: int):
    rng = np.random.default_rng(seed + 56_000)
    arrays = [rng.standard_normal(s).astype(np.float32) for _, s in reducing_input_types(recipe)]
    if recipe[1] == "bfloat16":
        from tests.helpers import bf16

        arrays = [bf16(a) for a in arrays]
    return arrays


def build_reducing(recipe):
    shape, dtype, steps, outputs = recipe

    def program(x, y, w):
        pool = [x, y, w]
        for name, args in steps:
            v = [pool[a] for a in args]
            if name in ("add", "mul", "sub"):
                out = getattr(F, name)(v[0], v[1])
            elif name in ("row_sum", "row_mean", "row_max", "row_sumsq"):
                # statistics in float32, as models compute them (a sum accumulated in bfloat16 depends on the order of
                # its terms far beyond any tolerance), then back to the program's type
                wide = v[0] if dtype != "bfloat16" else prims.cast(v[0], "float32")
                if name == "row_sum":
                    out = F.sum(wide, -1, keepdim=True)
                elif name == "row_mean":
                    out = F.mean(wide, -1, keepdim=True)
                elif name == "row_max":
                    out = F.amax(wide, -1, keepdim=True)
                else:
                    out = F.mean(F.mul(wide, wide), -1, keepdim=True)
                out = out if dtype != "bfloat16" else prims.cast(out, dtype)
            elif name == "div_shift":
                out = F.div(v[0], F.add(F.abs(v[1]), 1.0))
            elif name == "tanh":
                out = prims.tanh(v[0])
            elif name == "exp_capped":
                out = prims.exp(F.minimum(v[0], 3.0))
            elif name == "half":
                out = F.mul(v[0], 0.5)
            else:
                out = F.mul(v[0], w)
            pool.append(out)
        results = []
        for kind, v in outputs:
            t = pool[v]
            wide = t if t.dtype != "bfloat16" or kind in ("value", "stat", "max_last") else prims.cast(t, "float32")
            if kind in ("value", "stat"):
                results.append(t)
            elif kind == "sum_first":
                results.append(F.sum(wide, 0))
            elif kind == "sum_leading":
                results.append(F.sum(wide, tuple(range(len(shape) - 1))))
            elif kind == "sum_all":
                results.append(F.sum(wide))
            elif kind == "sum_last":
                results.append(F.sum(wide, -1))
            else:
                results.append(F.amax(wide, -1))
        return tuple(results)

    return program


# ---- programs of matrix products: every operand layout, ragged sizes, the epilogues, two products in a row --------------

GEMM_M = [1, 7, 64, 100, 128, 129, 300, 1000]
GEMM_K = [8, 16, 33, 40, 50, 64, 72, 256, 1000]
GEMM_N = [8, 24, 30, 64, 65, 128, 136, 512]


def draw_gemm_recipe(seed: int):
    """(dtype, out dtype, m, k, n, lhs contraction axis, rhs contraction axis, tail, n2): `tail` is "none", "relu", "add"
    (a residual of the product's shape), "mask" (the product where another tensor is positive), "scale" (an element-wise
    step after the product) or "chain" (a second product with a [n, n2] matrix)."""
    rng = np.random.default_rng(seed + 33_000)
    dtype = ["bfloat16", "bfloat16", "float32"][int(rng.integers(3))]
    out = dtype if rng.random() < 0.7 else "float32"
    m, k, n = (int(rng.choice(c)) for c in (GEMM_M, GEMM_K, GEMM_N))
    tail = ["none", "relu", "add", "scale", "chain", "mask"][int(rng.integers(6))]
    return dtype, out, m, k, n, int(rng.integers(2)), int(rng.integers(2)), tail, int(rng.choice(GEMM_N))


def gemm_input_types(recipe):
    dtype, out, m, k, n, lc, rc, tail, n2 = recipe
    types = [(dtype, (m, k) if lc == 1 else (k, m)), (dtype, (k, n) if rc == 0 else (n, k))]
    if tail in ("add", "mask"):
        types.append((out, (m, n)))
    if tail == "chain":
        types.append((out, (n, n2)))
    return types


def draw_gemm_inputs(recipe, seed: int):
    rng = np.random.default_rng(seed + 34_000)
    arrays = []
    for dtype, shape in gemm_input_types(recipe):
        a = (rng.standard_normal(shape) / np.sqrt(shape[0])).astype(np.float32) if len(arrays) else rng.standard_normal(shape).astype(np.float32)
        if dtype == "bfloat16":
            from tests.helpers import bf16

            a = bf16(a)
        arrays.append(a)
    return arrays


def build_gemm(recipe, exact: bool = False):
    """With `exact`, everything is float64 (the inputs too): the ground truth."""
    dtype, out, m, k, n, lc, rc, tail, n2 = recipe
    accum, out = ("float64", "float64") if exact else ("float32", out)

    def program(x, w, *rest):
        y = prims.dot_general(x, w, (((lc,), (rc,)), ((), ())), accum, out)
        if tail == "relu":
            y = F.relu(y)
        elif tail == "add":
            y = F.add(y, rest[0])
        elif tail == "mask":  # a relu's backward: the product where the relu's output was positive
            y = F.where(F.lt(0.0, rest[0]), y, 0.0)
        elif tail == "scale":
            y = F.mul(prims.tanh(y), 0.5)
        elif tail == "chain":
            y = prims.dot_general(y, rest[0], (((1,), (0,)), ((), ())), accum, out)
        return y

    return program


# ---- small random models differentiated by autograd: loss and every parameter's gradient --------------------------------

MODEL_LAYERS = ["linear_relu", "linear", "layer_norm", "rms_norm", "residual_mlp", "gelu", "silu", "swiglu"]


def draw_model_recipe(seed: int):
    """(rows, width, layers, loss, classes): each layer is (kind, sizes); parameters are created per layer. `loss` is
    "mse" (against a target of the last width) or "ce" (cross entropy against integer classes, after a head)."""
    rng = np.random.default_rng(seed + 21_000)
    rows = int(rng.choice([48, 64, 200]))
    width = int(rng.choice([32, 64, 96]))
    layers, d = [], width
    for _ in range(int(rng.integers(2, 5))):
        kind = MODEL_LAYERS[int(rng.integers(len(MODEL_LAYERS)))]
        if kind in ("linear_relu", "linear"):
            d2 = int(rng.choice([32, 64, 128]))
            layers.append((kind, (d, d2)))
            d = d2
        elif kind in ("residual_mlp", "swiglu"):
            layers.append((kind, (d, int(rng.choice([64, 128])))))
        else:
            layers.append((kind, (d,)))
    loss = ["mse", "ce"][int(rng.integers(2))]
    if loss == "mse" and all(kind in ("gelu", "silu") for kind, _ in layers):
        layers.append(("linear", (d, d)))  # something to differentiate with respect to
    return rows, width, layers, loss, int(rng.choice([10, 50])), d


def model_parameter_shapes(recipe):
    rows, width, layers, loss, classes, d_out = recipe
    shapes = []
    for kind, size in layers:
        if kind in ("linear_relu", "linear"):
            shapes.append(size)
        elif kind == "residual_mlp":
            shapes += [size, (size[1], size[0])]
        elif kind == "swiglu":
            shapes += [size, size, (size[1], size[0])]
        elif kind == "layer_norm":
            shapes += [size, size]
        elif kind == "rms_norm":
            shapes.append(size)
    if loss == "ce":
        shapes.append((d_out, classes))
    return shapes


def model_input_types(recipe, dtype="float32"):
    rows, width, layers, loss, classes, d_out = recipe
    target = ("int64", (rows,)) if loss == "ce" else (dtype, (rows, d_out))
    return [(dtype, (rows, width)), target] + [(dtype, s) for s in model_parameter_shapes(recipe)]


def draw_model_inputs(recipe, seed: int):
    rows, width, layers, loss, classes, d_out = recipe
    rng = np.random.default_rng(seed + 22_000)
    x = rng.standard_normal((rows, width)).astype(np.float32)
    target = rng.integers(0, classes, rows) if loss == "ce" else rng.standard_normal((rows, d_out)).astype(np.float32)
    params = []
    for shape in model_parameter_shapes(recipe):
        params.append((rng.standard_normal(shape) / np.sqrt(shape[0])).astype(np.float32) if len(shape) == 2
                      else (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32))
    return [x, target] + params


def build_model(recipe, dtype="float32"):
    """`step(x, target, *params) -> (loss, *gradients)`, float32 products accumulated in float32 (float64 for the ground
    truth)."""
    from lumen_b200 import autograd

    rows, width, layers, loss, classes, d_out = recipe

    def forward(x, target, *params):
        it = iter(params)
        h = x
        for kind, size in layers:
            if kind == "linear_relu":
                h = F.relu(F.matmul(h, next(it), dtype, dtype))
            elif kind == "linear":
                h = F.matmul(h, next(it), dtype, dtype)
            elif kind == "residual_mlp":
                w1, w2 = next(it), next(it)
                h = F.add(h, F.matmul(F.relu(F.matmul(h, w1, dtype, dtype)), w2, dtype, dtype))
            elif kind == "swiglu":
                g, u, d = next(it), next(it), next(it)
                h = F.add(h, F.matmul(F.swiglu(F.matmul(h, g, dtype, dtype), F.matmul(h, u, dtype, dtype)), d, dtype, dtype))
            elif kind == "layer_norm":
                h = F.layer_norm(h, next(it), next(it))
            elif kind == "rms_norm":
                h = F.rms_norm(h, next(it), 1e-5)
            elif kind == "gelu":
                h = F.gelu(h)
            else:
                h = F.silu(h)
        if loss == "ce":
            return F.mean(F.cross_entropy(F.matmul(h, next(it), dtype, dtype), target))
        r = F.sub(h, target)
        return F.mean(F.mul(r, r))

    n_params = len(model_parameter_shapes(recipe))

    def step(x, target, *params):
        value, grads = autograd.value_and_grad(lambda *p: forward(x, target, *p), tuple(range(n_params)))(*params)
        return (value, *grads)

    return step


# ---- optimizer steps over lists of parameters of unrelated shapes (the horizontally fused launches) ----------------------

PARAMETER_SHAPES = [(7,), (128,), (33, 5), (64, 64), (1000,), (3, 4, 8), (256, 130), (1,), (300007,), (96, 1024), (2, 3)]


def draw_optimizer_recipe(seed: int):
    """(kind, dtype, shapes, learning rate as an operand?): "sgd" or "adamw" over 2 - 24 parameters drawn from shapes
    that share no row length, some repeated."""
    rng = np.random.default_rng(seed + 63_000)
    kind = ["sgd", "adamw"][int(rng.integers(2))]
    dtype = ["float32", "bfloat16"][int(rng.integers(2))]
    count = int(rng.integers(2, 25))
    shapes = [PARAMETER_SHAPES[int(rng.integers(len(PARAMETER_SHAPES)))] for _ in range(count)]
    return kind, dtype, shapes, bool(rng.integers(2))


def optimizer_input_types(recipe):
    kind, dtype, shapes, runtime_rate = recipe
    types = []
    for s in shapes:
        types += [(dtype, s), (dtype, s)] + ([("float32", s), ("float32", s)] if kind == "adamw" else [])
    return types + ([("float32", ())] if runtime_rate else [])


def draw_optimizer_inputs(recipe, seed: int):
    kind, dtype, shapes, runtime_rate = recipe
    rng = np.random.default_rng(seed + 64_000)
    arrays = []
    for t, s in optimizer_input_types(recipe):
        if s == () and t == "float32" and runtime_rate and len(arrays) == len(optimizer_input_types(recipe)) - 1:
            arrays.append(np.float32(3.0) if kind == "adamw" else np.float32(0.05))  # the step count / the learning rate
            continue
        a = rng.standard_normal(s).astype(np.float32)
        if kind == "adamw" and len(arrays) % 4 == 3:
            a = np.abs(a)  # second moments are not negative
        if t == "bfloat16":
            from tests.helpers import bf16

            a = bf16(a)
        arrays.append(a)
    return arrays


def build_optimizer(recipe):
    """`step(*tensors)`: per parameter (p, g) -> p' for SGD, (p, g, m, v) -> (p', m', v') for AdamW; the trailing 0-d
    operand, when present, is SGD's learning rate or AdamW's step count."""
    from lumen_b200 import nn

    kind, dtype, shapes, runtime_rate = recipe
    per = 4 if kind == "adamw" else 2

    def step(*tensors):
        scalar = tensors[-1] if runtime_rate else None
        results = []
        for k in range(len(shapes)):
            group = tensors[per * k : per * (k + 1)]
            if kind == "sgd":
                results.append(nn.sgd_update(group[0], group[1], scalar if runtime_rate else 0.05))
            else:
                results += list(nn.adamw_update(group[0], group[2], group[3], group[1], scalar if runtime_rate else 3))
        return tuple(results)

    return step


# ---- programs of indexing functions: gathers, one-hot rows, triangles, paddings, concatenations, arg-reductions ----------

def draw_indexing_recipe(seed: int):
    """(dtype, id dtype, vocabulary, batch, sequence, width, steps): a table [vocabulary, width] gathered by ids
    [batch, sequence] plus a positional table [sequence, width], followed by one to three of: "triu" (upper triangle of
    the last two axes), "pad" (constant blocks around the last two axes), "cat_self" / "stack_self" (the value beside a
    scaled copy of itself along a drawn axis), "clamp"; the outputs add the arg-maximum and arg-minimum over the last
    axis, a one-hot of the ids compared with the arg-maximum, and the row sums of the one-hot times a weight."""
    rng = np.random.default_rng(seed + 47_000)
    dtype = ["float32", "bfloat16"][int(rng.integers(2))]
    ids = ["int64", "int32"][int(rng.integers(2))]
    vocab, batch, seq, width = (int(rng.choice(c)) for c in ([5, 50, 1000], [1, 2, 5], [1, 7, 32, 100], [8, 33, 64, 96]))
    steps = []
    for _ in range(int(rng.integers(1, 4))):
        name = ["triu", "pad", "cat_self", "stack_self", "clamp"][int(rng.integers(5))]
        if name == "triu":
            steps.append((name, int(rng.integers(-2, 3))))
        elif name == "pad":
            steps.append((name, tuple(int(p) for p in rng.integers(0, 4, size=4))))
        elif name in ("cat_self", "stack_self"):
            steps.append((name, int(rng.integers(0, 3))))
        else:
            steps.append((name, (-0.5, 0.75)))
    return dtype, ids, vocab, batch, seq, width, steps


def indexing_input_types(recipe):
    dtype, ids, vocab, batch, seq, width, _ = recipe
    return [(dtype, (vocab, width)), (dtype, (seq, width)), (ids, (batch, seq))]


def draw_indexing_inputs(recipe, seed: int):
    dtype, ids, vocab, batch, seq, width, _ = recipe
    rng = np.random.default_rng(seed + 48_000)
    table, pos = (rng.standard_normal(s).astype(np.float32) for s in ((vocab, width), (seq, width)))
    picks = rng.integers(0, vocab, (batch, seq)).astype(ids)
    if dtype == "bfloat16":
        from tests.helpers import bf16

        table, pos = bf16(table), bf16(pos)
    return [table, pos, picks]


def build_indexing(recipe):
    dtype, ids, vocab, batch, seq, width, steps = recipe

    def program(table, pos, picks):
        h = F.add(prims.gather(table, picks, 0), pos)  # [batch, sequence, width]
        first = h
        for name, param in steps:
            if name == "triu":
                h = F.triu(h, param)
            elif name == "pad":
                h = F.pad(h, param, 1.5)
            elif name == "cat_self":
                h = F.cat([h, F.mul(h, 2.0)], param)
            elif name == "stack_self":
                h = F.stack([h, F.neg(h)], param)
            else:
                h = F.clamp(h, param[0], param[1])
        best = F.argmax(first, -1)
        hot = F.one_hot(picks, vocab, "float32")
        return (h, best, F.argmin(first, -1), F.eq(prims.cast(best, ids), picks),
                F.sum(F.mul(hot, prims.cast(prims.iota(ids, (batch, seq, vocab), 2), "float32")), -1))

    return program
