"""Parity of the generated fused kernels with the CPU oracle, through the C ABI, on a B200."""

import numpy as np
import pytest
import torch

from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from lumen_b200.runtime import Fusion
from tests.helpers import BF16, bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def chain(x, g, b):
    y = F.relu(x * g + b)
    return y, prims.reduce_sum(y * y, (1,), "float32")


def chain_inputs(rows, cols, dtype, seed=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32)
    if dtype == "bfloat16":
        x, g, b = bf16(x), bf16(g), bf16(b)
    return x, g, b


def device_run(graph, inputs, cuda):
    outs = Fusion(graph)(*[to_torch(a, cuda) for a in inputs])
    torch.cuda.synchronize()
    return [to_numpy(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(64, 4096), (7, 1000), (33, 36), (1, 8), (5, 3)])
def test_chain_matches_oracle(cuda, dtype, shape):
    """y = relu(x*g+b) is bit-exact (one rounding per primitive); the row sum of squares differs from the
    sequential sum only by its order (rtol 1e-5, the reference's own tolerance for device reductions,
    tests/graph_compiler/test_elementwise_fusion.py:112-120)."""
    rows, cols = shape
    g = tracer.trace(chain, (dtype, shape), (dtype, (cols,)), (dtype, (cols,)))
    inputs = chain_inputs(rows, cols, dtype)
    y, s = device_run(g, inputs, cuda)
    want_y, want_s = run_oracle(g, inputs)
    assert y.dtype == want_y.dtype
    np.testing.assert_array_equal(y.view(np.uint16 if dtype == "bfloat16" else np.uint32), want_y.view(np.uint16 if dtype == "bfloat16" else np.uint32))
    np.testing.assert_allclose(s, want_s, rtol=1e-5, atol=1e-6)


def test_chain_sum_only(cuda):
    def f(x, g, b):
        return chain(x, g, b)[1]

    g = tracer.trace(f, ("float32", (128, 512)), ("float32", (512,)), ("float32", (512,)))
    inputs = chain_inputs(128, 512, "float32")
    (s,) = device_run(g, inputs, cuda)
    (want,) = run_oracle(g, inputs)
    np.testing.assert_allclose(s, want, rtol=1e-5)


def test_full_size_chain_properties(cuda):
    """At the benchmark's full size ([16384, 4096]) the oracle is too slow to run whole: check rows sampled against
    it, and size-independent properties: y >= 0, s == sum(y*y) recomputed in float64 from the device's y."""
    rows, cols = 16384, 4096
    g = tracer.trace(chain, ("float32", (rows, cols)), ("float32", (cols,)), ("float32", (cols,)))
    x, gg, b = chain_inputs(rows, cols, "float32")
    y, s = device_run(g, (x, gg, b), cuda)
    assert (y >= 0).all()
    np.testing.assert_allclose(s, (y.astype(np.float64) ** 2).sum(1), rtol=1e-5)
    sample = np.arange(0, rows, 1021)
    small = tracer.trace(chain, ("float32", (len(sample), cols)), ("float32", (cols,)), ("float32", (cols,)))
    want_y, want_s = run_oracle(small, (x[sample], gg, b))
    np.testing.assert_array_equal(y[sample], want_y)
    np.testing.assert_allclose(s[sample], want_s, rtol=1e-5)


def test_layer_norm_rows(cuda):
    """Layer norm spelled from prims (tests/graph_compiler/test_normalizations.py:103-106) as one row kernel; the
    bfloat16 variant widens to float32 for the statistics and narrows the result, as a bfloat16 model does
    (a sum accumulated in bfloat16 itself depends on the order of its 1024 terms far beyond any tolerance)."""
    def ln16(a, w, b):
        return F.layer_norm(a.float(), w.float(), b.float()).bfloat16()

    for dtype, f, tol in (("float32", F.layer_norm, 1e-5), ("bfloat16", ln16, 2**-7)):
        g = tracer.trace(f, (dtype, (96, 1024)), (dtype, (1024,)), (dtype, (1024,)))
        rng = np.random.default_rng(5)
        a = rng.standard_normal((96, 1024)).astype(np.float32) * 2 + 0.5
        w = rng.uniform(0.5, 1.5, 1024).astype(np.float32)
        b = rng.standard_normal(1024).astype(np.float32)
        inputs = (a, w, b) if dtype == "float32" else (bf16(a), bf16(w), bf16(b))
        (y,) = device_run(g, inputs, cuda)
        (want,) = run_oracle(g, inputs)
        np.testing.assert_allclose(y.astype(np.float32), want.astype(np.float32), rtol=tol, atol=tol)


def test_bfloat16_accumulated_sum(cuda):
    """A sum accumulated in bfloat16 (F.sum of a bfloat16 tensor): within the reference's 2e-1 for
    bf16-accumulated reductions (tests/graph_compiler/test_elementwise_fusion.py:112-120) on short rows."""
    g = tracer.trace(lambda x: F.sum(x, -1), ("bfloat16", (64, 32)))
    x = bf16(np.random.default_rng(8).standard_normal((64, 32)))
    (s,) = device_run(g, (x,), cuda)
    (want,) = run_oracle(g, (x,))
    np.testing.assert_allclose(s.astype(np.float32), want.astype(np.float32), rtol=2e-1, atol=2e-1)


def test_softmax_rows(cuda):
    g = tracer.trace(lambda x: F.softmax(x, -1), ("float32", (50, 300)))
    x = np.random.default_rng(6).standard_normal((50, 300)).astype(np.float32) * 3
    (y,) = device_run(g, (x,), cuda)
    (want,) = run_oracle(g, (x,))
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-7)


def test_embedding_gather_is_exact(cuda):
    """tokens[ids] + positions: indices clamped (lumen/reference/mod.rs:414-423), result bit-exact."""
    def f(tok, pos, ids):
        return (tok[ids] + pos).reshape(8 * 64, 128)

    g = tracer.trace(f, ("float32", (256, 128)), ("float32", (64, 128)), ("int64", (8, 64)))
    rng = np.random.default_rng(0)
    tok = rng.standard_normal((256, 128)).astype(np.float32)
    pos = rng.standard_normal((64, 128)).astype(np.float32)
    ids = rng.integers(-3, 260, (8, 64))  # some out of range: clamped
    (y,) = device_run(g, (tok, pos, ids), cuda)
    (want,) = run_oracle(g, (tok, pos, ids))
    np.testing.assert_array_equal(y, want)


def test_integer_rules_are_exact(cuda):
    """Integer division by zero is -1, overflow wraps, casts saturate (lumen/reference/mod.rs:448-468,203-220)."""
    def f(a, b, x):
        q = prims.div(a, b)
        return q, prims.mul(a, b), prims.cast(x, "int32"), prims.cast(x, "uint8"), prims.lt(a, b), prims.max(a, b)

    g = tracer.trace(f, ("int32", (64,)), ("int32", (64,)), ("float32", (64,)))
    rng = np.random.default_rng(2)
    a = rng.integers(-(2**31), 2**31 - 1, 64).astype(np.int32)
    b = rng.integers(-(2**31), 2**31 - 1, 64).astype(np.int32)
    b[:4] = 0
    a[4], b[4] = -(2**31), -1
    x = (rng.standard_normal(64) * 1e10).astype(np.float32)
    x[:3] = [np.nan, np.inf, -np.inf]
    got = device_run(g, (a, b, x), cuda)
    want = run_oracle(g, (a, b, x))
    for u, v in zip(got, want):
        np.testing.assert_array_equal(u, v)
    assert got[0][0] == -1


def test_unsigned_division_by_the_largest_value(cuda):
    """A divisor of all ones is -1 only for signed types (where the quotient is the wrapped negation and the remainder
    0); for unsigned types it is the largest value, an ordinary divisor."""
    for dtype in ("uint8", "uint32", "int32", "int8"):
        info = np.iinfo(dtype)
        rng = np.random.default_rng(4)
        a = rng.integers(info.min, info.max, 256, dtype=dtype, endpoint=True)
        b = rng.integers(info.min, info.max, 256, dtype=dtype, endpoint=True)
        b[::3] = np.array(-1).astype(dtype)  # all ones
        a[0], a[3] = info.min, info.max
        g = tracer.trace(lambda x, y: (prims.div(x, y), prims.rem(x, y)), (dtype, (256,)), (dtype, (256,)))
        got, want = device_run(g, (a, b), cuda), run_oracle(g, (a, b))
        for u, v in zip(got, want):
            np.testing.assert_array_equal(u, v, err_msg=dtype)


@pytest.mark.parametrize("dtype", ["int8", "int16", "int32", "int64"])
@pytest.mark.parametrize("shape", [(7, 5, 32), (300, 32), (40, 257)])
def test_integer_extrema_of_negations(cuda, dtype, shape):
    """Row minima and maxima of negated integers, however the negation is spelled (`neg`, `0 - x`, `x * -1`, `abs`), alone
    and beside a full-sized result of the same kernel. The toolchain turns a chain of signed 32-bit max over literal
    negations into the extremum over x and -x together; the generated kernels spell negations so that it cannot."""
    info = np.iinfo(dtype)
    rng = np.random.default_rng(6)
    x = rng.integers(info.min, info.max, shape, dtype=dtype, endpoint=True)
    y = rng.integers(info.min, info.max, shape, dtype=dtype, endpoint=True)

    def program(a, b):
        m = prims.max(a, b)
        return (F.amin(a, -1), F.amax(prims.neg(a), -1), F.amax(F.sub(0, a), -1), F.amax(F.mul(a, -1), -1), F.amax(F.abs(b), -1),
                m, F.amin(m, -1), F.amin(prims.neg(m), -1),
                prims.max(prims.max(prims.max(prims.neg(a), prims.neg(b)), prims.neg(m)), F.sub(0, prims.min(a, b))))  # fmt: skip

    g = tracer.trace(program, (dtype, shape), (dtype, shape))
    want = run_oracle(g, (x, y))
    import lumen_b200

    got = lumen_b200.compile(program)(to_torch(x, cuda), to_torch(y, cuda))
    torch.cuda.synchronize()
    for k, (u, v) in enumerate(zip(got, want)):
        np.testing.assert_array_equal(to_numpy(u), v, err_msg=f"output {k}")


def test_unsupported_primitive_is_named(cuda):
    from lumen_b200._lib import LumenError

    g = tracer.trace(lambda x: prims.reduce_sum(x, (1,), "float32"), ("float32", (4, 5, 6)))
    with pytest.raises(LumenError, match="reduce_sum"):
        Fusion(g)


def test_column_reductions(cuda):
    """Sums over the leading axis (weight gradients of a layer norm): partial sums per row slice, then a finalize
    pass, both in a fixed order; against the oracle's sequential sums."""
    rows, cols = 1000, 384

    def f(dy, x, mean, rstd):
        xhat = (x.float() - mean.reshape(rows, 1)) * rstd.reshape(rows, 1)
        g = dy.float()
        return prims.reduce_sum(g * xhat, (0,), "float32").bfloat16(), prims.reduce_sum(g, (0,), "float32")

    g = tracer.trace(f, ("bfloat16", (rows, cols)), ("bfloat16", (rows, cols)), ("float32", (rows,)), ("float32", (rows,)))
    rng = np.random.default_rng(7)
    inputs = (bf16(rng.standard_normal((rows, cols))), bf16(rng.standard_normal((rows, cols))),
              rng.standard_normal(rows).astype(np.float32), rng.uniform(0.5, 2, rows).astype(np.float32))
    got = device_run(g, inputs, cuda)
    want = run_oracle(g, inputs)
    np.testing.assert_allclose(got[0].astype(np.float32), want[0].astype(np.float32), rtol=2**-7, atol=2**-7 * np.abs(want[0].astype(np.float32)).max())
    np.testing.assert_allclose(got[1], want[1], rtol=1e-4, atol=1e-4 * np.abs(want[1]).max())
    again = device_run(g, inputs, cuda)
    np.testing.assert_array_equal(got[1], again[1])


def test_cross_entropy_rows(cuda):
    """Per-row logsumexp - x[target] with the target logit gathered by a data-dependent index, and its gradient."""
    rows, classes = 96, 1000
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((rows, classes)) * 3).astype(np.float32)
    t = rng.integers(0, classes, rows)
    g = tracer.trace(lambda a, c: F.cross_entropy_forward_prims(a, c), ("float32", x.shape), ("int64", t.shape))
    loss, lse = device_run(g, (x, t), cuda)
    want_loss, want_lse = run_oracle(g, (x, t))
    np.testing.assert_allclose(lse, want_lse, rtol=1e-5)
    np.testing.assert_allclose(loss, want_loss, rtol=1e-5, atol=1e-5)
    gb = tracer.trace(lambda a, c, l, gg: F.cross_entropy_backward_prims(a, c, l, gg).bfloat16(),
                      ("float32", x.shape), ("int64", t.shape), ("float32", (rows,)), ("float32", (rows,)))
    gg = rng.standard_normal(rows).astype(np.float32)
    (dx,) = device_run(gb, (x, t, want_lse, gg), cuda)
    (want,) = run_oracle(gb, (x, t, want_lse, gg))
    np.testing.assert_allclose(dx.astype(np.float32), want.astype(np.float32), rtol=2**-7, atol=1e-6)


def test_inplace_update(cuda):
    """`p - lr * g` written over `p` (a donated output): the kernel is generated without read-only loads."""
    from lumen_b200 import nn
    from lumen_b200.compiler import compile_graph
    from lumen_b200.plan import Plan

    def step(p, gr):
        return nn.sgd_update(p, gr, 0.5)

    gph = tracer.trace(step, ("float32", (300, 70)), ("float32", (300, 70)))
    rng = np.random.default_rng(9)
    p0, gr = rng.standard_normal((300, 70)).astype(np.float32), rng.standard_normal((300, 70)).astype(np.float32)
    (want,) = run_oracle(gph, (p0, gr))
    plan = Plan(compile_graph(gph, {0: 0}), cuda)
    assert "option inplace" in plan.compiled.text
    p_t, g_t = to_torch(p0, cuda), to_torch(gr, cuda)
    plan.run([p_t, g_t], [p_t])
    torch.cuda.synchronize()
    np.testing.assert_array_equal(to_numpy(p_t), want)


_ = BF16
