"""Pins the CPU oracle (oracle/oracle.cpp) to the reference's own known-answer checks for this path.

The reference holds no binary fixtures here; its tests recompute expectations in NumPy. Each test below restates
one of those checks (cited) against the oracle, plus exact-arithmetic rounding vectors from tests/golden/."""

import json
import os

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from oracle import oracle
from tests.helpers import BF16, attention_f64, bf16

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def run1(f, *arrays):
    names = {v: k for k, v in oracle.NUMPY.items()}
    g = tracer.trace(f, *[(names[np.dtype(a.dtype)], a.shape) for a in arrays])
    return oracle.run(g, arrays)


def test_rounding_matches_exact_arithmetic():
    """round() of lumen/reference/mod.rs:189-200: one correct rounding from f64 (lumen/tensor/dtype.rs:217-239)."""
    with open(os.path.join(GOLDEN, "rounding_vectors.json")) as f:
        v = json.load(f)
    xs = [float.fromhex(h) for h in v["inputs_hex"]]
    for dtype in ("bfloat16", "float16", "float32"):
        want = [float.fromhex(h) for h in v[dtype]]
        got = [oracle.round_to(x, dtype) for x in xs]
        for x, g, w in zip(xs, got, want):
            assert g == w and np.signbit(g) == np.signbit(w), (dtype, x.hex(), g, w)


def test_bf16_cast_matches_the_reference_bit_trick():
    """`_bf16` of tests/test_transformer_example.py:211-216: add 0x7FFF plus the lowest kept bit, truncate."""
    rng = np.random.default_rng(0)
    a = np.concatenate([(rng.standard_normal(4096) * 10.0 ** rng.integers(-20, 20, 4096)).astype(np.float32),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40], np.float32)])
    bits = a.view(np.uint32)
    want = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
    (got,) = run1(lambda x: prims.cast(x, "bfloat16"), a)
    np.testing.assert_array_equal(got.astype(np.float32).view(np.uint32), want.view(np.uint32))


def test_integer_edge_rules():
    """Division by zero is -1 and remainder by zero the dividend, abs of the minimum wraps, products wrap
    (tests/codegen/test_elementwise.py:113-180; lumen/reference/mod.rs:448-468,563-570)."""
    a = np.array([7, -7, -(2**31), 2**31 - 1, 5, 0], np.int32)
    b = np.array([0, 0, -1, 2, -3, 0], np.int32)
    q, r, m, ab, sg = run1(lambda x, y: (prims.div(x, y), prims.rem(x, y), prims.mul(x, y), prims.abs(x), prims.sign(x)), a, b)
    np.testing.assert_array_equal(q, [-1, -1, -(2**31), 2**30 - 1, -1, -1])
    np.testing.assert_array_equal(r, [7, -7, 0, 1, 2, 0])
    np.testing.assert_array_equal(m, (a.astype(np.int64) * b.astype(np.int64)).astype(np.int32))
    np.testing.assert_array_equal(ab, np.abs(a))  # abs(INT_MIN) wraps to INT_MIN in numpy too
    np.testing.assert_array_equal(sg, np.sign(a))
    (n,) = run1(lambda x: prims.not_(x), a)
    np.testing.assert_array_equal(n, ~a)
    (nb,) = run1(lambda x: prims.not_(x), np.array([True, False]))
    np.testing.assert_array_equal(nb, [False, True])


def test_float_to_int_casts_saturate():
    """Casts saturate and send NaN to 0 (lumen/reference/mod.rs:203-220)."""
    x = np.array([np.nan, np.inf, -np.inf, 3e9, -3e9, 2.9, -2.9, 255.5, 300.0], np.float32)
    i32, u8 = run1(lambda t: (prims.cast(t, "int32"), prims.cast(t, "uint8")), x)
    np.testing.assert_array_equal(i32, [0, 2**31 - 1, -(2**31), 2**31 - 1, -(2**31), 2, -2, 255, 300])
    np.testing.assert_array_equal(u8, [0, 255, 0, 255, 0, 2, 0, 255, 255])


def test_max_propagates_nan_and_min_is_negated_max():
    x = np.array([1.0, np.nan, 2.0, -0.0], np.float32)
    y = np.array([np.nan, 1.0, 1.0, 0.0], np.float32)
    mx, mn = run1(lambda a, b: (F.maximum(a, b), F.minimum(a, b)), x, y)
    assert np.isnan(mx[:2]).all() and np.isnan(mn[:2]).all()
    assert mx[2] == 2.0 and mn[2] == 1.0


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-5), ("bfloat16", 1e-2)])
def test_matmul_against_numpy(dtype, tol):
    """`a @ b` within tol * max|want| (tests/codegen/test_dot_general.py:30-42)."""
    rng = np.random.default_rng(3)
    a = rng.standard_normal((70, 96)).astype(np.float32)
    b = rng.standard_normal((96, 50)).astype(np.float32)
    if dtype == "bfloat16":
        a, b = bf16(a), bf16(b)
    (got,) = run1(lambda x, y: F.matmul(x, y, "float32", dtype), a, b)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(got.astype(np.float64) - want).max() <= tol * np.abs(want).max()


def test_matmul_accumulates_sequentially_in_float32():
    """Products and partial sums rounded to the accumulator in contracting order (mod.rs:958-970)."""
    rng = np.random.default_rng(4)
    a = rng.standard_normal((5, 300)).astype(np.float32)
    b = rng.standard_normal((300, 4)).astype(np.float32)
    (got,) = run1(lambda x, y: F.matmul(x, y, "float32", "float32"), a, b)
    want = np.zeros((5, 4), np.float32)
    for k in range(300):
        want = want + a[:, k : k + 1] * b[k : k + 1, :]
    np.testing.assert_array_equal(got, want)


# (B, Sq, Sk, N, Nkv, H, Hv), causal — the shapes of tests/functional/test_attention.py:56-63, shortened where long
CASES = [((2, 20, 20, 4, 4, 16, 16), False), ((1, 13, 7, 2, 2, 8, 8), False), ((2, 20, 20, 4, 2, 16, 16), True),
         ((1, 1, 30, 8, 2, 32, 32), True), ((2, 5, 40, 2, 1, 16, 24), False), ((1, 7, 20, 2, 2, 32, 32), True)]  # fmt: skip


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", CASES)
def test_attention_forward_against_float64(case, dtype):
    """TOL of tests/functional/test_attention.py:54,100-102: 2e-6 (f32), 2e-2 (bf16), rtol = atol."""
    (b, sq, sk, n, nkv, h, hv), causal = case
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal(s).astype(np.float32) for s in ((b, sq, n, h), (b, sk, nkv, h), (b, sk, nkv, hv)))
    if dtype == "bfloat16":
        q, k, v = bf16(q), bf16(k), bf16(v)
    o, lse = run1(lambda a, c, d: F.attention_forward_prims(a, c, d, 1 / np.sqrt(h), causal), q, k, v)
    want, want_lse = attention_f64(q, k, v, causal)
    tol = {"float32": 2e-6, "bfloat16": 2e-2}[dtype]
    np.testing.assert_allclose(o.astype(np.float64), want, rtol=tol, atol=tol)
    np.testing.assert_allclose(lse[..., 0], want_lse, rtol=1e-5, atol=1e-5)


def test_attention_backward_against_finite_differences():
    """FlashAttention-2's backward as traced (lumen/functional/attention/flash.py:51-85), against float64
    numerical gradients of the float64 forward."""
    rng = np.random.default_rng(1)
    b, s, n, h = 1, 6, 2, 4
    q, k, v, do = (rng.standard_normal((b, s, n, h)).astype(np.float32) for _ in range(4))
    scale = 1 / np.sqrt(h)

    def fwd_bwd(q_, k_, v_, do_):
        o, lse = F.attention_forward_prims(q_, k_, v_, scale, True)
        return F.attention_backward_prims(q_, k_, v_, o, lse, do_, scale, True)

    dq, dk, dv = run1(fwd_bwd, q, k, v, do)

    def loss(q_, k_, v_):
        return (attention_f64(q_, k_, v_, True)[0] * do).sum()

    for x, g in ((q, dq), (k, dk), (v, dv)):
        num = np.zeros_like(x, np.float64)
        for i in np.ndindex(x.shape):
            xp, xm = x.astype(np.float64).copy(), x.astype(np.float64).copy()
            xp[i] += 1e-5
            xm[i] -= 1e-5
            args = [xp if t is x else t for t in (q, k, v)], [xm if t is x else t for t in (q, k, v)]
            num[i] = (loss(*args[0]) - loss(*args[1])) / 2e-5
        np.testing.assert_allclose(g, num, rtol=1e-4, atol=1e-5)


def test_layer_norm_and_softmax_against_numpy():
    """Rows as spelled in tests/graph_compiler/test_normalizations.py:103-106; softmax 1e-6, norms 1e-5
    (tests/graph_compiler/test_elementwise_fusion.py:159-166)."""
    rng = np.random.default_rng(2)
    a = rng.standard_normal((9, 64)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 64).astype(np.float32)
    (y,) = run1(lambda x, s: F.layer_norm(x, s), a, w)
    xc = a.astype(np.float64) - a.astype(np.float64).mean(-1, keepdims=True)
    np.testing.assert_allclose(y, xc / np.sqrt((xc * xc).mean(-1, keepdims=True) + 1e-5) * w, rtol=1e-5, atol=1e-6)
    (p,) = run1(lambda x: F.softmax(x, -1), a)
    e = np.exp(a.astype(np.float64) - a.max(-1, keepdims=True))
    np.testing.assert_allclose(p, e / e.sum(-1, keepdims=True), rtol=1e-6, atol=1e-7)


def test_reductions():
    """f32 sums within 1e-5, integers and max exact, sums in row-major order with the accumulator rounded each
    step (tests/graph_compiler/test_elementwise_fusion.py:112-120; lumen/reference/mod.rs:645-695)."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 33, 5)).astype(np.float32)
    s, m = run1(lambda t: (F.sum(t, 1), F.amax(t, (0, 2))), x)
    np.testing.assert_allclose(s, x.astype(np.float64).sum(1), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(m, x.max((0, 2)))
    seq = np.zeros((4, 5), np.float32)
    for j in range(33):
        seq = seq + x[:, j, :]
    np.testing.assert_array_equal(s, seq)
    i = rng.integers(-100, 100, (6, 7)).astype(np.int32)
    (si,) = run1(lambda t: F.sum(t, 0), i)
    np.testing.assert_array_equal(si, i.sum(0))
    # a bfloat16 sum accumulates in bfloat16: each partial sum is rounded (F.sum, functions.py:265-271)
    xb = bf16(rng.standard_normal(200))
    (sb,) = run1(lambda t: F.sum(t), xb)
    acc = np.float32(0)
    for e in xb.astype(np.float32):
        acc = np.float32(np.float32(acc + e).astype(BF16))
    assert float(sb.astype(np.float32)) == float(acc)


def test_cross_entropy_and_gather_scatter():
    """`logsumexp - x[target]` rows (lumen/functional/cross_entropy/logits.py:19-34); gather clamps indices and
    scatter_add accumulates in order (lumen/reference/mod.rs:414-423,731-808)."""
    rng = np.random.default_rng(6)
    x = rng.standard_normal((10, 17)).astype(np.float32)
    t = rng.integers(0, 17, 10)
    loss, lse = run1(lambda a, c: F.cross_entropy_forward_prims(a, c), x, t)
    x64 = x.astype(np.float64)
    want_lse = np.log(np.exp(x64 - x64.max(-1, keepdims=True)).sum(-1)) + x64.max(-1)
    np.testing.assert_allclose(lse, want_lse, rtol=1e-6)
    np.testing.assert_allclose(loss, want_lse - x64[np.arange(10), t], rtol=1e-5, atol=1e-6)
    g = rng.standard_normal(10).astype(np.float32)
    (dx,) = run1(lambda a, c, l, gg: F.cross_entropy_backward_prims(a, c, l, gg), x, t, lse, g)
    p = np.exp(x64 - want_lse[:, None])
    p[np.arange(10), t] -= 1
    np.testing.assert_allclose(dx, p * g[:, None], rtol=1e-5, atol=1e-6)
    table = rng.standard_normal((5, 3)).astype(np.float32)
    ids = np.array([[0, 7], [-2, 4]])
    (rows,) = run1(lambda tb, i: prims.gather(tb, i, 0), table, ids)
    np.testing.assert_array_equal(rows, table[np.clip(ids, 0, 4)])
    u = rng.standard_normal((2, 2, 3)).astype(np.float32)
    (acc,) = run1(lambda tb, i, uu: prims.scatter_add(tb, i, uu, 0), table, ids, u)
    want = table.copy()
    for a in range(2):
        for b in range(2):
            want[np.clip(ids[a, b], 0, 4)] = want[np.clip(ids[a, b], 0, 4)] + u[a, b]
    np.testing.assert_array_equal(acc, want)


def test_multi_output_fusion_matches_its_body():
    """A fusion evaluates as its body, extra outputs through fusion_output (lumen/reference/mod.rs:71-79)."""
    def chain(x, g, b):
        y = F.relu(x * g + b)
        return y, prims.reduce_sum(y * y, (1,), "float32")

    body = tracer.trace(chain, ("float32", (6, 8)), ("float32", (8,)), ("float32", (8,)))
    outer = tracer.trace(lambda x, g, b: tuple(prims.fusion([x, g, b], body, "reduction")),
                         ("float32", (6, 8)), ("float32", (8,)), ("float32", (8,)))
    rng = np.random.default_rng(1)
    args = [rng.standard_normal(s).astype(np.float32) for s in ((6, 8), (8,), (8,))]
    for a, b in zip(oracle.run(outer, args), oracle.run(body, args)):
        np.testing.assert_array_equal(a, b)


def test_type_rules_reject_hidden_casts():
    """No promotion, explicit accumulation dtype (lumen/graph/primitive.rs:1163-1176)."""
    with pytest.raises(TypeError, match="dtypes"):
        tracer.trace(lambda a, b: a + b, ("float32", (4,)), ("bfloat16", (4,)))
    with pytest.raises(TypeError, match="accum"):
        tracer.trace(lambda a: prims.reduce_sum(a, (0,), "float64"), ("float32", (4,)))
    with pytest.raises(TypeError, match="accum"):
        tracer.trace(lambda a, b: prims.dot_general(a, b, (((1,), (0,)), ((), ())), "bfloat16"), ("float32", (4, 4)), ("float32", (4, 4)))
    g = tracer.trace(lambda a: prims.reduce_sum(a, (0,), "float32"), ("bfloat16", (4,)))
    assert g.types[g.outputs[0]].dtype == "float32"
