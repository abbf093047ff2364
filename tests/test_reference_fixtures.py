"""Pins the CPU oracle to outputs of the reference's OWN NumPy model of this path.

tests/golden/reference_*.npz were produced by tests/golden/make_reference_fixtures.py, which lifts `_bf16`,
`_rms_norm`, `_matmul`, `_attention`, `_logits` (tests/test_transformer_example.py:211-264) and `reference()`
(tests/functional/test_attention.py:17-31) out of the reference's test files and runs them. Here the same programs,
written with this package's tracer and functional ops, are evaluated by the oracle and compared with those outputs at
the reference's own tolerances (test_transformer_example.py:286-292, test_attention.py TOL); the bfloat16 rounding
bit for bit.
"""

import importlib.util
import os

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from oracle import oracle
from tests.helpers import BF16, bf16

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def run1(f, *arrays):
    names = {v: k for k, v in oracle.NUMPY.items()}
    g = tracer.trace(f, *[(names[np.dtype(a.dtype)], a.shape) for a in arrays])
    return oracle.run(g, arrays)


def test_bf16_rounding_is_the_references_bit_for_bit():
    fx = load("reference_bf16.npz")
    (got,) = run1(lambda x: prims.cast(x, "bfloat16"), fx["x"])
    np.testing.assert_array_equal(got.astype(np.float32).view(np.uint32), fx["y"].view(np.uint32))


def test_rms_norm_matches_the_references():
    """`F.rms_norm` in float32 with the default epsilon 2^-23 against `_rms_norm`."""
    fx = load("reference_rms_norm.npz")
    (got,) = run1(lambda x, w: F.rms_norm(x, w), fx["x"], fx["w"])
    np.testing.assert_allclose(got, fx["y"], rtol=2e-6, atol=1e-7)


def test_bf16_matmul_matches_the_references():
    """`F.matmul` of bfloat16 operands accumulated in float32 against `_matmul` (accumulated in float64): the
    float32 results agree to accumulation order, the bfloat16 results to one unit in the last place at most."""
    fx = load("reference_matmul.npz")
    x, w = bf16(fx["x"]), bf16(fx["w"])
    wide, narrow = run1(lambda a, b: (F.matmul(a, b.t(), "float32", "float32"), F.matmul(a, b.t(), "float32", "bfloat16")), x, w)
    scale = np.abs(fx["y_f32"]).max()
    assert np.abs(wide - fx["y_f32"]).max() <= 1e-5 * scale
    err = np.abs(narrow.astype(np.float32) - fx["y_bf16"])
    assert (err <= 2.0**-8 * np.abs(fx["y_bf16"]) + 1e-30).all()  # one bfloat16 ulp
    assert (err == 0).mean() > 0.97


def test_causal_attention_matches_the_references_bf16_model():
    """The traced `F.flash_attention` forward (probabilities rounded to bfloat16 before the value product) against
    `_attention`."""
    fx = load("reference_attention_bf16.npz")
    heads = int(fx["heads"])
    b, s, d = fx["q"].shape
    q, k, v = (bf16(fx[n]).reshape(b, s, heads, d // heads) for n in "qkv")
    (o, _lse) = run1(lambda a, bb, c: F.attention_forward_prims(a, bb, c, 1.0 / np.sqrt(d // heads), True), q, k, v)
    got = o.astype(np.float32).reshape(b * s, d)
    scale = np.abs(fx["o"]).max()
    assert np.abs(got - fx["o"]).max() <= 2.0**-7 * scale  # well inside the 2e-2 the reference allows devices
    assert (got == fx["o"]).mean() > 0.9


def _make_fixtures_module():
    spec = importlib.util.spec_from_file_location("make_reference_fixtures", os.path.join(GOLDEN, "make_reference_fixtures.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_matches_the_references_float64_on_its_cases(dtype):
    """`reference()` on the reference's CASES (GQA, causal with Sk != Sq, odd lengths, head dims 16..128, value head
    dim != key head dim), tolerance its TOL[dtype] scaled by the largest output as its tests do."""
    fx = load("reference_attention_f64.npz")
    draw = _make_fixtures_module().attention_case_inputs
    tol = float(fx["tol_" + dtype])
    for i, case in enumerate(fx["cases"]):
        *shape, causal = (int(x) for x in case)
        q, k, v = draw(i, shape)
        np.testing.assert_allclose([a.astype(np.float64).sum() for a in (q, k, v)], fx[f"sums{i}"], rtol=0, atol=0)
        want = fx[f"o{i}"] if dtype == "float32" else fx[f"ob{i}"]  # bfloat16: reference() of the rounded values
        if dtype == "bfloat16":
            q, k, v = bf16(q), bf16(k), bf16(v)
        h = shape[5]
        (o, _) = run1(lambda a, b, c: F.attention_forward_prims(a, b, c, 1.0 / np.sqrt(h), bool(causal)), q, k, v)
        got = o.astype(np.float64)
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= tol * max(np.abs(want).max(), 1.0), (i, np.abs(got - want).max())


def reference_model_logits(w, ids, cfg):
    """The reference's test transformer (tests/test_transformer_example.py:15-91: float32 weights and residual
    stream, RMSNorm, bfloat16 matmuls accumulated in float32, causal flash attention, ReLU MLP, float32 head) traced
    with this package's ops. `w` maps the names `_logits` reads to traced tensors."""
    vocab, seq, dim, heads, hidden, layers, batch = cfg
    tokens = batch * seq

    def matmul(x, weight, out="bfloat16"):
        return F.matmul(x.bfloat16(), weight.t().bfloat16(), "float32", out)

    x = (w["embed.tokens"][ids] + w["embed.positions"]).reshape(tokens, dim)
    for layer in range(layers):
        p = f"layers.{layer}."
        r = x
        n = F.rms_norm(x.float(), w[p + "attn.norm"]).bfloat16()
        q, k, v = (matmul(n, w[p + "attn.w" + c]).reshape(batch, seq, heads, dim // heads) for c in "qkv")
        o, _ = F.attention_forward_prims(q, k, v, 1.0 / np.sqrt(dim // heads), True)
        x = r.bfloat16() + matmul(o.reshape(tokens, dim), w[p + "attn.wo"])
        r = x
        n = F.rms_norm(x.float(), w[p + "mlp.norm"]).bfloat16()
        x = r + matmul(F.relu(matmul(n, w[p + "mlp.w1"])), w[p + "mlp.w2"])
    x = F.rms_norm(x.float(), w["norm"]).bfloat16()
    return matmul(x, w["head"], "float32")


def test_transformer_forward_matches_the_references_numpy_model():
    """The whole 2-layer forward against `_logits`, by the reference's own criterion
    (test_transformer_example.py:286-292): every logit within 2e-2 of the largest, and the same prediction wherever
    the two best logits are more than 4e-2 of the largest apart."""
    fx = load("reference_logits.npz")
    cfg = [int(x) for x in fx["config"]]
    names = sorted(k[2:] for k in fx.files if k.startswith("w."))
    arrays = [fx["ids"]] + [fx["w." + n] for n in names]

    def program(ids, *weights):
        return reference_model_logits(dict(zip(names, weights)), ids, cfg)

    (got,) = run1(program, *arrays)
    want = fx["logits"]
    assert got.shape == want.shape == (cfg[6] * cfg[1], cfg[0])
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-2 * scale, (np.abs(got - want).max(), scale)
    top = np.sort(want, -1)
    clear = top[:, -1] - top[:, -2] > 4e-2 * scale
    assert clear.sum() > 0
    np.testing.assert_array_equal(got.argmax(-1)[clear], want.argmax(-1)[clear])


_ = BF16
