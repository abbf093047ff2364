"""`lumen_b200.autograd` on the oracle: vector-Jacobian products traced as strict prims, against float64 finite
differences for the single rules and against an independent PyTorch float64 model for a whole transformer step
written in plain functional ops (lumen/autograd/transforms.py:206-275, lumen/autograd/rules.py)."""

import numpy as np
import pytest

from lumen_b200 import autograd
from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from lumen_b200 import transformer as T
from oracle import oracle
from tests.helpers import bf16
from tests.model_reference import torch_step
from tests.test_train_step import batch_of


def run(fn, *arrays):
    names = {v: k for k, v in oracle.NUMPY.items()}
    g = tracer.trace(fn, *[(names[np.dtype(a.dtype)], a.shape) for a in arrays])
    return g, oracle.run(g, arrays)


def numeric_grad(f, arrays, k, eps=1e-6):
    """Central differences of the float64 scalar function `f` with respect to `arrays[k]`."""
    base = [a.astype(np.float64) for a in arrays]
    out = np.zeros_like(base[k])
    for i in np.ndindex(base[k].shape):
        hi, lo = [a.copy() for a in base], [a.copy() for a in base]
        hi[k][i] += eps
        lo[k][i] -= eps
        out[i] = (f(*hi) - f(*lo)) / (2 * eps)
    return out


RULES = [
    # traced function of float64 tensors returning a scalar, the same in NumPy, input shapes
    (lambda a, b: F.sum(a * b / (b * b + 1.5) - a), lambda a, b: (a * b / (b * b + 1.5) - a).sum(), [(3, 4), (3, 4)]),
    (lambda a, b: F.sum(F.exp(a) * F.tanh(b) + F.sqrt(a * a + 1.0) * F.rsqrt(b * b + 2.0)),
     lambda a, b: (np.exp(a) * np.tanh(b) + np.sqrt(a * a + 1) / np.sqrt(b * b + 2)).sum(), [(2, 5), (2, 5)]),
    (lambda a, b: F.sum(F.maximum(a, b) * a + F.relu(b)), lambda a, b: (np.maximum(a, b) * a + np.maximum(b, 0)).sum(), [(4, 3), (4, 3)]),
    (lambda a, b: F.sum(F.amax(a, -1) * F.sum(b, 0)), lambda a, b: (a.max(-1) * b.sum(0)).sum(), [(4, 5), (3, 4)]),
    (lambda a, b: F.sum(F.softmax(a, -1) * b), lambda a, b: (np.exp(a - a.max(-1, keepdims=True)) / np.exp(a - a.max(-1, keepdims=True)).sum(-1, keepdims=True) * b).sum(), [(3, 6), (3, 6)]),
    (lambda a, b: F.sum(F.matmul(a, b.t(), "float64", "float64") * F.matmul(a, b.t(), "float64", "float64")),
     lambda a, b: ((a @ b.T) ** 2).sum(), [(4, 6), (5, 6)]),
    (lambda a, b: F.sum(F.log(F.sigmoid(a) + 0.1) * b.reshape(6, 2).permute(1, 0).reshape(3, 4)),
     lambda a, b: (np.log(1 / (1 + np.exp(-a)) + 0.1) * b.reshape(6, 2).T.reshape(3, 4)).sum(), [(3, 4), (3, 4)]),
    (lambda a, b: F.sum(prims.concatenate([prims.slice(a, (0, 1), (3, 3)), b], 1) * prims.concatenate([b, prims.slice(a, (0, 0), (3, 2))], 1)),
     lambda a, b: (np.concatenate([a[:, 1:3], b], 1) * np.concatenate([b, a[:, 0:2]], 1)).sum(), [(3, 4), (3, 2)]),
    (lambda a, b: F.sum(F.where(F.gt(a, 0.0), a * b, b - a)), lambda a, b: np.where(a > 0, a * b, b - a).sum(), [(3, 4), (3, 4)]),
]


@pytest.mark.parametrize("case", range(len(RULES)))
def test_rules_match_finite_differences(case):
    traced, plain, shapes = RULES[case]
    rng = np.random.default_rng(case)
    arrays = [rng.standard_normal(s) for s in shapes]

    def program(*xs):
        value, grads = autograd.value_and_grad(traced, argnums=tuple(range(len(xs))))(*xs)
        return (value, *grads)

    _, outs = run(program, *arrays)
    assert outs[0] == pytest.approx(plain(*arrays), rel=1e-12)
    for k in range(len(arrays)):
        np.testing.assert_allclose(outs[1 + k], numeric_grad(plain, arrays, k), rtol=1e-6, atol=1e-7)


def test_ties_share_the_gradient():
    """`max` splits a tie evenly and `reduce_max` averages over the positions equal to the maximum (rules.py:398-421)."""
    a = np.array([[1.0, 3.0, 3.0], [2.0, 2.0, 2.0]])
    b = np.array([[1.0, 0.0, 4.0], [2.0, 5.0, 1.0]])
    _, (gm,) = run(lambda x, y: autograd.grad(lambda u, v: F.sum(F.maximum(u, v)))(x, y), a, b)
    np.testing.assert_array_equal(gm, [[0.5, 1.0, 0.0], [0.5, 0.0, 1.0]])
    _, (gr,) = run(lambda x: autograd.grad(lambda u: F.sum(F.amax(u, -1)))(x), a)
    np.testing.assert_allclose(gr, [[0.0, 0.5, 0.5], [1 / 3, 1 / 3, 1 / 3]])


def test_weight_gradient_of_a_narrowed_weight_keeps_the_accumulator():
    """`x @ w.bfloat16()` with float32 `w`: the gradient of `w` is the float32 accumulator of its product, not that
    value rounded to bfloat16 and widened again; the gradient of the bfloat16 `x` is rounded once to bfloat16
    (rules.py:28-60,425-489)."""
    rng = np.random.default_rng(0)
    x, w, g = bf16(rng.standard_normal((8, 16))), rng.standard_normal((16, 4)).astype(np.float32), bf16(rng.standard_normal((8, 4)))

    def program(x_, w_, g_):
        out, pull = autograd.vjp(lambda a, b: F.matmul(a, b.bfloat16(), "float32", "bfloat16"), x_, w_)
        return pull(g_)

    graph, (dx, dw) = run(program, x, w, g)
    assert dx.dtype == x.dtype and dw.dtype == np.float32
    want = x.astype(np.float32).T @ g.astype(np.float32)
    np.testing.assert_allclose(dw, want, rtol=1e-6)
    assert not np.array_equal(dw, bf16(dw).astype(np.float32))  # not a bfloat16 value widened
    dots = [n for n in graph.nodes if n.op == "dot_general"]
    assert len(dots) == 3 and all(n.params["accum_dtype"] == "float32" for n in dots)


def transformer_loss(cfg, batch):
    """The baseline transformer written in plain functional ops (no hand-derived backward anywhere)."""
    d, h = cfg.d_model, cfg.heads

    def loss(ids, targets, *weights):
        w = dict(zip([n for n, _ in T.param_shapes(cfg)], weights))
        x = (w["embed.tokens"][ids] + w["embed.positions"]).reshape(batch * cfg.seq, d)
        for layer in range(cfg.layers):
            p = f"layers.{layer}."
            hh = F.layer_norm(x, w[p + "attn.norm.w"], w[p + "attn.norm.b"])
            qkv = F.matmul(hh, w[p + "attn.wqkv"].t(), "float32", "float32")
            q, k, v = (prims.slice(qkv, (0, i * d), (batch * cfg.seq, (i + 1) * d)).reshape(batch, cfg.seq, h, d // h) for i in range(3))
            o, _ = F.flash_attention(q, k, v, causal=True)
            x = x + F.matmul(o.reshape(batch * cfg.seq, d), w[p + "attn.wo"].t(), "float32", "float32")
            hh = F.layer_norm(x, w[p + "mlp.norm.w"], w[p + "mlp.norm.b"])
            x = x + F.matmul(F.relu(F.matmul(hh, w[p + "mlp.w1"].t(), "float32", "float32")), w[p + "mlp.w2"].t(), "float32", "float32")
        x = F.layer_norm(x, w["norm.w"], w["norm.b"])
        logits = F.matmul(x, w["head"].t(), "float32", "float32")
        return F.mean(F.cross_entropy(logits, targets.reshape(batch * cfg.seq)))

    return loss


def test_a_whole_transformer_step_differentiates_like_pytorch():
    """Forward + `value_and_grad` of a 2-layer float32 transformer (gather, layer norm, packed qkv slices,
    `F.flash_attention`, ReLU MLP, cross entropy), evaluated by the oracle, against PyTorch autograd in float64."""
    cfg = T.Config(vocab=48, d_model=32, heads=2, hidden=64, layers=2, seq=16)
    batch = 2
    params = T.init_params(cfg, 0)
    names = [n for n, _ in T.param_shapes(cfg)]
    ids, targets = batch_of(cfg, batch)
    argnums = tuple(range(2, 2 + len(names)))

    def program(ids_, targets_, *weights):
        value, grads = autograd.value_and_grad(transformer_loss(cfg, batch), argnums)(ids_, targets_, *weights)
        return (value, *grads)

    graph, outs = run(program, ids, targets, *[params[n] for n in names])
    want_loss, want = torch_step(cfg, {k: v.astype(np.float64) for k, v in params.items()}, ids, targets)
    assert float(outs[0]) == pytest.approx(want_loss, rel=1e-5)
    for name, got in zip(names, outs[1:]):
        scale = max(np.abs(want[name]).max(), 1e-8)
        assert np.abs(got - want[name]).max() <= 2e-4 * scale, name
    fusions = [n.params["name"] for n in graph.nodes if n.op == "fusion"]
    assert fusions.count("flash_attention") == cfg.layers and fusions.count("flash_attention_backward") == cfg.layers


def test_gated_mlp_of_the_reference_example_differentiates():
    """`(sigmoid(x wg^T) * (x wu^T)) wd^T` - the gated MLP of the reference's example model (examples/transformer.py:
    36-86), written forward-only and differentiated by autograd: against central differences in float64."""
    def mlp(x, wg, wu, wd):
        g = F.matmul(x, wg.t(), "float64", "float64")
        u = F.matmul(x, wu.t(), "float64", "float64")
        return F.sum(F.matmul(F.sigmoid(g) * u, wd.t(), "float64", "float64") * 0.25)

    def plain(x, wg, wu, wd):
        return ((1 / (1 + np.exp(-(x @ wg.T))) * (x @ wu.T)) @ wd.T).sum() * 0.25

    rng = np.random.default_rng(5)
    arrays = [rng.standard_normal(s) for s in ((4, 6), (8, 6), (8, 6), (6, 8))]
    _, outs = run(lambda *xs: autograd.grad(mlp, argnums=(0, 1, 2, 3))(*xs), *arrays)
    for k in range(4):
        np.testing.assert_allclose(outs[k], numeric_grad(plain, arrays, k), rtol=1e-6, atol=1e-8)
