"""A training step nobody derived by hand: a transformer written in plain functional ops, differentiated by
`lumen_b200.autograd`, cleaned, pattern-matched (attention forward and backward), fused, lowered to a plan and run on a
B200 - against the oracle evaluating the traced program primitive by primitive."""

import numpy as np
import pytest
import torch

import lumen_b200
from lumen_b200 import autograd, tracer
from lumen_b200 import transformer as T
from lumen_b200.compiler import compile_graph
from lumen_b200.plan import Plan
from lumen_b200.runtime import TORCH_DTYPES, device_status
from tests.helpers import run_oracle, to_numpy, to_torch
from tests.test_autograd import transformer_loss
from tests.test_train_step import batch_of

pytestmark = pytest.mark.gpu


def test_autograd_step_runs_on_the_gpu_and_matches_the_oracle(cuda):
    cfg = T.Config(vocab=512, d_model=128, heads=2, hidden=256, layers=2, seq=128)
    batch = 2
    names = [n for n, _ in T.param_shapes(cfg)]
    argnums = tuple(range(2, 2 + len(names)))

    def program(ids, targets, *weights):
        value, grads = autograd.value_and_grad(transformer_loss(cfg, batch), argnums)(ids, targets, *weights)
        return (value, *grads)

    g = tracer.trace(program, ("int64", (batch, cfg.seq)), ("int64", (batch, cfg.seq)), *[("float32", s) for _, s in T.param_shapes(cfg)])
    params = T.init_params(cfg, 0)
    ids, targets = batch_of(cfg, batch)
    args = [ids, targets] + [params[n] for n in names]
    compiled = compile_graph(g)
    kinds = [line.split()[1] for line in compiled.text.splitlines() if line.startswith("s ")]
    assert kinds.count("attn_fwd") == cfg.layers and kinds.count("attn_bwd") == cfg.layers and kinds.count("gemm") == 3 * (4 * cfg.layers + 1)
    outs = [torch.full(g.types[v].shape, float("nan"), dtype=TORCH_DTYPES[g.types[v].dtype], device=cuda) for v in g.outputs]
    Plan(compiled, cuda).run([to_torch(a, cuda) for a in args], outs)
    device_status()
    want = run_oracle(g, args)
    assert abs(float(outs[0]) - float(want[0])) <= 1e-5 * abs(float(want[0]))
    for name, got, w in zip(names, outs[1:], want[1:]):
        assert np.abs(to_numpy(got) - w).max() <= 2e-4 * max(np.abs(w).max(), 1e-12), name


def test_compile_differentiates_a_user_function(cuda):
    """`lumen_b200.compile` of a function that calls `autograd.grad` itself: a two-layer MLP regression step with its
    SGD update, against the same arithmetic in float64."""
    from lumen_b200 import functional as F

    def step(x, y, w1, w2):
        def loss(a, b):
            h = F.relu(F.matmul(x, a, "float32", "float32"))
            return F.mean((F.matmul(h, b, "float32", "float32") - y) * (F.matmul(h, b, "float32", "float32") - y))

        value, (g1, g2) = autograd.value_and_grad(loss, (0, 1))(w1, w2)
        return value, w1 - g1 * 0.1, w2 - g2 * 0.1

    rng = np.random.default_rng(0)
    x, y = rng.standard_normal((256, 64)).astype(np.float32), rng.standard_normal((256, 8)).astype(np.float32)
    w1, w2 = (0.1 * rng.standard_normal((64, 128))).astype(np.float32), (0.1 * rng.standard_normal((128, 8))).astype(np.float32)
    compiled = lumen_b200.compile(step)
    value, n1, n2 = compiled(*[to_torch(a, cuda) for a in (x, y, w1, w2)])
    device_status()
    x64, y64, a, b = (t.astype(np.float64) for t in (x, y, w1, w2))
    h = np.maximum(x64 @ a, 0)
    r = h @ b - y64
    gb = h.T @ (2 * r / r.size)
    ga = x64.T @ (((2 * r / r.size) @ b.T) * (h > 0))
    assert float(value) == pytest.approx((r * r).mean(), rel=1e-5)
    np.testing.assert_allclose(to_numpy(n1), a - 0.1 * ga, rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(to_numpy(n2), b - 0.1 * gb, rtol=1e-4, atol=1e-6)
