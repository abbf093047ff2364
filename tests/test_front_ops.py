"""The torch-style functions beside the training path (`rms_norm`, `log_softmax`, `clamp`, ... and the AdamW step of
examples/optim.py) traced as prims: the oracle evaluating the traced graph against a float64 NumPy restatement
(as the reference's own tests check them, tests/graph_compiler/test_normalizations.py:103-147), and the fusion pass
turning each into kernels the backend accepts. CPU only; tests/test_fusion_pass_gpu.py runs the same programs on a GPU."""

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import graph as G
from lumen_b200 import nn, prims, tracer
from lumen_b200.fusion_pass import fuse
from lumen_b200.prims import TracedTensor
from tests.helpers import bf16, run_oracle


def rms_program(x, w):
    return F.rms_norm(x, w, 1e-6)


def log_softmax_program(x):
    return F.log_softmax(x, -1)


def clamp_program(x):
    return F.clamp(F.reciprocal(F.square(x) + 1.0), 0.2, 0.9)


def adamw_graph(dtype, shape, step, **kw):
    g = G.Graph()
    prims.push_graph(g)
    try:
        p = TracedTensor(g, g.add_input(dtype, shape))
        m = TracedTensor(g, g.add_input("float32", shape))
        v = TracedTensor(g, g.add_input("float32", shape))
        gr = TracedTensor(g, g.add_input(dtype, shape))
        outs = nn.adamw_update(p, m, v, gr, step, **kw)
    finally:
        prims.pop_graph()
    g.set_outputs([o.var for o in outs])
    return g


def adamw_inputs(dtype, shape, seed=0):
    rng = np.random.default_rng(seed)
    narrow = bf16 if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32))
    return [narrow(rng.standard_normal(shape)), (0.1 * rng.standard_normal(shape)).astype(np.float32),
            rng.uniform(0, 0.01, shape).astype(np.float32), narrow(0.1 * rng.standard_normal(shape))]


def test_rms_norm_matches_float64():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((16, 96)).astype(np.float32), rng.uniform(0.5, 1.5, 96).astype(np.float32)
    g = tracer.trace(rms_program, ("float32", x.shape), ("float32", w.shape))
    (y,) = run_oracle(g, [x, w])
    x64 = x.astype(np.float64)
    np.testing.assert_allclose(y, x64 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 1e-6) * w, rtol=1e-5, atol=1e-6)
    with pytest.raises(TypeError, match="weight"):
        tracer.trace(rms_program, ("float32", (4, 8)), ("float32", (4,)))


def test_rms_norm_in_bfloat16_rounds_once_before_the_weight():
    rng = np.random.default_rng(1)
    x, w = bf16(rng.standard_normal((8, 64))), bf16(rng.uniform(0.5, 1.5, 64))
    g = tracer.trace(lambda a, b: F.rms_norm(a, b), ("bfloat16", x.shape), ("bfloat16", w.shape))
    (y,) = run_oracle(g, [x, w])
    x64 = x.astype(np.float64)
    normed = bf16(x64 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 2.0**-7))  # default eps: bfloat16's epsilon
    want = bf16(normed.astype(np.float64) * w.astype(np.float64))
    assert np.mean(y.astype(np.float32) == want.astype(np.float32)) > 0.99  # float32 row statistics may move a rounding
    np.testing.assert_allclose(y.astype(np.float32), want.astype(np.float32), rtol=2**-7, atol=2**-8)


def test_log_softmax_and_clamp_match_float64():
    rng = np.random.default_rng(2)
    x = (3 * rng.standard_normal((12, 80))).astype(np.float32)
    (y,) = run_oracle(tracer.trace(log_softmax_program, ("float32", x.shape)), [x])
    s = x.astype(np.float64) - x.max(-1, keepdims=True)
    np.testing.assert_allclose(y, s - np.log(np.exp(s).sum(-1, keepdims=True)), rtol=1e-5, atol=1e-6)
    (z,) = run_oracle(tracer.trace(clamp_program, ("float32", x.shape)), [x])
    np.testing.assert_allclose(z, np.clip(1 / (x.astype(np.float64) ** 2 + 1), 0.2, 0.9), rtol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_adamw_step_matches_float64(dtype):
    shape, step = (32, 48), 3
    g = adamw_graph(dtype, shape, step, lr=1e-2, weight_decay=0.1)
    p, m, v, gr = adamw_inputs(dtype, shape)
    new_p, new_m, new_v = run_oracle(g, [p, m, v, gr])
    g64, b1, b2 = gr.astype(np.float64), 0.9, 0.999
    m64, v64 = b1 * m + (1 - b1) * g64, b2 * v + (1 - b2) * g64 * g64
    want = p.astype(np.float64) * (1 - 1e-2 * 0.1) - 1e-2 * (m64 / (1 - b1**step)) / (np.sqrt(v64 / (1 - b2**step)) + 1e-8)
    np.testing.assert_allclose(new_m, m64, rtol=1e-6, atol=1e-8)
    np.testing.assert_allclose(new_v, v64, rtol=1e-6, atol=1e-10)
    tol = 2**-8 if dtype == "bfloat16" else 1e-5
    np.testing.assert_allclose(new_p.astype(np.float64), want, rtol=tol, atol=tol * 1e-2)
    assert new_p.dtype == p.dtype and new_m.dtype == np.float32


def test_the_fusion_pass_makes_one_kernel_of_each():
    for program, specs in ((rms_program, [("float32", (64, 256)), ("float32", (256,))]),
                           (log_softmax_program, [("float32", (64, 256))]), (clamp_program, [("float32", (64, 256))])):
        fused_graph = fuse(tracer.trace(program, *specs))
        kernels = [n for n in fused_graph.nodes if n.op == "fusion"]
        assert len(kernels) == 1, (program.__name__, [n.op for n in fused_graph.nodes])
    body = [n for n in adamw_graph("bfloat16", (64, 256), 1).nodes if n.op == "fusion"]
    assert len(body) == 1 and len(body[0].params["body"].outputs) == 3
