"""Plans made by `lb_compile` (the backend's C++ lowering) run on the GPU and give, bit for bit, what the plans of the
optimising Python lowering give for the same module - the two differ in placement, not in kernels - and what the
oracle gives within the kernels' tolerances."""

import numpy as np
import pytest
import torch

from lumen_b200 import autograd, tracer
from lumen_b200 import functional as F
from lumen_b200.attention_pass import match_attention
from lumen_b200.compiler import compile_graph
from lumen_b200.fusion_pass import fuse
from lumen_b200.plan import Plan
from lumen_b200.runtime import TORCH_DTYPES, device_status
from lumen_b200.simplify import clean
from tests.helpers import bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def run_both(fn, arrays, cuda, **native_options):
    g = tracer.trace(fn, *[("bfloat16" if a.dtype.itemsize == 2 else str(a.dtype), a.shape) for a in arrays])
    fused = fuse(match_attention(clean(g)))
    inputs = [to_torch(a, cuda) for a in arrays]
    results = []
    for plan in (Plan.native(fused, **native_options), Plan(compile_graph(g), cuda)):
        outs = [torch.full(g.types[v].shape, float("nan"), dtype=TORCH_DTYPES[g.types[v].dtype], device=cuda) for v in g.outputs]
        plan.run(inputs, outs)
        device_status()
        results.append([to_numpy(o) for o in outs])
    return g, results


def test_fused_chain(cuda):
    def chain(x, g, b):
        y = F.relu(x * g + b)
        return y, F.sum(y * y, 1)

    rng = np.random.default_rng(1)
    arrays = [rng.standard_normal((512, 1024)).astype(np.float32), rng.uniform(0.5, 1.5, 1024).astype(np.float32),
              (0.1 * rng.standard_normal(1024)).astype(np.float32)]  # fmt: skip
    g, (native, python) = run_both(chain, arrays, cuda)
    want = run_oracle(g, arrays)
    np.testing.assert_array_equal(native[0], want[0])
    np.testing.assert_allclose(native[1], want[1], rtol=1e-5)
    for a, b in zip(native, python):
        assert a.tobytes() == b.tobytes()


def test_mlp_products_and_relu(cuda):
    def mlp(x, w1, w2):
        return F.matmul(F.relu(F.matmul(x, w1, "float32", "bfloat16")), w2, "float32", "bfloat16")

    rng = np.random.default_rng(2)
    arrays = [bf16(rng.standard_normal((512, 256))), bf16(rng.standard_normal((256, 1024)) / 16), bf16(rng.standard_normal((1024, 128)) / 32)]
    g, (native, python) = run_both(mlp, arrays, cuda)
    want = run_oracle(g, arrays)[0].astype(np.float32)
    np.testing.assert_allclose(native[0].astype(np.float32), want, rtol=2e-2, atol=2e-2 * np.abs(want).max())
    assert native[0].tobytes() == python[0].tobytes()


@pytest.mark.parametrize("deterministic", [True, False])
def test_attention_step(cuda, deterministic):
    def program(q, k, v, do):
        def loss(q_, k_, v_):
            return F.sum(F.flash_attention(q_, k_, v_, causal=True)[0].float() * do.float())

        value, grads = autograd.value_and_grad(loss, (0, 1, 2))(q, k, v)
        return (value, *grads)

    rng = np.random.default_rng(3)
    arrays = [bf16(rng.standard_normal((2, 256, 4, 64))) for _ in range(4)]
    g, (native, python) = run_both(program, arrays, cuda, deterministic=deterministic)
    want = run_oracle(g, arrays)
    assert abs(float(native[0]) - float(want[0])) <= 2e-2 * max(abs(float(want[0])), 1.0)
    for got, w, ref in zip(native[1:], want[1:], python[1:]):
        w = w.astype(np.float32)
        np.testing.assert_allclose(got.astype(np.float32), w, rtol=2e-2, atol=2e-2 * np.abs(w).max())
        if deterministic:
            assert got.tobytes() == ref.tobytes()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_training_step(cuda, dtype):
    """The transformer training step (forward, backward, SGD update) lowered by `lb_compile` and by the optimising
    lowering: the loss and every updated weight are bit-identical, and the loss is the oracle's."""
    from lumen_b200 import transformer as T
    from tests.helpers import BF16
    from tests.test_train_step import batch_of

    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=1, seq=128, dtype=dtype)
    g, names, _ = T.trace_train_step(cfg, 2)
    params = T.init_params(cfg, 0)
    ids, targets = batch_of(cfg, 2)
    cast = (lambda a: a.astype(BF16)) if dtype == "bfloat16" else (lambda a: a)
    arrays = [ids, targets] + [cast(params[n]) for n in names]
    inputs = [to_torch(a, cuda) for a in arrays]
    fused = fuse(match_attention(clean(g)))
    results = []
    for plan in (Plan.native(fused), Plan(compile_graph(g), cuda)):
        outs = [torch.full(g.types[v].shape, float("nan"), dtype=TORCH_DTYPES[g.types[v].dtype], device=cuda) for v in g.outputs]
        plan.run(inputs, outs)
        device_status()
        results.append([to_numpy(o) for o in outs])
    for name, a, b in zip(["loss", *names], *results):
        assert a.tobytes() == b.tobytes(), name
    want = run_oracle(g, arrays)
    assert abs(float(results[0][0]) - float(want[0])) <= (1e-5 if dtype == "float32" else 2e-2) * abs(float(want[0]))


def test_train_step_runner_on_the_native_lowering(cuda):
    """`TrainStep(lowering="native")`: the runner over a plan made by `lb_compile` with the weights donated - five steps
    (the later ones replayed from the recorded CUDA graph) give the losses and weights of the default runner, bit for bit."""
    from lumen_b200 import transformer as T
    from tests.test_train_step import batch_of

    cfg = T.Config(vocab=128, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16", lr=5e-2)
    ids, targets = batch_of(cfg, 4)
    results = []
    for lowering in ("optimising", "native"):
        step = T.TrainStep(cfg, 4, T.init_params(cfg, 0), cuda, lowering=lowering)
        step.load_batch(ids, targets)
        losses = [float(step.step().item()) for _ in range(5)]
        device_status()
        results.append((losses, step.state_dict()))
    assert results[0][0] == results[1][0] and results[0][0][-1] < results[0][0][0]
    for name in results[0][1]:
        assert results[0][1][name].tobytes() == results[1][1][name].tobytes(), name


def test_concatenation_by_copies(cuda):
    """Two products concatenated along the last axis: the C++ lowering copies each into its columns of the result."""
    def program(x, a, b):
        return F.cat([F.matmul(x, a, "float32", "bfloat16"), F.matmul(x, b, "float32", "bfloat16")], 1)

    rng = np.random.default_rng(4)
    arrays = [bf16(rng.standard_normal((256, 128))), bf16(rng.standard_normal((128, 64)) / 8), bf16(rng.standard_normal((128, 192)) / 8)]
    g = tracer.trace(program, *[("bfloat16", a.shape) for a in arrays])
    out = torch.full((256, 256), float("nan"), dtype=torch.bfloat16, device=cuda)
    Plan.native(fuse(clean(g))).run([to_torch(a, cuda) for a in arrays], [out])
    device_status()
    want = run_oracle(g, arrays)[0].astype(np.float32)
    np.testing.assert_allclose(to_numpy(out).astype(np.float32), want, rtol=2e-2, atol=2e-2 * np.abs(want).max())
