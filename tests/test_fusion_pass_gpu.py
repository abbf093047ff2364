"""Programs traced as bare prims, grouped by the fusion pass, lowered to a plan and run on a B200 against the oracle
evaluating the unfused graph."""

import numpy as np
import pytest
import torch

from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from lumen_b200.compiler import compile_graph
from lumen_b200.plan import Plan
from lumen_b200.runtime import TORCH_DTYPES, device_status
from tests.helpers import bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def run_plan(g, inputs, cuda):
    compiled = compile_graph(g)
    outs = [torch.empty(g.types[v].shape, dtype=TORCH_DTYPES[g.types[v].dtype], device=cuda) for v in g.outputs]
    Plan(compiled, cuda).run([to_torch(x, cuda) for x in inputs], outs)
    device_status()
    return compiled, [to_numpy(o) for o in outs]


def test_softmax_program_from_bare_prims(cuda):
    def program(x, w):
        p = F.softmax(x, -1)
        return p, F.sum(p * w, -1) * 0.5

    g = tracer.trace(program, ("float32", (512, 1024)), ("float32", (512, 1024)))
    rng = np.random.default_rng(0)
    inputs = [rng.standard_normal((512, 1024), dtype=np.float32), rng.standard_normal((512, 1024), dtype=np.float32)]
    compiled, got = run_plan(g, inputs, cuda)
    assert len(compiled.labels) <= 2
    want = run_oracle(g, inputs)
    np.testing.assert_allclose(got[0], want[0], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(got[1], want[1], rtol=1e-5, atol=1e-6)


def test_mlp_block_from_bare_prims_uses_gemm_epilogues(cuda):
    dims = (((1,), (0,)), ((), ()))

    def program(x, w1, w2, r):
        h = F.relu(prims.dot_general(x, w1, dims, "float32", "bfloat16"))
        return prims.dot_general(h, w2, dims, "float32", "bfloat16") + r

    g = tracer.trace(program, ("bfloat16", (384, 256)), ("bfloat16", (256, 512)), ("bfloat16", (512, 256)), ("bfloat16", (384, 256)))
    rng = np.random.default_rng(1)
    inputs = [bf16(rng.standard_normal((384, 256)) / 16), bf16(rng.standard_normal((256, 512)) / 16),
              bf16(rng.standard_normal((512, 256)) / 16), bf16(rng.standard_normal((384, 256)))]
    compiled, got = run_plan(g, inputs, cuda)
    assert compiled.labels == ["dot_general_relu", "dot_general_add"]
    want = run_oracle(g, inputs)[0].astype(np.float32)
    np.testing.assert_allclose(got[0].astype(np.float32), want, rtol=2**-6, atol=2**-6 * np.abs(want).max())


def test_compile_surface_runs_a_traced_function(cuda, tmp_path):
    """`lumen_b200.compile(fn, device="cuda")`: traced on the first call per signature, results owned by the compiled
    function and overwritten by the next call, a second signature compiles its own plan."""
    import lumen_b200

    def fn(x, w, scale):
        return F.relu(x * w) * scale, F.sum(x, -1)

    f = lumen_b200.compile(fn, device="cuda", use_graphs=True)
    rng = np.random.default_rng(5)
    x = torch.from_numpy(rng.standard_normal((256, 512), dtype=np.float32)).to(cuda)
    w = torch.from_numpy(rng.standard_normal((256, 512), dtype=np.float32)).to(cuda)
    for _ in range(3):  # plain run, recording, replay
        y, s = f(x, w, 0.5)
        device_status()
        torch.testing.assert_close(y, torch.relu(x * w) * 0.5, rtol=1e-6, atol=0)
        torch.testing.assert_close(s, x.sum(-1), rtol=1e-5, atol=1e-5)
    assert "reduce_sum" in str(f) and len(f.steps()) <= 2
    first = y
    y2, _ = f(x * 2, w, 0.5)
    assert y2.data_ptr() == first.data_ptr()  # the compiled function owns its results
    small, _ = f(x[:64], w[:64], 0.5)
    assert small.shape == (64, 512) and len(f.signatures) == 2
    written = f.dump_code(str(tmp_path))
    kernels = [p for p in written if p.endswith(".cu")]
    assert len(kernels) == len(f.steps()) and all("fused_kernel" in open(p).read() for p in kernels)


def test_compiled_function_with_attention_and_projection(cuda):
    """`F.flash_attention` inside a compiled function: the q/k/v projection GEMM, the attention fusion reading strided
    views of it in place, and an output projection with a residual add in its epilogue."""
    import lumen_b200

    b, s, n, h = 2, 256, 2, 64
    d = n * h
    dims = (((1,), (0,)), ((), ()))

    def block(x, wqkv, wo):
        qkv = prims.dot_general(x, wqkv, dims, "float32", "bfloat16")
        q, k, v = (prims.slice(qkv, (0, i * d), (b * s, (i + 1) * d)).reshape(b, s, n, h) for i in range(3))
        o, _ = F.flash_attention(q, k, v, causal=True)
        return prims.dot_general(o.reshape(b * s, d), wo, dims, "float32", "bfloat16") + x

    rng = np.random.default_rng(7)
    x, wqkv, wo = (bf16(rng.standard_normal(shape) / np.sqrt(shape[0] if len(shape) > 1 else 1))
                   for shape in ((b * s, d), (d, 3 * d), (d, d)))
    f = lumen_b200.compile(block)
    got = f(to_torch(x, cuda), to_torch(wqkv, cuda), to_torch(wo, cuda))
    device_status()
    assert [st["label"] for st in f.steps()] == ["dot_general", "flash_attention", "dot_general_add"]
    g = tracer.trace(block, ("bfloat16", x.shape), ("bfloat16", wqkv.shape), ("bfloat16", wo.shape))
    want = run_oracle(g, [x, wqkv, wo])[0].astype(np.float32)
    np.testing.assert_allclose(to_numpy(got).astype(np.float32), want, rtol=2e-2, atol=2e-2 * np.abs(want).max())


def test_normalisations_and_the_adamw_step_beside_the_training_path(cuda):
    """`rms_norm`, `log_softmax`, a clamp chain and the AdamW step (tests/test_front_ops.py pins them to float64 on the
    oracle) through the fusion pass and the generated kernels: one kernel each, rtol 1e-5 against the oracle
    (elementwise values of the AdamW step bit-exact: one rounding per primitive, no reduction)."""
    from tests.test_front_ops import adamw_graph, adamw_inputs, clamp_program, log_softmax_program, rms_program

    rng = np.random.default_rng(9)
    x = (2 * rng.standard_normal((300, 1000))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 1000).astype(np.float32)
    for program, inputs in ((rms_program, [x, w]), (log_softmax_program, [x]), (clamp_program, [x])):
        g = tracer.trace(program, *[("float32", a.shape) for a in inputs])
        compiled, got = run_plan(g, inputs, cuda)
        assert len(compiled.labels) == 1, (program.__name__, compiled.labels)
        np.testing.assert_allclose(got[0], run_oracle(g, inputs)[0], rtol=1e-5, atol=1e-6)
    for dtype in ("float32", "bfloat16"):
        g = adamw_graph(dtype, (129, 520), 7, lr=1e-2, weight_decay=0.1)
        inputs = adamw_inputs(dtype, (129, 520), seed=3)
        compiled, got = run_plan(g, inputs, cuda)
        assert compiled.labels == ["adamw_update"]
        want = run_oracle(g, inputs)
        for a, b in zip(got, want):
            # division and square root are correctly rounded on both sides
            np.testing.assert_array_equal(a.astype(np.float32), b.astype(np.float32))


def test_compile_takes_dlpack_arrays_in_place(cuda):
    """Arguments that are not torch tensors but export DLPack are imported without a copy (same device pointer)."""
    import lumen_b200

    class Foreign:  # stands for another framework's array
        def __init__(self, t):
            self.t = t

        def __dlpack__(self, **kw):
            return self.t.__dlpack__(**kw)

        def __dlpack_device__(self):
            return self.t.__dlpack_device__()

    f = lumen_b200.compile(lambda x, y: F.relu(x - y), device="cuda")
    x = torch.randn((64, 128), device=cuda)
    y = torch.randn((64, 128), device=cuda)
    got = f(Foreign(x), Foreign(y))
    torch.testing.assert_close(got, torch.relu(x - y), rtol=0, atol=0)
    assert f.latest.keep[0][0].data_ptr() == x.data_ptr()
