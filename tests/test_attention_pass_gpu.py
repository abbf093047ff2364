"""Attention written in bare prims (softmax and two matmuls; the traced FlashAttention-2 backward), recognised by the
attention passes and run on the tcgen05 kernels, against the oracle evaluating the program as written."""

import numpy as np
import pytest
import torch

from lumen_b200.compiler import compile_graph
from lumen_b200.plan import Plan
from lumen_b200.runtime import TORCH_DTYPES, device_status
from lumen_b200 import tracer
from tests.helpers import run_oracle, to_numpy, to_torch
from tests.test_attention_pass import FULL, GROUPED, forward_and_backward, heads_first_output, inputs_for, softmax_and_two_matmuls

pytestmark = pytest.mark.gpu


def close(got, want, tol=2e-2):
    want = want.astype(np.float64)
    np.testing.assert_allclose(got.astype(np.float64), want, rtol=tol, atol=tol * max(np.abs(want).max(), 1e-6))


@pytest.mark.parametrize("fn,specs,steps", [
    (softmax_and_two_matmuls, [FULL] * 3, ["attn_fwd"]),
    (heads_first_output, [FULL] * 3, ["attn_fwd"]),
    (forward_and_backward, [FULL, GROUPED, GROUPED, FULL], ["attn_fwd", "attn_bwd"]),
])
def test_programs_in_bare_prims_run_on_the_attention_kernels(cuda, fn, specs, steps):
    g = tracer.trace(fn, *specs)
    args = inputs_for(specs, seed=3)
    compiled = compile_graph(g)
    assert [line.split()[1] for line in compiled.text.splitlines() if line.startswith("s ")] == steps
    outs = [torch.full(g.types[v].shape, float("nan"), dtype=TORCH_DTYPES[g.types[v].dtype], device=cuda) for v in g.outputs]
    Plan(compiled, cuda).run([to_torch(a, cuda) for a in args], outs)
    device_status()
    want = run_oracle(g, args)
    for got, w in zip(outs, want):
        close(to_numpy(got).astype(np.float32), w.astype(np.float32))
