"""Programs written with the composed functions of `lumen_b200.functional`, compiled and run on the GPU against the oracle
evaluating the same traced program: a SwiGLU MLP step differentiated by autograd, and the reductions / arg-reductions /
logical functions inside generated kernels."""

import numpy as np
import pytest

import lumen_b200
from lumen_b200 import autograd
from lumen_b200 import functional as F
from lumen_b200 import tracer
from lumen_b200.runtime import device_status
from tests.helpers import run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def oracle_of(fn, arrays):
    g = tracer.trace(fn, *[(str(a.dtype), a.shape) for a in arrays])
    return run_oracle(g, list(arrays))


def test_swiglu_mlp_step(cuda):
    """`down(silu(x gate) * (x up))` with a mean-square loss: value and the three weight gradients of the compiled step
    against the oracle (float32: 1e-5 on the loss, 2e-4 of the largest value on the gradients)."""

    def step(x, y, gate, up, down):
        def loss(g, u, d):
            h = F.swiglu(F.matmul(x, g, "float32", "float32"), F.matmul(x, u, "float32", "float32"))
            r = F.matmul(h, d, "float32", "float32") - y
            return F.mean(r * r)

        value, grads = autograd.value_and_grad(loss, (0, 1, 2))(gate, up, down)
        return (value, *grads)

    rng = np.random.default_rng(3)
    x, y = rng.standard_normal((256, 64)).astype(np.float32), rng.standard_normal((256, 32)).astype(np.float32)
    gate, up = ((0.2 * rng.standard_normal((64, 128))).astype(np.float32) for _ in range(2))
    down = (0.2 * rng.standard_normal((128, 32))).astype(np.float32)
    args = [x, y, gate, up, down]
    got = lumen_b200.compile(step)(*[to_torch(a, cuda) for a in args])
    device_status()
    want = oracle_of(step, args)
    assert abs(float(got[0]) - float(want[0])) <= 1e-5 * abs(float(want[0]))
    for g, w in zip(got[1:], want[1:]):
        assert np.abs(to_numpy(g) - w).max() <= 2e-4 * np.abs(w).max()


def test_reductions_and_logical_functions_in_generated_kernels(cuda):
    """amin / argmax / argmin / any / all / isnan / gelu / triu over rows of a matrix, compiled into generated kernels:
    integer and boolean results bit-exact, gelu within 1e-5."""

    def program(x):
        return (F.amin(x, 1), F.argmax(x, 1), F.argmin(x, 1), F.any(x > 2.5, 1), F.all(F.isfinite(x), 1), F.isnan(x), F.gelu(x),
                F.triu(x, 1))  # fmt: skip

    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 96)).astype(np.float32)
    x[3, 7] = np.nan
    x[5, 9] = x[5, 40] = 9.0  # a tie: the first index wins
    got = lumen_b200.compile(program)(to_torch(x, cuda))
    device_status()
    want = oracle_of(program, [x])
    for k, (g, w) in enumerate(zip(got, want)):
        g = to_numpy(g)
        if k == 6:
            np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-6, equal_nan=True)
        else:
            np.testing.assert_array_equal(g, w, err_msg=f"output {k}")
