"""Empty and degenerate operands through the C ABI: a launch over zero elements is skipped (the reference skips a
zero-size grid, lumen/runtime/kernel/cuda/mod.rs:131-133), a product over an empty contraction is zero (the
interpreter's empty sum, lumen/reference/mod.rs:958-970), and nothing faults or reports an error."""

import numpy as np
import pytest
import torch

import lumen_b200
from lumen_b200 import functional as F
from lumen_b200 import tracer
from lumen_b200.runtime import attention_backward, attention_forward, device_status, gemm, scatter_add_rows
from tests.helpers import bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def test_fused_kernels_over_zero_rows(cuda):
    def chain(x, g, b):
        y = F.relu(x * g + b)
        return y, F.sum(y * y, 1)

    x = np.zeros((0, 256), np.float32)
    g, b = np.ones(256, np.float32), np.zeros(256, np.float32)
    y, s = lumen_b200.compile(chain)(to_torch(x, cuda), to_torch(g, cuda), to_torch(b, cuda))
    device_status()
    assert tuple(y.shape) == (0, 256) and tuple(s.shape) == (0,)
    want = run_oracle(tracer.trace(chain, ("float32", (0, 256)), ("float32", (256,)), ("float32", (256,))), [x, g, b])
    assert want[0].shape == (0, 256) and want[1].shape == (0,)


@pytest.mark.parametrize("shape", [(0, 128, 64), (128, 0, 64), (128, 256, 0)])
def test_gemm_with_an_empty_dimension(cuda, shape):
    m, n, k = shape
    a, b = torch.ones((m, k), dtype=torch.bfloat16, device=cuda), torch.ones((k, n), dtype=torch.bfloat16, device=cuda)
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=cuda)
    gemm(a, b, out)
    device_status()
    if k == 0:  # an empty sum
        assert bool((out == 0).all())
        want = run_oracle(tracer.trace(lambda x, y: F.matmul(x, y, "float32", "float32"), ("bfloat16", (m, k)), ("bfloat16", (k, n))),
                          [bf16(np.ones((m, k))), bf16(np.ones((k, n)))])[0]  # fmt: skip
        np.testing.assert_array_equal(to_numpy(out), want)


def test_attention_with_an_empty_batch(cuda):
    q = torch.zeros((0, 128, 2, 64), dtype=torch.bfloat16, device=cuda)
    o, lse = attention_forward(q, q, q, causal=True)
    grads = attention_backward(q, q, q, o, q, lse, causal=True)
    device_status()
    assert tuple(o.shape) == (0, 128, 2, 64) and all(tuple(g.shape) == (0, 128, 2, 64) for g in grads)


@pytest.mark.parametrize("deterministic", [True, False])
def test_scatter_add_without_updates(cuda, deterministic):
    table = to_torch(bf16(np.random.default_rng(0).standard_normal((32, 64))), cuda)
    ids = torch.zeros((0,), dtype=torch.int64, device=cuda)
    updates = torch.zeros((0, 64), dtype=torch.bfloat16, device=cuda)
    out = scatter_add_rows(table, ids, updates, deterministic=deterministic)
    device_status()
    assert torch.equal(out, table)


def test_more_than_two_to_the_31_elements(cuda):
    """A matrix of 65,600 x 32,768 bfloat16 logits (2.15e9 elements: element offsets no longer fit 32 bits) through an
    elementwise kernel and a row kernel: rows from the start, the middle and beyond the 2^31-th element equal the oracle
    on those rows (the elementwise result bit for bit, the log-sum-exp and the loss within 1e-5)."""
    rows, cols = 65_600, 32_768
    assert rows * cols > 2**31
    gen = torch.Generator(device=cuda).manual_seed(7)
    x = torch.empty((rows, cols), dtype=torch.bfloat16, device=cuda)
    for r0 in range(0, rows, 8200):  # filled piecewise: the float32 draw of the whole matrix would take 8.6 GB
        x[r0 : r0 + 8200] = torch.randn((min(8200, rows - r0), cols), generator=gen, device=cuda).bfloat16()
    targets = torch.randint(0, cols, (rows,), generator=gen, device=cuda)

    def program(a, t):
        loss, lse = F.cross_entropy_forward_prims(a.float(), t)
        return a * 0.5, loss, lse

    half, loss, lse = lumen_b200.compile(program)(x, targets)
    device_status()
    sample = [0, 1, 32_767, 65_535, 65_536, 65_599]  # row 65,536 starts at element 2^31
    xs, ts = to_numpy(x[sample]), to_numpy(targets[sample])
    want = run_oracle(tracer.trace(program, ("bfloat16", xs.shape), ("int64", ts.shape)), [xs, ts])
    np.testing.assert_array_equal(to_numpy(half[sample]).view(np.uint16), want[0].view(np.uint16))
    np.testing.assert_allclose(to_numpy(loss[sample]), want[1], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(to_numpy(lse[sample]), want[2], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("shape", [(1048576,), (300007,), (3, 300007), (300007, 3), (2, 524288), (1000003,), (4096, 1536)])
def test_long_flat_tensors(cuda, shape):
    """Tensors whose last dimension (or whole extent, for the reductions over everything) is longer than the 262,144
    elements one block takes as a row, with lengths that are powers of two, have small divisors only, or are prime:
    element-wise results bit for bit, the whole-tensor sum of squares within 1e-6 of itself (the oracle adds a million
    terms one after the other in float32 - the split reduction is the more accurate of the two, so it is held against
    the float64 sum), the maximum exactly."""
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)

    def program(a):
        return a * a + 1.0, F.sum(a * a), F.amax(a), F.mean(a)

    got = lumen_b200.compile(program)(to_torch(x, cuda))
    device_status()
    square, total, largest, mean = (to_numpy(t) for t in got)
    want = run_oracle(tracer.trace(program, ("float32", shape)), [x])
    np.testing.assert_array_equal(square.view(np.uint32), want[0].view(np.uint32))
    exact = (x.astype(np.float64) ** 2).sum()
    assert abs(float(total) - exact) <= 1e-6 * exact
    assert float(largest) == float(want[2]) == float(x.max())
    assert abs(float(mean) - x.astype(np.float64).mean()) <= 1e-6 * np.abs(x).astype(np.float64).mean()


@pytest.mark.parametrize("shape", [(4, 1000000), (2, 3, 524288), (2, 600, 1000), (6, 300006), (3, 300007), (2, 2, 600014)])
def test_rows_longer_than_a_block_takes(cuda, shape):
    """Sums and maxima over the trailing axes of tensors that also have leading ones, with rows of more than 262,144
    elements: each row is reduced in pieces and the pieces' results per row (a prime length, or twice a prime, as a head
    of whole pieces and a tail). Sums within 1e-6 of the float64 sum of magnitudes, maxima exact."""
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    axes = (-2, -1) if len(shape) == 3 else (-1,)

    def program(a):
        return F.sum(a, axes), F.amax(a * a, axes), F.sum(a * a, -1)

    got = [to_numpy(t) for t in lumen_b200.compile(program)(to_torch(x, cuda))]
    device_status()
    wide = x.astype(np.float64)
    assert got[0].shape == wide.sum(axes).shape
    assert (np.abs(got[0] - wide.sum(axes)) <= 1e-6 * np.abs(wide).sum(axes)).all()
    np.testing.assert_array_equal(got[1], (x * x).max(axes))
    assert (np.abs(got[2] - (wide * wide).sum(-1)) <= 1e-6 * (wide * wide).sum(-1)).all()


@pytest.mark.parametrize("dtype", ["uint8", "bfloat16", "float32", "float64"])
@pytest.mark.parametrize("shape,perm", [((3, 70, 50), (0, 2, 1)), ((5, 33, 7, 40), (0, 3, 2, 1)), ((5, 33, 7, 40), (3, 1, 0, 2)),
                                        ((2, 100, 3), (2, 0, 1)), ((64, 9, 130), (2, 1, 0)), ((6, 1000), (1, 0))])
def test_permuted_views_are_copied_exactly(cuda, dtype, shape, perm):
    """A permutation of a tensor's axes returned as it is (copied out of the view) and read by a kernel (copied to a dense
    place first), for element sizes of 1, 2, 4 and 8 bytes and axes that are and are not multiples of the 32 x 32 tiles
    the transposing copies move: exactly numpy's transpose."""
    rng = np.random.default_rng(len(shape) + sum(perm))
    if dtype == "uint8":
        x = rng.integers(0, 255, shape, dtype=np.uint8)
    else:
        x = rng.standard_normal(shape).astype(np.float32)
        x = bf16(x) if dtype == "bfloat16" else x.astype(dtype)
    from lumen_b200 import prims

    def program(a):
        t = prims.transpose(a, perm)
        return t, prims.max(t, t)

    moved, through_kernel = (to_numpy(t) for t in lumen_b200.compile(program)(to_torch(x, cuda)))
    device_status()
    want = np.ascontiguousarray(np.transpose(x, perm))
    view = {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[want.dtype.itemsize]
    np.testing.assert_array_equal(moved.view(view), want.view(view))
    np.testing.assert_array_equal(through_kernel.view(view), want.view(view))
