"""Parity of lb_gemm with the oracle's dot_general, small shapes and large: the CUDA-core kernel accumulates in the interpreter's order and
is bit-exact; the tcgen05 kernel sums in tensor-core order and is held to the reference's bf16 tolerance."""

import numpy as np
import pytest
import torch

from lumen_b200 import functional as F
from lumen_b200 import tracer
from lumen_b200.runtime import device_status, gemm, gemm_scratch_bytes
from tests.helpers import bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def operands(m, n, k, seed, batch=None):
    rng = np.random.default_rng(seed)
    lead = () if batch is None else (batch,)
    a = (rng.standard_normal(lead + (m, k)) / np.sqrt(k)).astype(np.float32)
    b = (rng.standard_normal(lead + (k, n)) / np.sqrt(k)).astype(np.float32)
    return a, b


def oracle_matmul(a, b, dtype, out_dtype):
    g = tracer.trace(lambda x, y: F.matmul(x, y, "float32", out_dtype), (dtype, a.shape), (dtype, b.shape))
    return run_oracle(g, [a, b])[0]


@pytest.mark.parametrize("shape", [(64, 48, 40), (130, 70, 33), (1, 5, 7)])
def test_float32_gemm_is_bit_exact(cuda, shape):
    """float32 operands: products and sums rounded one by one in contracting order (lumen/reference/mod.rs:958-970)."""
    m, n, k = shape
    a, b = operands(m, n, k, 0)
    out = torch.empty((m, n), dtype=torch.float32, device=cuda)
    gemm(to_torch(a, cuda), to_torch(b, cuda), out)
    np.testing.assert_array_equal(to_numpy(out), oracle_matmul(a, b, "float32", "float32"))


def test_simt_bf16_gemm_is_bit_exact(cuda):
    a, b = operands(96, 80, 72, 1)
    a, b = bf16(a), bf16(b)
    for out_dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        out = torch.empty((96, 80), dtype=td, device=cuda)
        gemm(to_torch(a, cuda), to_torch(b, cuda), out, kernel="simt")
        want = oracle_matmul(a, b, "bfloat16", out_dtype)
        np.testing.assert_array_equal(to_numpy(out).astype(np.float32), want.astype(np.float32))


MAJORS = [("row", "row"), ("row", "col"), ("col", "row"), ("col", "col")]


def with_major(x, major, cuda):
    """A [.., R, C] device tensor whose memory is row-major ("row") or column-major ("col")."""
    t = to_torch(x, cuda)
    if major == "col":
        t = t.transpose(-1, -2).contiguous().transpose(-1, -2)
    return t


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_1cta"])
@pytest.mark.parametrize("majors", MAJORS)
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 320), (200, 264, 136), (384, 1000, 72), (8, 8, 8), (1152, 520, 448)])
def test_tcgen05_gemm_all_majors(cuda, shape, majors, kernel):
    """Both tensor-core kernels (CTA pairs for M > 128 under "tcgen05", one CTA per tile under "tcgen05_1cta"),
    every operand major (the transposed views of the backward GEMMs), ragged edges in M, N and K: float32
    outputs differ from the oracle only by the order of the float32 sums, so they are held to 1e-4 (far inside the
    reference's 1e-2 * max|want| for bf16 operands, tests/codegen/test_dot_general.py:41-42,168-169)."""
    m, n, k = shape
    a, b = operands(m, n, k, 2)
    a, b = bf16(a), bf16(b)
    want = oracle_matmul(a, b, "bfloat16", "float32")
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=cuda)
    gemm(with_major(a, majors[0], cuda), with_major(b, majors[1], cuda), out, kernel=kernel)
    device_status()
    got = to_numpy(out)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4 * np.abs(want).max())
    assert np.abs(got - want).max() <= 1e-2 * np.abs(want).max()


def test_tcgen05_gemm_bf16_output_batched_relu(cuda):
    a, b = operands(192, 320, 128, 3, batch=3)
    a, b = bf16(a), bf16(b)
    want = oracle_matmul(a, b, "bfloat16", "float32")
    out = torch.empty((3, 192, 320), dtype=torch.bfloat16, device=cuda)
    gemm(to_torch(a, cuda), to_torch(b, cuda), out, epilogue="relu", kernel="tcgen05")
    device_status()
    want = np.maximum(want, 0)
    np.testing.assert_allclose(to_numpy(out).astype(np.float32), want, rtol=2**-6, atol=2**-6 * np.abs(want).max())


def test_tcgen05_matches_exact_accumulation_at_large_k(cuda):
    """K = 4096 over several waves of tiles, against the ORACLE's dot_general on the same operands: the CUDA-core
    kernel (the interpreter's order) bit for bit, the tensor-core result within 1e-3 of the largest value; and linearity
    in A as a size-independent property."""
    m, n, k = 1024, 2048, 4096
    a, b = operands(m, n, k, 4)
    want = oracle_matmul(bf16(a), bf16(b), "bfloat16", "float32")
    a_t, b_t = to_torch(bf16(a), cuda), to_torch(bf16(b), cuda)
    fast = torch.empty((m, n), dtype=torch.float32, device=cuda)
    exact = torch.empty((m, n), dtype=torch.float32, device=cuda)
    gemm(a_t, b_t, fast, kernel="tcgen05")
    gemm(a_t, b_t, exact, kernel="simt")
    device_status()
    np.testing.assert_array_equal(to_numpy(exact), want)
    scale = float(np.abs(want).max())
    assert float(np.abs(to_numpy(fast) - want).max()) <= 1e-3 * scale
    doubled = torch.empty_like(fast)
    gemm(a_t * 2, b_t, doubled, kernel="tcgen05")
    torch.testing.assert_close(doubled, fast * 2, rtol=0, atol=0)


@pytest.mark.parametrize("shape", [(256, 512, 8192), (1024, 1024, 16384), (200, 264, 4104)])
def test_split_k_weight_gradient_shapes(cuda, shape):
    """Few output tiles and a long K (dW = dY^T X with both operands transposed views): K is cut into ranges,
    partial tiles are added in a fixed order. Same tolerance as the unsplit kernel, bf16 output, reproducible."""
    m, n, k = shape
    rng = np.random.default_rng(5)
    a = bf16(rng.standard_normal((k, m)) / np.sqrt(k))  # stored [K, M]: A = a.T is a transposed view
    b = bf16(rng.standard_normal((k, n)))
    nbytes = gemm_scratch_bytes(m, n, k)
    assert nbytes > 0
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
    a_t, b_t = to_torch(a, cuda), to_torch(b, cuda)
    split = torch.empty((m, n), dtype=torch.bfloat16, device=cuda)
    whole = torch.empty((m, n), dtype=torch.float32, device=cuda)
    gemm(a_t.t(), b_t, split, kernel="tcgen05", scratch=scratch)
    gemm(a_t.t(), b_t, whole, kernel="simt")
    device_status()
    want = oracle_matmul(np.ascontiguousarray(a.T), b, "bfloat16", "float32")  # the oracle's dot_general on the same operands
    np.testing.assert_array_equal(to_numpy(whole), want)
    np.testing.assert_allclose(to_numpy(split).astype(np.float32), want, rtol=2**-7, atol=2**-7 * np.abs(want).max())
    again = torch.empty_like(split)
    gemm(a_t.t(), b_t, again, kernel="tcgen05", scratch=scratch)
    assert torch.equal(split, again)


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_1cta"])
@pytest.mark.parametrize("shape", [(384, 512, 256), (200, 264, 136), (256, 512, 8192)])
@pytest.mark.parametrize("epilogue", ["add", "mask_positive"])
def test_tcgen05_gemm_add_and_mask_epilogues(cuda, shape, epilogue, kernel):
    """The elementwise tails a `dot_general` fusion carries into the GEMM: `other + product` (a residual add) and
    `other > 0 ? product : 0` (a relu's backward), on aligned, ragged and split-K shapes. The product is rounded to
    bfloat16 first, as its own primitive; the reference value applies the tail to the CUDA-core kernel's exactly
    accumulated, rounded product, so the two differ only where tensor-core summation order moved a rounding."""
    m, n, k = shape
    rng = np.random.default_rng(11)
    a, b = bf16(rng.standard_normal((m, k)) / np.sqrt(k)), bf16(rng.standard_normal((k, n)))
    other = bf16(rng.standard_normal((m, n)))
    a_t, b_t, o_t = to_torch(a, cuda), to_torch(b, cuda), to_torch(other, cuda)
    nbytes = gemm_scratch_bytes(m, n, k)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=cuda) if nbytes else None
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda)
    gemm(a_t, b_t, got, epilogue=epilogue, aux=o_t, kernel=kernel, scratch=scratch)
    exact = torch.empty((m, n), dtype=torch.bfloat16, device=cuda)
    gemm(a_t, b_t, exact, kernel="simt")
    device_status()
    np.testing.assert_array_equal(to_numpy(exact), oracle_matmul(a, b, "bfloat16", "bfloat16"))  # the oracle's rounded product
    product, oth = exact.float(), o_t.float()
    want = (oth + product).bfloat16().float() if epilogue == "add" else torch.where(oth > 0, product, torch.zeros_like(product))
    scale = float(want.abs().max())
    torch.testing.assert_close(got.float(), want, rtol=2**-6, atol=2**-6 * scale)
    if epilogue == "mask_positive":
        assert torch.equal(got.float() == 0, (oth <= 0) | (got.float() == 0)) and bool(((got.float() == 0) | (oth > 0)).all())


def test_gemm_epilogue_operand_is_checked(cuda):
    a = torch.zeros((256, 64), dtype=torch.bfloat16, device=cuda)
    b = torch.zeros((64, 256), dtype=torch.bfloat16, device=cuda)
    out = torch.zeros((256, 256), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(Exception, match="epilogue"):
        gemm(a, b, out, epilogue="add")
    with pytest.raises(Exception, match="shape"):
        gemm(a, b, out, epilogue="add", aux=torch.zeros((256, 128), dtype=torch.bfloat16, device=cuda))


def test_benchmark_size_checksums(cuda):
    """8192 x 8192 x 8192 (the matmul benchmark's forward and both backward products), checked through properties
    that need no full-size reference: the column sums of A B equal (column sums of A) B and the row sums equal
    A (row sums of B), both evaluated in float64 from the same bfloat16 operands; a sampled block of the output
    equals the oracle's product of the matching operand slices."""
    n = 8192
    gen = torch.Generator(device=cuda).manual_seed(2)
    a = (torch.randn((n, n), generator=gen, device=cuda) / n**0.5).bfloat16()
    b = (torch.randn((n, n), generator=gen, device=cuda) / n**0.5).bfloat16()
    dy = torch.randn((n, n), generator=gen, device=cuda).bfloat16()
    y = torch.empty((n, n), dtype=torch.float32, device=cuda)
    da = torch.empty((n, n), dtype=torch.bfloat16, device=cuda)
    db = torch.empty((n, n), dtype=torch.bfloat16, device=cuda)
    gemm(a, b, y)
    gemm(dy, b.t(), da)  # dA = dY B^T
    gemm(a.t(), dy, db)  # dB = A^T dY
    device_status()
    for left, right, out, tol in ((a, b, y, 1e-4), (dy, b.t(), da, 2**-7), (a.t(), dy, db, 2**-7)):
        l64, r64, o64 = left.double(), right.double(), out.double()
        cols = l64.sum(0) @ r64
        rows = l64 @ r64.sum(1)
        scale = float(o64.abs().max()) * n**0.5  # a sum of n outputs, each off by at most tol * max|out|
        assert float((o64.sum(0) - cols).abs().max()) <= tol * scale
        assert float((o64.sum(1) - rows).abs().max()) <= tol * scale
        # a [128, 256] block of the output against the oracle's dot_general of the matching operand slices
        want = oracle_matmul(to_numpy(left[4096:4224].contiguous()), to_numpy(right[:, 7936:8192].contiguous()), "bfloat16", "float32")
        block = to_numpy(out[4096:4224, 7936:8192].float())
        assert float(np.abs(block - want).max()) <= tol * float(np.abs(want).max())


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_1cta"])
def test_tcgen05_gemm_takes_float16_operands(cuda, kernel):
    """float16 operands on the tensor-core kernels (the MMA's operand-format bit): float32 and float16 outputs, a
    transposed operand and a ragged shape, against the oracle's float16 dot_general
    (tests/codegen/test_dot_general.py:128-169 runs the same dtypes)."""
    m, n, k = 264, 328, 200
    a, b = operands(m, n, k, 7)
    a, b = a.astype(np.float16), b.astype(np.float16)
    want = oracle_matmul(a, b, "float16", "float32")
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=cuda)
    gemm(to_torch(a, cuda), to_torch(np.ascontiguousarray(b.T), cuda).t(), out, kernel=kernel)
    device_status()
    np.testing.assert_allclose(to_numpy(out), want, rtol=1e-4, atol=1e-4 * np.abs(want).max())
    narrow = torch.full((m, n), float("nan"), dtype=torch.float16, device=cuda)
    gemm(to_torch(a, cuda), to_torch(b, cuda), narrow, epilogue="relu", kernel=kernel)
    device_status()
    want16 = np.maximum(want, 0).astype(np.float16).astype(np.float32)
    np.testing.assert_allclose(to_numpy(narrow).astype(np.float32), want16, rtol=2**-9, atol=2**-9 * np.abs(want16).max())
