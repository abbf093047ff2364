"""Parity of the tcgen05 flash-attention kernels with the traced program evaluated by the oracle, and with a
float64 NumPy attention at sizes the oracle is too slow for."""

import numpy as np
import pytest
import torch

from lumen_b200 import functional as F
from lumen_b200 import tracer
from lumen_b200.runtime import attention_backward, attention_forward, device_status
from tests.helpers import attention_f64, bf16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu

TOL = 2e-2  # bfloat16, rtol = atol (tests/functional/test_attention.py:54)


def qkv(b, sq, sk, n, nkv, h, seed=3):
    rng = np.random.default_rng(seed)
    return tuple(bf16(rng.standard_normal(s)) for s in ((b, sq, n, h), (b, sk, nkv, h), (b, sk, nkv, h)))


# (B, Sq, Sk, N, Nkv, H), causal: ragged lengths, GQA, a KV cache shape, both head dims
CASES = [
    ((2, 128, 128, 2, 2, 128), False),
    ((1, 256, 256, 2, 2, 128), True),
    ((2, 100, 100, 4, 2, 64), True),
    ((1, 130, 77, 2, 2, 64), False),
    ((1, 70, 200, 2, 1, 128), True),
    ((1, 300, 300, 3, 3, 128), True),
    ((1, 1, 300, 8, 2, 128), True),
]


@pytest.mark.parametrize("case", CASES)
def test_forward_matches_the_traced_program(cuda, case):
    (b, sq, sk, n, nkv, h), causal = case
    q, k, v = qkv(b, sq, sk, n, nkv, h)
    g = tracer.trace(lambda a, c, d: F.attention_forward_prims(a, c, d, h**-0.5, causal),
                     ("bfloat16", q.shape), ("bfloat16", k.shape), ("bfloat16", v.shape))
    want_o, want_lse = run_oracle(g, [q, k, v])
    o, lse = attention_forward(to_torch(q, cuda), to_torch(k, cuda), to_torch(v, cuda), causal=causal)
    device_status()
    np.testing.assert_allclose(to_numpy(o).astype(np.float32), want_o.astype(np.float32), rtol=TOL, atol=TOL)
    np.testing.assert_allclose(to_numpy(lse), want_lse[..., 0], rtol=1e-3, atol=1e-3)


def test_forward_reads_strided_views_in_place(cuda):
    """q, k, v as slices of one packed [B, S, 3, N, H] projection: no copies (strided accesses,
    lumen/graph_compiler/passes/attention/forward.rs:598-772)."""
    rng = np.random.default_rng(5)
    packed = to_torch(bf16(rng.standard_normal((2, 192, 3, 2, 64))), cuda)
    q, k, v = packed[:, :, 0], packed[:, :, 1], packed[:, :, 2]
    o, _ = attention_forward(q, k, v, causal=True)
    device_status()
    want, _ = attention_f64(to_numpy(q.contiguous()), to_numpy(k.contiguous()), to_numpy(v.contiguous()), True)
    np.testing.assert_allclose(to_numpy(o).astype(np.float64), want, rtol=TOL, atol=TOL)


def test_forward_at_benchmark_length(cuda):
    """Sequence 4096, head dim 128, causal (the benchmark shape at batch 1, 2 heads): against float64."""
    q, k, v = qkv(1, 4096, 4096, 2, 2, 128)
    o, lse = attention_forward(to_torch(q, cuda), to_torch(k, cuda), to_torch(v, cuda), causal=True)
    device_status()
    want, want_lse = attention_f64(q, k, v, True)
    np.testing.assert_allclose(to_numpy(o).astype(np.float64), want, rtol=TOL, atol=TOL)
    np.testing.assert_allclose(to_numpy(lse), want_lse, rtol=1e-3, atol=1e-3)
    # size-independent property: a row's output is a convex combination of value rows
    assert np.isfinite(to_numpy(o).astype(np.float32)).all()
    assert float(np.abs(to_numpy(o).astype(np.float32)).max()) <= float(np.abs(v.astype(np.float32)).max()) + 1e-2


def close(got, want, tol=TOL):
    """rtol = atol = tol with atol scaled by max|want| (tests/functional/test_attention.py:409-413)."""
    want = want.astype(np.float64)
    np.testing.assert_allclose(got.astype(np.float64), want, rtol=tol, atol=tol * max(np.abs(want).max(), 1e-6))


BWD_CASES = [
    ((1, 128, 128, 1, 1, 128), False),
    ((2, 128, 128, 2, 2, 128), True),
    ((1, 256, 256, 2, 2, 64), True),
    ((2, 100, 100, 4, 2, 64), True),
    ((1, 130, 77, 2, 2, 64), False),
    ((1, 70, 200, 2, 1, 128), True),
    ((1, 300, 300, 3, 3, 128), True),
]


@pytest.mark.parametrize("case", BWD_CASES)
def test_backward_matches_the_traced_program(cuda, case):
    """dq, dk, dv against the CPU running the same traced forward+backward program
    (tests/functional/test_attention.py:382-413), including grouped-query heads and ragged lengths."""
    (b, sq, sk, n, nkv, h), causal = case
    q, k, v = qkv(b, sq, sk, n, nkv, h)
    do = bf16(np.random.default_rng(9).standard_normal(q.shape))
    scale = h**-0.5

    def program(q_, k_, v_, do_):
        o, lse = F.attention_forward_prims(q_, k_, v_, scale, causal)
        return F.attention_backward_prims(q_, k_, v_, o, lse, do_, scale, causal)

    g = tracer.trace(program, *[("bfloat16", a.shape) for a in (q, k, v, do)])
    want = run_oracle(g, [q, k, v, do])
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=causal)
    got = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    device_status()
    for name, a, w in zip(("dq", "dk", "dv"), got, want):
        close(to_numpy(a).astype(np.float32), w.astype(np.float32))


def test_backward_is_deterministic_and_finite_at_benchmark_length(cuda):
    """Sequence 4096, head dim 128, causal: two runs are bit-identical (no atomics;
    tests/functional/test_attention.py:403-407), and dV matches P^T dO recomputed in float64 for one head."""
    q, k, v = qkv(1, 4096, 4096, 2, 2, 128)
    do = bf16(np.random.default_rng(9).standard_normal(q.shape))
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=True)
    first = attention_backward(tq, tk, tv, o, tdo, lse, causal=True)
    second = attention_backward(tq, tk, tv, o, tdo, lse, causal=True)
    device_status()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
        assert torch.isfinite(a.float()).all()
    qh, kh, vh, doh = (a[0, :, 0].astype(np.float64) for a in (q, k, v, do))
    s = qh @ kh.T / np.sqrt(128)
    s = np.where(np.tril(np.ones((4096, 4096), bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    close(to_numpy(first[2])[0, :, 0].astype(np.float32), p.T @ doh)
    dp = doh @ vh.T
    delta = (doh * (p @ vh)).sum(-1, keepdims=True)
    ds = p * (dp - delta) / np.sqrt(128)
    close(to_numpy(first[0])[0, :, 0].astype(np.float32), ds @ kh)
    close(to_numpy(first[1])[0, :, 0].astype(np.float32), ds.T @ qh)


# The shapes the 12-layer training step runs (head dim 64, sequence 2048) and the next length up: 16 to 64 key tiles per
# query tile, so the K/V ring, the barrier parities and the lazy rescaling all wrap many times.
LONG_D64 = [
    ((2, 2048, 2048, 2, 2, 64), True),
    ((1, 2048, 2048, 4, 2, 64), True),   # grouped-query heads 4:2
    ((1, 4096, 4096, 2, 2, 64), True),
    ((1, 2048, 2048, 2, 2, 64), False),
]


@pytest.mark.parametrize("case", LONG_D64)
def test_head_dim_64_at_training_lengths(cuda, case):
    """Forward and backward of the head-dim-64 kernels at the training step's sequence length against float64:
    o, dq, dk, dv within 2e-2 (of the largest value), the log-sum-exp within 1e-3; two backward runs bit-identical."""
    (b, sq, sk, n, nkv, h), causal = case
    q, k, v = qkv(b, sq, sk, n, nkv, h, seed=11)
    do = bf16(np.random.default_rng(12).standard_normal(q.shape))
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=causal)
    got = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    again = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    device_status()
    want_o, want_lse, want = attention_f64(q, k, v, causal, do)
    close(to_numpy(o).astype(np.float32), want_o)
    np.testing.assert_allclose(to_numpy(lse), want_lse, rtol=1e-3, atol=1e-3)
    for name, a, a2, w in zip(("dq", "dk", "dv"), got, again, want):
        assert torch.equal(a, a2), name
        close(to_numpy(a).astype(np.float32), w)


# The single-kernel backward (head dim 64): ragged lengths, grouped-query heads, Sq != Sk, several query tiles per key
# tile, and the training step's length.
ATOMIC_CASES = [
    ((1, 128, 128, 1, 1, 64), False),
    ((1, 256, 256, 2, 2, 64), True),
    ((2, 100, 100, 4, 2, 64), True),
    ((1, 130, 77, 2, 2, 64), False),
    ((1, 70, 200, 2, 1, 64), True),
    ((1, 300, 300, 3, 3, 64), True),
    ((1, 640, 640, 4, 1, 64), True),   # four query heads accumulate into one kv head over five query tiles
]


@pytest.mark.parametrize("case", ATOMIC_CASES)
def test_single_kernel_backward_matches_the_traced_program(cuda, case):
    """`lb_attention_bwd_atomic` (dQ added atomically into a float32 accumulator, the reference backend's default mode)
    against the CPU running the traced forward+backward program, at the tolerance of the deterministic pair; dK and dV
    are bit-identical between two runs, dQ agrees to the last bfloat16 bits."""
    (b, sq, sk, n, nkv, h), causal = case
    q, k, v = qkv(b, sq, sk, n, nkv, h)
    do = bf16(np.random.default_rng(9).standard_normal(q.shape))
    scale = h**-0.5

    def program(q_, k_, v_, do_):
        o, lse = F.attention_forward_prims(q_, k_, v_, scale, causal)
        return F.attention_backward_prims(q_, k_, v_, o, lse, do_, scale, causal)

    g = tracer.trace(program, *[("bfloat16", a.shape) for a in (q, k, v, do)])
    want = run_oracle(g, [q, k, v, do])
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=causal)
    got = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal, deterministic=False)
    again = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal, deterministic=False)
    device_status()
    for name, a, a2, w in zip(("dq", "dk", "dv"), got, again, want):
        close(to_numpy(a).astype(np.float32), w.astype(np.float32))
        if name == "dq":
            close(to_numpy(a2).astype(np.float32), to_numpy(a).astype(np.float32), tol=1e-2)
        else:
            assert torch.equal(a, a2), name


@pytest.mark.parametrize("case", LONG_D64)
def test_single_kernel_backward_at_training_lengths(cuda, case):
    """The single-kernel backward at sequence 2048 / 4096 against float64 and against the deterministic pair."""
    (b, sq, sk, n, nkv, h), causal = case
    q, k, v = qkv(b, sq, sk, n, nkv, h, seed=11)
    do = bf16(np.random.default_rng(12).standard_normal(q.shape))
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=causal)
    got = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal, deterministic=False)
    pair = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    device_status()
    _, _, want = attention_f64(q, k, v, causal, do)
    for name, a, a2, w in zip(("dq", "dk", "dv"), got, pair, want):
        close(to_numpy(a).astype(np.float32), w)
        close(to_numpy(a).astype(np.float32), to_numpy(a2).astype(np.float32), tol=1e-2)


def test_single_kernel_entry_runs_other_head_dims_as_the_pair(cuda):
    """`lb_attention_bwd_atomic` covers head dim 64; at head dim 128 it runs exactly what `lb_attention_bwd` runs
    (the accumulator is left unused), so the results are bit-identical to the deterministic entry's."""
    q, k, v = qkv(1, 256, 256, 2, 2, 128)
    do = bf16(np.random.default_rng(9).standard_normal(q.shape))
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=True)
    pair = attention_backward(tq, tk, tv, o, tdo, lse, causal=True)
    other = attention_backward(tq, tk, tv, o, tdo, lse, causal=True, deterministic=False)
    device_status()
    for a, b in zip(pair, other):
        assert torch.equal(a, b)


def random_attention_case(seed):
    """Batch 1-3, query and key lengths 1-700 (equal, or ragged either way), 1-6 query heads over a divisor of key/value
    heads, head dim 64 or 128 (the tensor-core kernels) or 32 / 80 (the SIMT kernels), causal or not."""
    rng = np.random.default_rng(seed + 400)
    h = int(rng.choice([64, 64, 128, 128, 32, 80]))
    n = int(rng.choice([1, 2, 3, 4, 6]))
    nkv = int(rng.choice([d for d in (1, 2, 3, 4, 6) if n % d == 0]))
    sq = int(rng.choice([1, 17, 64, 127, 128, 129, 255, 256, 300, 513, 700]))
    sk = sq if rng.random() < 0.5 else int(rng.choice([1, 17, 64, 127, 128, 129, 255, 256, 300, 513, 700]))
    causal = bool(rng.random() < 0.6)
    if causal and sk < sq:
        sk = sq  # a causal mask aligned to the last key needs at least as many keys as queries
    return (int(rng.integers(1, 4)), sq, sk, n, nkv, h), causal


@pytest.mark.parametrize("seed", range(32))
def test_random_attention_shapes_against_float64(cuda, seed):
    """Forward and both backward forms (the deterministic pair; the single kernel with atomic dQ, which head dim 64
    takes) on random shapes against float64: o, dq, dk, dv within 2e-2 (of the value and of the largest value), the
    log-sum-exp within 1e-3; the deterministic backward repeats bit for bit."""
    (b, sq, sk, n, nkv, h), causal = random_attention_case(seed)
    q, k, v = qkv(b, sq, sk, n, nkv, h, seed=seed + 50)
    do = bf16(np.random.default_rng(seed + 60).standard_normal(q.shape))
    tq, tk, tv, tdo = (to_torch(a, cuda) for a in (q, k, v, do))
    o, lse = attention_forward(tq, tk, tv, causal=causal)
    pair = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    again = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal)
    single = attention_backward(tq, tk, tv, o, tdo, lse, causal=causal, deterministic=False)
    device_status()
    want_o, want_lse, grads = attention_f64(q, k, v, causal, do)
    close(to_numpy(o).astype(np.float32), want_o)
    np.testing.assert_allclose(to_numpy(lse), want_lse, rtol=1e-3, atol=1e-3)
    for name, a, a2, s, w in zip(("dq", "dk", "dv"), pair, again, single, grads):
        # with a single key the probabilities are 1 and dq, dk are exactly zero: the tolerance is then 2e-2 of the
        # operands' unit scale times bfloat16's epsilon rather than of a zero maximum
        for result in (a, s):
            np.testing.assert_allclose(to_numpy(result).astype(np.float64), w, rtol=TOL, atol=TOL * max(np.abs(w).max(), 2.0**-8), err_msg=name)
        assert torch.equal(a, a2), name
