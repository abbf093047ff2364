"""The torch-style functions of `lumen_b200.functional` that are compositions of prims, evaluated by the oracle against
NumPy: the reductions written through an order-reversing flip (amin, min, all), first-index arg-reductions, the
logical functions on truth values, concatenations (cat, stack, pad), triangles, and the gated activations
(lumen/functional/functions.py:504-685)."""

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import tracer
from tests.helpers import run_oracle


def run(fn, *arrays):
    g = tracer.trace(fn, *[(str(a.dtype), a.shape) for a in arrays])
    return run_oracle(g, list(arrays))


@pytest.fixture
def xy():
    rng = np.random.default_rng(21)
    return rng.standard_normal((5, 7)).astype(np.float32), rng.standard_normal((5, 7)).astype(np.float32)


def test_min_reductions_and_arg_reductions(xy):
    x, _ = xy
    x[2, 3] = x[2, 5] = x.max() + 1  # a tie: the first index wins
    ints = (x * 10).astype(np.int32)
    u8 = np.abs(ints).astype(np.uint8)
    np.testing.assert_array_equal(run(lambda a: F.amin(a, 1), x)[0], x.min(1))
    np.testing.assert_array_equal(run(lambda a: F.amin(a, 0, keepdim=True), ints)[0], ints.min(0, keepdims=True))
    np.testing.assert_array_equal(run(lambda a: F.amin(a, 1), u8)[0], u8.min(1))  # unsigned: flipped bitwise
    assert run(lambda a: F.min(a), x)[0] == x.min() and run(lambda a: F.max(a), x)[0] == x.max()
    np.testing.assert_array_equal(run(lambda a: F.argmax(a, 1), x)[0], x.argmax(1).astype(np.int32))
    np.testing.assert_array_equal(run(lambda a: F.argmin(a, 0, keepdim=True), x)[0], x.argmin(0)[None].astype(np.int32))
    assert run(lambda a: F.argmax(a), x)[0] == x.argmax()  # flattened


def test_logical_functions_take_truth_values(xy):
    x, y = xy
    x[0, 0] = 0.0
    ints = (y * 3).astype(np.int64)
    np.testing.assert_array_equal(run(lambda a, b: F.logical_and(a, b), x, ints)[0], np.logical_and(x, ints))
    np.testing.assert_array_equal(run(lambda a, b: F.logical_or(a, b), x, ints)[0], np.logical_or(x, ints))
    np.testing.assert_array_equal(run(lambda a: F.logical_not(a), ints)[0], np.logical_not(ints))
    np.testing.assert_array_equal(run(lambda a: F.any(a, 1), ints)[0], ints.any(1))
    np.testing.assert_array_equal(run(lambda a: F.all(a, 0, keepdim=True), ints)[0], ints.all(0, keepdims=True))
    assert run(lambda a: F.all(a > -100.0), x)[0] and not run(lambda a: F.any(a > 100.0), x)[0]


def test_float_classification(xy):
    x, _ = xy
    x[1, 1], x[2, 2], x[3, 3] = np.nan, np.inf, -np.inf
    np.testing.assert_array_equal(run(F.isnan, x)[0], np.isnan(x))
    np.testing.assert_array_equal(run(F.isfinite, x)[0], np.isfinite(x))
    ints = np.arange(6, dtype=np.int32)
    assert run(F.isfinite, ints)[0].all() and not run(F.isnan, ints)[0].any()
    np.testing.assert_array_equal(run(F.sign, x)[0][np.isfinite(x)], np.sign(x)[np.isfinite(x)])
    np.testing.assert_array_equal(run(F.abs, x)[0][~np.isnan(x)], np.abs(x)[~np.isnan(x)])


def test_concatenations_and_triangles(xy):
    x, y = xy
    np.testing.assert_array_equal(run(lambda a, b: F.cat([a, b], 1), x, y)[0], np.concatenate([x, y], 1))
    np.testing.assert_array_equal(run(lambda a, b: F.stack([a, b], 0), x, y)[0], np.stack([x, y], 0))
    np.testing.assert_array_equal(run(lambda a, b: F.stack([a, b], -1), x, y)[0], np.stack([x, y], -1))
    np.testing.assert_array_equal(run(lambda a: F.pad(a, (1, 2, 0, 3), value=-1.0), x)[0],
                                  np.pad(x, ((0, 3), (1, 2)), constant_values=-1.0))  # fmt: skip
    np.testing.assert_array_equal(run(lambda a: F.pad(a, (0, 0)), x)[0], x)
    for k in (-1, 0, 2):
        np.testing.assert_array_equal(run(lambda a: F.triu(a, k), x)[0], np.triu(x, k))
    with pytest.raises(ValueError):
        run(lambda a: F.pad(a, (1,)), x)


def test_gated_activations_and_pow(xy):
    x, y = xy
    silu = x / (1.0 + np.exp(-x.astype(np.float64)))
    np.testing.assert_allclose(run(F.silu, x)[0], silu, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(run(lambda a, b: F.swiglu(a, b), x, y)[0], silu * y, rtol=1e-6, atol=1e-7)
    x64 = x.astype(np.float64)
    gelu = 0.5 * x64 * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x64 + 0.044715 * x64**3)))
    np.testing.assert_allclose(run(F.gelu, x)[0], gelu, rtol=1e-5, atol=1e-6)
    pos = np.abs(x) + 0.5
    np.testing.assert_allclose(run(lambda a, b: F.pow(a, b), pos, y)[0], pos.astype(np.float64) ** y, rtol=1e-6)
    with pytest.raises(TypeError):
        run(F.silu, np.arange(4, dtype=np.int32))
