"""`lb_scatter_add_rows` against the oracle's `scatter_add` (lumen/reference/mod.rs:765-808). The deterministic form
adds a row's updates in update order with a rounding after every add, so it is bit-exact, also where thousands of
updates hit one row; the atomic form agrees to rounding."""

import numpy as np
import pytest
import torch

from lumen_b200 import prims, tracer
from lumen_b200.runtime import scatter_add_rows
from oracle import oracle
from tests.helpers import bf16, to_numpy, to_torch

pytestmark = pytest.mark.gpu


def oracle_scatter(table, ids, updates):
    names = {v: k for k, v in oracle.NUMPY.items()}
    g = tracer.trace(lambda t, i, u: prims.scatter_add(t, i, u, 0), *[(names[np.dtype(a.dtype)], a.shape) for a in (table, ids, updates)])
    return oracle.run(g, [table, ids, updates])[0]


CASES = [
    # rows, width, picks, id dtype, value dtype, spread of the ids
    (64, 96, 512, np.int64, "bfloat16", 64),      # heavy collisions, 8 per row on average
    (1000, 256, 3000, np.int32, "float32", 1000),
    (16, 40, 5000, np.int64, "bfloat16", 2),      # two rows take 2500 picks each: the rank-sorted long-segment path
    (33, 8, 1, np.int64, "float32", 33),
    (128, 1024, 4096, np.int64, "bfloat16", 128),
]


@pytest.mark.parametrize("rows,width,picks,id_dtype,dtype,spread", CASES)
def test_deterministic_scatter_add_is_bit_exact(cuda, rows, width, picks, id_dtype, dtype, spread):
    rng = np.random.default_rng(rows + picks)
    cast = bf16 if dtype == "bfloat16" else (lambda a: np.asarray(a, np.float32))
    table = cast(rng.standard_normal((rows, width)))
    updates = cast(rng.standard_normal((picks, width)))
    ids = rng.integers(-2, spread + 2, picks).astype(id_dtype)  # a few out of range on both sides: clamped
    want = oracle_scatter(table, ids, updates)
    got = scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=True)
    again = scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=True)
    np.testing.assert_array_equal(to_numpy(got).view(np.uint16 if dtype == "bfloat16" else np.uint32),
                                  want.view(np.uint16 if dtype == "bfloat16" else np.uint32))
    assert torch.equal(got, again)


def test_atomic_scatter_add_agrees_to_rounding(cuda):
    rng = np.random.default_rng(5)
    table = np.zeros((64, 128), np.float32)
    updates = rng.standard_normal((1024, 128)).astype(np.float32)
    ids = rng.integers(0, 64, 1024).astype(np.int64)
    want = oracle_scatter(table, ids, updates)
    got = scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=False)
    np.testing.assert_allclose(to_numpy(got), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("seed", range(40))
def test_random_scatter_adds(cuda, seed):
    """Random tables (1 - 500 rows of 1 - 1000 values), 0 - 5000 updates spread over all rows, a few rows or one row, ids
    of either width with some out of range: the deterministic form equals the oracle bit for bit and repeats; the atomic
    form agrees within the rounding of a float32 sum (1e-5 of the row's sum of magnitudes, plus bfloat16's half ulp)."""
    rng = np.random.default_rng(seed + 900)
    rows = int(rng.choice([1, 2, 7, 33, 64, 100, 500]))
    width = int(rng.choice([1, 3, 8, 33, 64, 100, 256, 1000]))
    picks = int(rng.choice([0, 1, 17, 300, 1000, 5000]))
    dtype = ["float32", "bfloat16"][int(rng.integers(2))]
    id_dtype = [np.int64, np.int32][int(rng.integers(2))]
    spread = int(rng.choice([1, max(rows // 8, 1), rows]))
    cast = bf16 if dtype == "bfloat16" else (lambda a: np.asarray(a, np.float32))
    table = cast(rng.standard_normal((rows, width)))
    updates = cast(rng.standard_normal((picks, width)))
    ids = rng.integers(-1, spread + 1, picks).astype(id_dtype)
    want = oracle_scatter(table, ids, updates)
    got = scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=True)
    again = scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=True)
    bits = np.uint16 if dtype == "bfloat16" else np.uint32
    np.testing.assert_array_equal(to_numpy(got).view(bits), want.view(bits), err_msg=f"{rows}x{width}, {picks} updates, {dtype}")
    assert torch.equal(got, again)
    atomic = to_numpy(scatter_add_rows(to_torch(table, cuda), to_torch(ids, cuda), to_torch(updates, cuda), deterministic=False)).astype(np.float64)
    # float64 sums and the magnitudes that bound a float32 sum's rounding, rows clamped as the primitive clamps them
    exact, magnitude = table.astype(np.float64), np.abs(table.astype(np.float64))
    clamped = np.clip(ids.astype(np.int64), 0, rows - 1)
    np.add.at(exact, clamped, updates.astype(np.float64))
    np.add.at(magnitude, clamped, np.abs(updates.astype(np.float64)))
    bound = 1e-5 * magnitude + (2.0**-8 * np.abs(exact) if dtype == "bfloat16" else 0.0)
    assert (np.abs(atomic - exact) <= bound + 1e-30).all(), f"{rows}x{width}, {picks} updates, {dtype}"
