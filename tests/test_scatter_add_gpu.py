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
