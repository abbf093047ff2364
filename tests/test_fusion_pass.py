"""The fusion pass on graphs of bare prims: what it groups, and that grouping changes no value (the oracle evaluates
fusion bodies primitive by primitive, so the fused graph must give bit-identical results)."""

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import prims, tracer
from lumen_b200.compiler import compile_graph
from lumen_b200.fusion_pass import fuse
from tests.helpers import bf16, run_oracle


def fusions(g):
    return [n for n in g.nodes if n.op == "fusion"]


def bare(g):
    return [n.op for n in g.nodes if n.op not in ("fusion", "fusion_output", "reshape", "slice", "dot_general", "concatenate")]


def same_values(g, fused, inputs):
    want, got = run_oracle(g, inputs), run_oracle(fused, inputs)
    assert len(want) == len(got)
    for a, b in zip(want, got):
        assert a.dtype == b.dtype and a.shape == b.shape
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_chain_with_a_row_sum_becomes_one_fusion():
    def chain(x, gg, b):
        y = F.relu(x * gg + b)
        return y, prims.reduce_sum(y * y, (1,), "float32")

    g = tracer.trace(chain, ("float32", (64, 256)), ("float32", (256,)), ("float32", (256,)))
    fused = fuse(g)
    assert len(fusions(fused)) == 1 and not bare(fused)
    f = fusions(fused)[0]
    assert f.params["name"] == "row" and len(f.params["body"].outputs) == 2  # y and the row sums: a multi-output fusion
    rng = np.random.default_rng(0)
    same_values(g, fused, [rng.standard_normal((64, 256), dtype=np.float32), rng.standard_normal(256, dtype=np.float32),
                           rng.standard_normal(256, dtype=np.float32)])
    assert compile_graph(g).labels == ["row"]


def test_softmax_row_is_one_fusion_and_a_reduction_keeps_its_epilogue():
    def program(x, w):
        p = F.softmax(x, -1)  # two reductions over the row and the elementwise work between and after them
        s = F.sum(p * w, -1) * 0.5  # a reduction with a prologue and an epilogue
        return p, s

    g = tracer.trace(program, ("float32", (32, 128)), ("float32", (32, 128)))
    fused = fuse(g)
    assert not bare(fused)
    assert len(fusions(fused)) <= 2
    rng = np.random.default_rng(1)
    same_values(g, fused, [rng.standard_normal((32, 128), dtype=np.float32), rng.standard_normal((32, 128), dtype=np.float32)])


def test_column_and_row_reductions_do_not_share_a_kernel():
    def program(x):
        return F.sum(x, 0), F.sum(x, 1)

    g = tracer.trace(program, ("float32", (128, 64)))
    fused = fuse(g)
    assert len(fusions(fused)) == 2 and not bare(fused)
    same_values(g, fused, [np.random.default_rng(2).standard_normal((128, 64), dtype=np.float32)])


def test_gemm_takes_its_elementwise_tail_as_an_epilogue():
    dims = (((1,), (0,)), ((), ()))

    def program(a, w, r, u):
        y = prims.dot_general(a, w, dims, "float32", "bfloat16")
        z = F.relu(prims.dot_general(y + r, w, dims, "float32", "bfloat16"))  # y + r feeds only this product's operand
        m = F.where(F.gt(u, 0), prims.dot_general(z, w, dims, "float32", "bfloat16"), 0)
        return m

    t = ("bfloat16", (128, 128))
    g = tracer.trace(program, t, t, t, t)
    fused = fuse(g)
    names = [f.params["name"] for f in fusions(fused)]
    assert names.count("dot_general") == 3 and not bare(fused)
    labels = compile_graph(g).labels
    assert labels == ["dot_general_add", "dot_general_relu", "dot_general_relu_backward"]
    rng = np.random.default_rng(3)
    same_values(g, fused, [bf16(rng.standard_normal((128, 128)) / 12) for _ in range(4)])


def test_traced_fusions_pass_through_and_constants_of_unfusible_readers_stay_plain():
    from lumen_b200 import transformer as T

    cfg = T.Config(vocab=32, d_model=32, heads=2, hidden=64, layers=1, seq=16, dtype="float32")
    g, _, _ = T.trace_train_step(cfg, 2)
    fused = fuse(g)
    assert [n.op for n in fused.nodes] == [n.op for n in g.nodes]


@pytest.mark.parametrize("shape", [(1000003,), (3, 300007), (2, 2, 600014), (4, 1000000), (4096, 1536), (131072,)])
def test_long_reductions_are_split_without_changing_their_values(shape):
    """`simplify.split_long_reductions` (the last step of `clean`): sums and maxima over more elements than one block
    takes as a row - whole tensors and rows, lengths with and without useful divisors (1,000,003 and 300,007 are prime,
    600,014 is twice a prime) - evaluated by the oracle before and after the pass: maxima equal, sums within the
    rounding of a float32 sum; a reduction that fits one block is left as it is."""
    from lumen_b200.simplify import LONGEST_ROW, clean

    whole = len(shape) == 1 or shape == (4096, 1536)

    def program(x):
        return (F.sum(x), F.amax(x * x)) if whole else (F.sum(x, -1), F.amax(x * x, -1))

    g = tracer.trace(program, ("float32", shape))
    cleaned = clean(g)
    x = np.random.default_rng(len(shape)).standard_normal(shape).astype(np.float32)
    before, after = run_oracle(g, [x]), run_oracle(cleaned, [x])
    row = shape[-1] if not whole else int(np.prod(shape))
    assert (sum(n.op in ("reduce_sum", "reduce_max") for n in cleaned.nodes) > 2) == (row > LONGEST_ROW)
    exact = x.astype(np.float64).sum() if whole else x.astype(np.float64).sum(-1)
    magnitude = np.abs(x.astype(np.float64)).sum() if whole else np.abs(x.astype(np.float64)).sum(-1)
    assert after[0].shape == before[0].shape and after[1].shape == before[1].shape
    assert (np.abs(after[0] - exact) <= 1e-6 * magnitude).all()
    np.testing.assert_array_equal(after[1], before[1])
