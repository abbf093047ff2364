"""Seeded random programs (tests/random_programs.py) compiled and run on the GPU against the oracle evaluating the same
traced program. Programs of exactly defined functions must agree bit for bit (NaNs in the same places); sums agree
within 1e-5 of the sum of magnitudes; programs that end in transcendental functions within a few ulp of the dtype."""

import os

import numpy as np
import pytest
import torch

import lumen_b200
from lumen_b200 import tracer
from lumen_b200.runtime import device_status
from tests import random_programs as R
from tests.helpers import BF16, run_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu

# how many seeds of each kind run; a longer hunt sets LUMEN_B200_TEST_SEEDS
EXACT_SEEDS = int(os.environ.get("LUMEN_B200_TEST_SEEDS", 24))
SMOOTH_SEEDS = int(os.environ.get("LUMEN_B200_TEST_SEEDS", 12))


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def run_both(seed, exact, cuda, lowering):
    recipe = R.draw_recipe(seed, exact)
    program, arrays = R.build(recipe), R.draw_inputs(recipe, seed)
    got = lumen_b200.compile(program, lowering=lowering)(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
    want = run_oracle(tracer.trace(program, *R.input_types(recipe)), arrays)
    assert len(got) == len(want)
    return recipe, got, want


def check_sum(kind, got, want, source, seed):
    axis = -1 if kind == "sum_last" else 0
    magnitudes = np.abs(np.nan_to_num(source.astype(np.float64), nan=0.0, posinf=0.0, neginf=0.0)).sum(axis)
    finite = np.isfinite(want)
    np.testing.assert_array_equal(np.isfinite(got), finite, err_msg=f"seed {seed}: {kind} finiteness")
    assert (np.abs(got[finite].astype(np.float64) - want[finite]) <= 1e-5 * magnitudes[finite] + 1e-30).all(), f"seed {seed}: {kind}"


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_exact_programs_match_the_oracle_bit_for_bit(cuda, seed):
    recipe, got, want = run_both(seed, True, cuda, "native" if seed % 4 else "optimising")
    outputs = recipe[4]
    for k, ((kind, _), g, w) in enumerate(zip(outputs, got, want)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        if kind in ("sum_last", "sum_first"):
            check_sum(kind, g, w, want[0], seed)
            continue
        if w.dtype in (np.float32, BF16):
            nan = np.isnan(w.astype(np.float32))
            np.testing.assert_array_equal(np.isnan(g.astype(np.float32)), nan, err_msg=f"seed {seed} output {k}: NaN places")
            np.testing.assert_array_equal(bits(g)[~nan], bits(w)[~nan], err_msg=f"seed {seed} output {k} ({kind})")
        else:
            np.testing.assert_array_equal(g, w, err_msg=f"seed {seed} output {k} ({kind})")


@pytest.mark.parametrize("seed", range(SMOOTH_SEEDS))
def test_programs_ending_in_transcendental_functions_match_within_tolerance(cuda, seed):
    """float32 results within 4e-6 of the value (a few ulp: CUDA's single-precision functions are within 2 ulp and one
    product or sum follows) plus 1e-6 of the output's largest magnitude where a sum cancels; bfloat16 results within two
    bfloat16 ulp (2^-6 of the value or of the largest magnitude), since a float32 difference can move the rounding of the
    function's result and of the product or sum after it."""
    recipe, got, want = run_both(seed, False, cuda, "native")
    outputs = recipe[4]
    for k, ((kind, _), g, w) in enumerate(zip(outputs, got, want)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        if w.dtype == bool:
            np.testing.assert_array_equal(g, w, err_msg=f"seed {seed} output {k}")
            continue
        g64, w64 = g.astype(np.float64), w.astype(np.float64)
        finite = np.isfinite(w64)
        np.testing.assert_array_equal(np.isfinite(g64), finite, err_msg=f"seed {seed} output {k}: finiteness")
        np.testing.assert_array_equal(g64[~finite & ~np.isnan(w64)], w64[~finite & ~np.isnan(w64)])
        half = recipe[1] == "bfloat16"
        if kind in ("sum_last", "sum_first"):
            source = want[0].astype(np.float64)
            axis = -1 if kind == "sum_last" else 0
            bound = (2.0**-6 if half else 2e-5) * np.abs(np.nan_to_num(source, nan=0.0, posinf=0.0, neginf=0.0)).sum(axis)
        else:
            largest = np.abs(w64[finite]).max() if finite.any() else 0.0
            bound = (2.0**-6 if half else 4e-6) * np.abs(w64) + (2.0**-6 if half else 1e-6) * largest
        error = np.abs(g64[finite] - w64[finite])
        assert (error <= (bound[finite] if np.ndim(bound) else bound) + 1e-30).all(), f"seed {seed} output {k} ({kind}): max error {error.max()}"


# seed 299: a dense slice that starts inside a 16-byte line (a generated kernel reads an aligned copy of it)
@pytest.mark.parametrize("seed", [*range(EXACT_SEEDS), *([299] if EXACT_SEEDS <= 299 else [])])
def test_programs_of_views_match_the_oracle_bit_for_bit(cuda, seed):
    """Reshapes, transposes, slices and concatenations between element-wise steps (all exactly defined): every result
    equals the oracle's bit for bit, whether a kernel reads the view, a copy step makes it dense or it is copied out."""
    recipe = R.draw_layout_recipe(seed)
    program, arrays = R.build_layout(recipe), R.draw_layout_inputs(recipe, seed)
    got = lumen_b200.compile(program, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
    want = run_oracle(tracer.trace(program, *[(recipe[0], s) for s in recipe[1]]), arrays)
    assert len(got) == len(want)
    for k, (g, w) in enumerate(zip(got, want)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        np.testing.assert_array_equal(bits(g), bits(w), err_msg=f"seed {seed} output {k}")


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_integer_programs_match_the_oracle_exactly(cuda, seed):
    """Wrapping add / sub / mul, division and remainder with their zero-divisor and overflow rules, bit operations, casts
    through float32 and through another integer type, comparisons, selects, and sums / maxima / minima over rows and
    columns (integer sums wrap, so their order does not matter): every result equals the oracle's."""
    recipe = R.draw_integer_recipe(seed)
    program, arrays = R.build_integer(recipe), R.draw_integer_inputs(recipe, seed)
    got = lumen_b200.compile(program, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
    want = run_oracle(tracer.trace(program, *[(recipe[1], recipe[0])] * recipe[3]), arrays)
    assert len(got) == len(want)
    for k, ((kind, _), g, w) in enumerate(zip(recipe[5], got, want)):
        assert g.shape == w.shape, f"seed {seed} output {k}"
        np.testing.assert_array_equal(bits(g), bits(w), err_msg=f"seed {seed} output {k} ({kind}, {recipe[1]})")


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_programs_that_reuse_their_reductions_are_as_accurate_as_the_oracle(cuda, seed):
    """Row sums, means and maxima combined again with the full tensor (one or two rounds, as in a layer normalisation),
    plus reductions over the first axis, the leading axes and everything. The oracle adds in index order and the kernels
    in trees, and what follows a cancelling sum amplifies the difference, so both are measured against the same program
    evaluated in float64: per output, the kernels' largest error is at most 4 times the oracle's plus 1e-6 (bfloat16
    programs: 2^-8) of the output's largest magnitude."""
    recipe = R.draw_reducing_recipe(seed)
    program, arrays = R.build_reducing(recipe), R.draw_reducing_inputs(recipe, seed)
    got = lumen_b200.compile(program, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
    want = run_oracle(tracer.trace(program, *R.reducing_input_types(recipe)), arrays)
    exact = (recipe[0], "float64", recipe[2], recipe[3])
    truth = run_oracle(tracer.trace(R.build_reducing(exact), *R.reducing_input_types(exact)), [a.astype(np.float64) for a in arrays])
    assert len(got) == len(want) == len(truth)
    floor = 2.0**-8 if recipe[1] == "bfloat16" else 1e-6
    for k, ((kind, _), g, w, t) in enumerate(zip(recipe[3], got, want, truth)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        t = t.astype(np.float64)
        assert np.isfinite(t).all() and np.isfinite(g.astype(np.float64)).all(), f"seed {seed} output {k}"
        ours, theirs = np.abs(g.astype(np.float64) - t).max(), np.abs(w.astype(np.float64) - t).max()
        assert ours <= 4 * theirs + floor * max(np.abs(t).max(), 1e-30), f"seed {seed} output {k} ({kind}): error {ours}, the oracle's {theirs}"


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_matrix_product_programs_are_as_accurate_as_the_oracle(cuda, seed):
    """`dot_general` over either axis of either operand, sizes from 1 to 1000 that are and are not multiples of the
    tiles or of a 16-byte row, bfloat16 and float32 operands, float32 accumulation, with a relu, a residual, an
    element-wise step or a second product behind it. Measured like the oracle against the float64 product of the same
    inputs: the largest error is at most 4 times the oracle's plus 1e-6 (bfloat16 results: 2^-8) of the largest value."""
    recipe = R.draw_gemm_recipe(seed)
    arrays = R.draw_gemm_inputs(recipe, seed)
    program = R.build_gemm(recipe)
    got = lumen_b200.compile(program, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = to_numpy(got)
    (want,) = run_oracle(tracer.trace(program, *R.gemm_input_types(recipe)), arrays)
    (truth,) = run_oracle(tracer.trace(R.build_gemm(recipe, exact=True), *[("float64", s) for _, s in R.gemm_input_types(recipe)]),
                          [a.astype(np.float64) for a in arrays])
    assert got.shape == want.shape and got.dtype == want.dtype
    floor = 2.0**-8 if recipe[1] == "bfloat16" else 1e-6
    ours, theirs = np.abs(got.astype(np.float64) - truth).max(), np.abs(want.astype(np.float64) - truth).max()
    assert ours <= 4 * theirs + floor * max(np.abs(truth).max(), 1e-30), f"seed {seed} {recipe}: error {ours}, the oracle's {theirs}"


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_differentiated_models_are_as_accurate_as_the_oracle(cuda, seed):
    """Two to four random layers (linear with and without relu, layer / RMS norm, residual MLP, SwiGLU, GELU, SiLU) under a
    mean-square or cross-entropy loss, differentiated by autograd with respect to every parameter, in float32: the loss
    and each gradient, measured like the oracle against the same step in float64 - the largest error at most 4 times the
    oracle's plus 2e-6 of the largest value."""
    recipe = R.draw_model_recipe(seed)
    arrays = R.draw_model_inputs(recipe, seed)
    step = R.build_model(recipe)
    got = lumen_b200.compile(step, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in got]
    want = run_oracle(tracer.trace(step, *R.model_input_types(recipe)), arrays)
    truth = run_oracle(tracer.trace(R.build_model(recipe, "float64"), *R.model_input_types(recipe, "float64")),
                       [a.astype(np.float64) if a.dtype == np.float32 else a for a in arrays])
    assert len(got) == len(want) == len(truth)
    for k, (g, w, t) in enumerate(zip(got, want, truth)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        assert np.isfinite(g).all(), f"seed {seed} output {k}"
        ours, theirs = np.abs(g.astype(np.float64) - t).max(), np.abs(w.astype(np.float64) - t).max()
        assert ours <= 4 * theirs + 2e-6 * max(np.abs(t).max(), 1e-30), f"seed {seed} output {k} of {recipe}: error {ours}, the oracle's {theirs}"


@pytest.mark.parametrize("seed", range(12))
def test_recorded_programs_replay_their_results(cuda, seed):
    """`compile(..., use_graphs=True)`: the plain run, the run that records the CUDA graph and two replays of it all give
    the oracle's bits for a program of exactly defined functions; new values in the same argument memory are picked up."""
    recipe = R.draw_recipe(seed + 1000, True)
    program, arrays = R.build(recipe), R.draw_inputs(recipe, seed)
    compiled = lumen_b200.compile(program, use_graphs=True)
    tensors = [to_torch(a, cuda) for a in arrays]
    graph = tracer.trace(program, *R.input_types(recipe))
    for call in range(4):
        if call == 3:  # other values in the same memory
            arrays = R.draw_inputs(recipe, seed + 500)
            for t, a in zip(tensors, arrays):
                t.copy_(to_torch(a, cuda))
        got = compiled(*tensors)
        device_status()
        got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
        want = run_oracle(graph, arrays)
        for k, ((kind, _), g, w) in enumerate(zip(recipe[4], got, want)):
            if kind in ("sum_last", "sum_first"):
                check_sum(kind, g, w, want[0], seed)
            elif w.dtype in (np.float32, BF16):
                nan = np.isnan(w.astype(np.float32))
                np.testing.assert_array_equal(bits(g)[~nan], bits(w)[~nan], err_msg=f"seed {seed} call {call} output {k}")
            else:
                np.testing.assert_array_equal(g, w, err_msg=f"seed {seed} call {call} output {k}")


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_optimizer_steps_over_odd_parameter_lists(cuda, seed):
    """SGD and AdamW over 2 - 24 parameters whose shapes share no row length (7, 1, 33 x 5, 300,007 ... elements), merged
    into one horizontally fused launch, with the learning rate / step count as a constant or as a 0-d operand. SGD's
    results and AdamW's moments are products, sums and roundings only: bit for bit. AdamW's new weights go through
    exp, a division and a square root: within 2e-6 (bfloat16 weights: one ulp) of the oracle's."""
    recipe = R.draw_optimizer_recipe(seed)
    kind, dtype, shapes, _ = recipe
    step, arrays = R.build_optimizer(recipe), R.draw_optimizer_inputs(recipe, seed)
    compiled = lumen_b200.compile(step, lowering="native" if seed % 3 else "optimising")
    # (a 0-d array becomes a 0-d tensor by hand: the shared helper goes through numpy's contiguous copy, which is 1-d)
    got = compiled(*[to_torch(a, cuda) if np.ndim(a) else torch.tensor(float(a), dtype=torch.float32, device=cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in got]
    want = run_oracle(tracer.trace(step, *R.optimizer_input_types(recipe)), arrays)
    assert len(got) == len(want)
    assert len(compiled.steps()) == 1  # one launch for all of them
    for k, (g, w) in enumerate(zip(got, want)):
        assert g.shape == w.shape and g.dtype == w.dtype
        if kind == "sgd" or k % 3 != 0:
            np.testing.assert_array_equal(bits(g), bits(w), err_msg=f"seed {seed} output {k} of {kind} {dtype} {shapes[k // (3 if kind == 'adamw' else 1)]}")
        else:
            rel = 2.0**-7 if dtype == "bfloat16" else 2e-6
            np.testing.assert_allclose(g.astype(np.float64), w.astype(np.float64), rtol=rel, atol=rel * 1e-2, err_msg=f"seed {seed} output {k}")


@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_indexing_programs_match_the_oracle_bit_for_bit(cuda, seed):
    """An embedding gather plus positions, then triangles, constant paddings, concatenations and stackings with scaled
    copies and clamps; the arg-maximum and arg-minimum over the last axis (first index on ties), a comparison with the
    ids and a one-hot product whose row sums have one non-zero term each: everything exactly the oracle's."""
    recipe = R.draw_indexing_recipe(seed)
    program, arrays = R.build_indexing(recipe), R.draw_indexing_inputs(recipe, seed)
    got = lumen_b200.compile(program, lowering="native" if seed % 3 else "optimising")(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in got]
    want = run_oracle(tracer.trace(program, *R.indexing_input_types(recipe)), arrays)
    assert len(got) == len(want)
    for k, (g, w) in enumerate(zip(got, want)):
        assert g.shape == w.shape, f"seed {seed} output {k}"
        np.testing.assert_array_equal(bits(g), bits(w), err_msg=f"seed {seed} output {k} of {recipe}")


@pytest.mark.parametrize("dtype", ["float16", "float64"])
@pytest.mark.parametrize("seed", range(EXACT_SEEDS))
def test_float16_and_float64_programs_match_the_oracle_bit_for_bit(cuda, seed, dtype):
    """The exactly defined element-wise programs in the generated kernels' other float types. float16: every primitive
    computes in float32 and rounds once, as the oracle does (row sums are taken of the float32 widening); float64:
    computed in float64 throughout. Sums are held like the float32 programs'."""
    recipe = R.in_dtype(R.draw_recipe(seed + 2000, True), dtype)
    program, arrays = R.build(recipe), R.draw_inputs(recipe, seed)
    got = lumen_b200.compile(program)(*[to_torch(a, cuda) for a in arrays])
    device_status()
    got = [to_numpy(t) for t in (got if isinstance(got, tuple) else (got,))]
    want = run_oracle(tracer.trace(program, *R.input_types(recipe)), arrays)
    assert len(got) == len(want)
    for k, ((kind, _), g, w) in enumerate(zip(recipe[4], got, want)):
        assert g.shape == w.shape and g.dtype == w.dtype, f"seed {seed} output {k}"
        if kind in ("sum_last", "sum_first"):
            check_sum(kind, g, w, want[0], seed)
        elif w.dtype.kind == "f":
            nan = np.isnan(w.astype(np.float64))
            np.testing.assert_array_equal(np.isnan(g.astype(np.float64)), nan, err_msg=f"seed {seed} output {k}: NaN places")
            np.testing.assert_array_equal(bits(g)[~nan], bits(w)[~nan], err_msg=f"seed {seed} output {k} ({kind})")
        else:
            np.testing.assert_array_equal(g, w, err_msg=f"seed {seed} output {k} ({kind})")
