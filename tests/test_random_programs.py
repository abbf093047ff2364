"""Seeded random programs (tests/random_programs.py) on the CPU: the oracle evaluates each one, and `lb_compile` and the
Python lowering make the same steps with the same workspace of it."""

import json

import pytest

from lumen_b200 import tracer
from lumen_b200.attention_pass import match_attention
from lumen_b200.compiler import compile_graph
from lumen_b200.fusion_pass import fuse
from lumen_b200.plan import _bind, lower_native
from lumen_b200.simplify import clean
from tests import random_programs as R
from tests.helpers import run_oracle


@pytest.mark.parametrize("exact", [True, False])
def test_both_lowerings_agree_on_random_programs(exact):
    lib = _bind()
    for seed in range(12):
        recipe = R.draw_recipe(seed, exact)
        g = tracer.trace(R.build(recipe), *R.input_types(recipe))
        results = run_oracle(g, R.draw_inputs(recipe, seed))
        assert [tuple(r.shape) for r in results] == [tuple(g.types[v].shape) for v in g.outputs], seed
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels, seed
        assert workspace == python.workspace_bytes, seed


def test_both_lowerings_agree_on_programs_of_views():
    """Reshapes, transposes, slices and concatenations between element-wise steps: both lowerings accept every program
    (views that a kernel cannot read as they are become copy steps) and make the same steps with the same workspace."""
    lib = _bind()
    copies = 0
    for seed in range(24):
        recipe = R.draw_layout_recipe(seed)
        g = tracer.trace(R.build_layout(recipe), *[(recipe[0], s) for s in recipe[1]])
        run_oracle(g, R.draw_layout_inputs(recipe, seed))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels, seed
        assert workspace == python.workspace_bytes, seed
        copies += labels.count("materialize_view")
    assert copies > 0  # the sample does reach the strided copies


def test_both_lowerings_agree_on_integer_programs():
    lib = _bind()
    for seed in range(16):
        recipe = R.draw_integer_recipe(seed)
        g = tracer.trace(R.build_integer(recipe), *[(recipe[1], recipe[0])] * recipe[3])
        run_oracle(g, R.draw_integer_inputs(recipe, seed))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels and workspace == python.workspace_bytes, seed


def test_both_lowerings_agree_on_programs_that_reuse_their_reductions():
    """Includes a value returned twice (seed 34): produced in its first output and copied to the second by both."""
    lib = _bind()
    for seed in list(range(12)) + [34]:
        recipe = R.draw_reducing_recipe(seed)
        g = tracer.trace(R.build_reducing(recipe), *R.reducing_input_types(recipe))
        run_oracle(g, R.draw_reducing_inputs(recipe, seed))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels and workspace == python.workspace_bytes, seed


def test_both_lowerings_agree_on_matrix_product_programs():
    lib = _bind()
    for seed in range(24):
        recipe = R.draw_gemm_recipe(seed)
        g = tracer.trace(R.build_gemm(recipe), *R.gemm_input_types(recipe))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels and workspace == python.workspace_bytes, (seed, recipe)


def test_both_lowerings_agree_on_differentiated_models():
    lib = _bind()
    for seed in range(8):
        recipe = R.draw_model_recipe(seed)
        g = tracer.trace(R.build_model(recipe), *R.model_input_types(recipe))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels and workspace == python.workspace_bytes, (seed, recipe)


def test_both_lowerings_merge_optimizer_steps_over_odd_parameter_lists():
    lib = _bind()
    for seed in range(10):
        recipe = R.draw_optimizer_recipe(seed)
        g = tracer.trace(R.build_optimizer(recipe), *R.optimizer_input_types(recipe))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        lib.lb_plan_destroy(handle)
        assert labels == python.labels == [f"{recipe[0]}_update_x{len(recipe[2])}"], (seed, labels)


def test_both_lowerings_agree_on_indexing_programs():
    """Includes paddings with a non-zero value (a constant outside any fusion: a generated kernel without operands) and
    concatenations of element-wise results (copied into place by both)."""
    lib = _bind()
    constants = 0
    for seed in range(16):
        recipe = R.draw_indexing_recipe(seed)
        g = tracer.trace(R.build_indexing(recipe), *R.indexing_input_types(recipe))
        run_oracle(g, R.draw_indexing_inputs(recipe, seed))
        python = compile_graph(g)
        handle = lower_native(fuse(match_attention(clean(g))))
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        workspace = lib.lb_plan_workspace_bytes(handle)
        lib.lb_plan_destroy(handle)
        assert labels == python.labels and workspace == python.workspace_bytes, (seed, recipe)
        constants += labels.count("constant")
    assert constants > 0
