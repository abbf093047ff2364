"""`lb_compile`, the backend's own C++ lowering of a module that has been through the passes (the counterpart of
`Cuda::lower(module, device)`, lumen/graph_compiler/device.rs:88-112): on the CPU it parses the module, generates and
compiles every fused kernel and builds the plan - steps, places, workspace size - or rejects the module with a message
naming the primitive it has no kernel for (lumen/codegen/devices/cuda/mod.rs:140-189 does the same)."""

import json

import pytest

from lumen_b200 import _lib, autograd, tracer
from lumen_b200 import functional as F
from lumen_b200.attention_pass import match_attention
from lumen_b200.fusion_pass import fuse
from lumen_b200.plan import _bind, lower_native
from lumen_b200.simplify import clean


def plan_of(graph, **kwargs):
    handle = lower_native(graph, **kwargs)
    lib = _bind()
    steps = [(s["kind"], s["label"]) for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
    workspace = lib.lb_plan_workspace_bytes(handle)
    lib.lb_plan_destroy(handle)
    return steps, workspace


def chain(x, g, b):
    y = F.relu(x * g + b)
    return y, F.sum(y * y, 1)


CHAIN_TYPES = (("float32", (64, 256)), ("float32", (256,)), ("float32", (256,)))


def test_fused_chain_is_one_step_written_into_the_outputs():
    steps, workspace = plan_of(fuse(clean(tracer.trace(chain, *CHAIN_TYPES))))
    assert steps == [("fusion", "row")] and workspace == 0  # both results are graph outputs: nothing lives in the workspace


def test_products_become_gemm_steps_with_their_relu():
    def mlp(x, w1, w2):
        return F.matmul(F.relu(F.matmul(x, w1, "float32", "bfloat16")), w2, "float32", "bfloat16")

    g = fuse(clean(tracer.trace(mlp, ("bfloat16", (256, 128)), ("bfloat16", (128, 512)), ("bfloat16", (512, 64)))))
    steps, workspace = plan_of(g)
    assert [k for k, _ in steps] == ["gemm", "gemm"]
    assert workspace == 256 * 512 * 2  # the hidden activation; the result is produced in the output


def test_intermediates_share_the_workspace_by_live_range():
    """A chain of four products: each intermediate is dead once the next product has read it, so the workspace holds two
    of the three at a time - the size the optimising lowering gives the same module."""
    from lumen_b200.compiler import compile_graph

    def chain4(x, a, b, c, d):
        for w in (a, b, c, d):
            x = F.matmul(x, w, "float32", "bfloat16")
        return x

    types = [("bfloat16", (512, 256))] + [("bfloat16", (256, 256))] * 4
    g = tracer.trace(chain4, *types)
    _, workspace = plan_of(fuse(clean(g)))
    assert workspace == 2 * 512 * 256 * 2 == compile_graph(g).workspace_bytes


def test_attention_forward_and_backward_with_and_without_determinism():
    def program(q, k, v, do):
        def loss(q_, k_, v_):
            return F.sum(F.flash_attention(q_, k_, v_, causal=True)[0].float() * do.float())

        value, grads = autograd.value_and_grad(loss, (0, 1, 2))(q, k, v)
        return (value, *grads)

    g = fuse(match_attention(clean(tracer.trace(program, *[("bfloat16", (2, 128, 4, 64))] * 4))))
    steps, pair = plan_of(g)
    assert [k for k, _ in steps].count("attn_fwd") == 1 and [k for k, _ in steps].count("attn_bwd") == 1
    _, atomic = plan_of(g, deterministic=False)
    assert atomic >= pair  # the float32 dQ accumulator of the single-kernel backward lives (only) at the backward step


def test_attention_written_from_prims_is_lowered_after_the_matcher():
    g = match_attention(clean(tracer.trace(lambda q, k, v: F.attention_forward_prims(q, k, v, 0.125, True)[0], *[("bfloat16", (2, 128, 4, 64))] * 3)))
    steps, _ = plan_of(fuse(g))
    assert steps == [("attn_fwd", "flash_attention")]


def test_a_module_that_skipped_the_fusion_pass_is_rejected_by_primitive():
    with pytest.raises(_lib.LumenError, match="primitive `broadcast_in_dim` outside a fusion"):
        lower_native(tracer.trace(chain, *CHAIN_TYPES))
    with pytest.raises(_lib.LumenError):
        _lib.check(_bind().lb_compile(b"not a module", -1, None, None))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_whole_training_step_is_lowered(dtype):
    """Forward, backward and SGD update of the transformer step as the passes leave it: generated kernels, products with
    their relu / residual-add / relu-backward epilogues, attention forward and backward on sliced views of the packed
    projection, the embedding's scatter-add, the attention gradients produced inside the concatenation that packs them."""
    from lumen_b200 import transformer as T

    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=1, seq=128, dtype=dtype)
    g, _, _ = T.trace_train_step(cfg, 2)
    steps, workspace = plan_of(fuse(match_attention(clean(g))))
    kinds = [k for k, _ in steps]
    assert kinds.count("gemm") == 15 and kinds.count("attn_fwd") == 1 and kinds.count("attn_bwd") == 1 and kinds.count("scatter_add") == 1
    assert kinds.count("copy") == 0 and workspace > 0  # the attention gradients are produced inside their concatenation
    assert kinds.count("multi") == 1 and [label for k, label in steps if k == "multi"] == ["sgd_update_x13"]  # the 13 updates as one launch


def test_the_data_parallel_step_gets_its_collective_steps():
    """The 2-rank training step: all-reduced gradients side by side in the arena, cut into buckets, each with an
    `all_reduce` step after its last gradient and a `wait` before its first reader - as many collectives, in the same
    places, and the same workspace as the Python lowering gives the same module."""
    from lumen_b200 import transformer as T
    from lumen_b200.compiler import compile_graph

    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=1, seq=128, dtype="bfloat16")
    g, _, donate = T.trace_train_step(cfg, 2, world=2)
    handle = lower_native(fuse(match_attention(clean(g))), True, donate, 100_000)
    lib = _bind()
    kinds = [s["kind"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
    python = compile_graph(g, donate, bucket_bytes=100_000)
    python_kinds = [line.split()[1] for line in python.text.splitlines() if line.startswith("s ")]

    def places(ks):  # (kind, number of kernel steps before it) of every collective step
        out, n = [], 0
        for k in ks:
            if k in ("all_reduce", "wait"):
                out.append((k, n))
            elif k not in ("copy", "fill", "transpose"):
                n += 1
        return out

    assert lib.lb_plan_num_collectives(handle) == len(python.buckets) == 3
    assert places(kinds) == places(python_kinds)
    assert lib.lb_plan_workspace_bytes(handle) == python.workspace_bytes
    lib.lb_plan_destroy(handle)


def test_a_concatenation_of_other_values_is_copied_into_place():
    """Operands that are not attention gradients (here two products) are copied into the concatenation by pitched
    copies."""
    def program(x, a, b):
        return F.cat([F.matmul(x, a, "float32", "bfloat16"), F.matmul(x, b, "float32", "bfloat16")], 1)

    g = fuse(clean(tracer.trace(program, ("bfloat16", (256, 128)), ("bfloat16", (128, 64)), ("bfloat16", (128, 192)))))
    steps, _ = plan_of(g)
    assert [k for k, _ in steps] == ["gemm", "gemm", "copy", "copy"]


def test_both_lowerings_make_the_same_steps_of_a_differentiated_program():
    """A SwiGLU MLP step differentiated by autograd returns its weight gradients as transposed views of the products
    that made them: `lb_compile` writes them into the outputs with the transpose kernel, names every product by its
    epilogue and needs the same workspace as the Python lowering of the same program; the plan keeps its own text."""
    from lumen_b200.compiler import compile_graph

    def step(x, y, gate, up, down):
        def loss(g, u, d):
            h = F.swiglu(F.matmul(x, g, "float32", "float32"), F.matmul(x, u, "float32", "float32"))
            r = F.matmul(h, d, "float32", "float32") - y
            return F.mean(r * r)

        value, grads = autograd.value_and_grad(loss, (0, 1, 2))(gate, up, down)
        return (value, *grads)

    types = [("float32", s) for s in ((256, 64), (256, 32), (64, 128), (64, 128), (128, 32))]
    g = tracer.trace(step, *types)
    python = compile_graph(g)
    handle = lower_native(fuse(match_attention(clean(g))))
    lib = _bind()
    labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
    assert labels == python.labels and labels.count("output_transpose") == 3
    assert lib.lb_plan_workspace_bytes(handle) == python.workspace_bytes
    text = lib.lb_plan_text(handle).decode()
    assert text.count("\ns transpose output_transpose ") == 3 and text.rstrip().endswith("end")
    lib.lb_plan_destroy(handle)


def test_both_lowerings_place_the_same_collectives_in_random_data_parallel_steps():
    """Random configurations (1 - 3 layers, float32 and bfloat16, SGD and AdamW), world sizes 2 - 8 and bucket sizes from
    one gradient per bucket to everything in one: both lowerings queue as many collectives, at the same places among the
    kernel steps, make the same steps and need the same workspace."""
    import numpy as np

    from lumen_b200 import transformer as T
    from lumen_b200.compiler import compile_graph

    lib = _bind()

    def places(ks):
        out, n = [], 0
        for k in ks:
            if k in ("all_reduce", "wait"):
                out.append((k, n))
            elif k not in ("copy", "fill", "transpose"):
                n += 1
        return out

    for seed in range(8):
        rng = np.random.default_rng(seed + 300)
        dtype = ["float32", "bfloat16"][int(rng.integers(2))]
        d = int(rng.choice([64, 128]))
        cfg = T.Config(vocab=int(rng.choice([64, 200])), d_model=d, heads=d // 64 if dtype == "bfloat16" else int(rng.choice([2, 4])),
                       hidden=int(rng.choice([128, 256])), layers=int(rng.integers(1, 4)), seq=int(rng.choice([64, 128])), dtype=dtype,
                       optimizer=["sgd", "adamw"][int(rng.integers(2))])
        world = int(rng.choice([2, 4, 8]))
        bucket = int(rng.choice([1, 50_000, 400_000, 1 << 30]))
        g, _, donate = T.trace_train_step(cfg, 2, world=world)
        handle = lower_native(fuse(match_attention(clean(g))), True, donate, bucket)
        steps = json.loads(lib.lb_plan_steps_json(handle).decode())
        python = compile_graph(g, donate, bucket_bytes=bucket)
        python_kinds = [line.split()[1] for line in python.text.splitlines() if line.startswith("s ")]
        what = (seed, cfg, world, bucket)
        assert lib.lb_plan_num_collectives(handle) == len(python.buckets) >= 1, what
        assert places([s["kind"] for s in steps]) == places(python_kinds), what
        assert [s["label"] for s in steps] == python.labels, what
        assert lib.lb_plan_workspace_bytes(handle) == python.workspace_bytes, what
        lib.lb_plan_destroy(handle)
