"""The traced training step on the CPU: its hand-derived backward against PyTorch autograd in float64 (through the
oracle), and its lowering to a plan."""

import numpy as np
import pytest

from lumen_b200 import transformer as T
from lumen_b200.compiler import compile_graph, reshape_view
from oracle import oracle
from tests.helpers import BF16, run_oracle
from tests.model_reference import torch_step


def batch_of(cfg, batch, seed=0):
    """`t = rng.integers(0, vocab, (batch, seq + 1))`; inputs `t[:, :-1]`, next-token targets `t[:, 1:]`."""
    t = np.random.default_rng(seed).integers(0, cfg.vocab, (batch, cfg.seq + 1))
    return np.ascontiguousarray(t[:, :-1]), np.ascontiguousarray(t[:, 1:])


def test_traced_step_matches_torch_autograd():
    cfg = T.Config(vocab=32, d_model=32, heads=2, hidden=64, layers=2, seq=16, dtype="float32", lr=0.1)
    batch = 3
    params = T.init_params(cfg, seed=0)
    # make layer norm scales and biases non-trivial so their gradients are exercised
    rng = np.random.default_rng(1)
    for k in params:
        if k.endswith("norm.w") or k.endswith("norm.b"):
            params[k] = (params[k] + 0.1 * rng.standard_normal(params[k].shape)).astype(np.float32)
        else:
            params[k] = (params[k] * 10).astype(np.float32)
    ids, targets = batch_of(cfg, batch)
    g, names, _ = T.trace_train_step(cfg, batch, with_grads=True)
    outs = oracle.run(g, [ids, targets] + [params[n] for n in names])
    loss, updated, grads = outs[0], outs[1 : 1 + len(names)], outs[1 + len(names) :]
    want_loss, want_grads = torch_step(cfg, params, ids, targets)
    assert abs(float(loss) - want_loss) <= 1e-5 * abs(want_loss)
    for n, got, new in zip(names, grads, updated):
        want = want_grads[n]
        scale = max(np.abs(want).max(), 1e-8)
        assert np.abs(got - want).max() <= 2e-4 * scale, n
        np.testing.assert_allclose(new, params[n] - np.float32(cfg.lr) * got, rtol=1e-6, atol=1e-7)


def test_step_lowers_to_a_plan():
    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16")
    g, names, donate = T.trace_train_step(cfg, 2, world=2)
    plan = compile_graph(g, donate)
    labels = plan.labels
    assert labels.count("flash_attention") == cfg.layers and labels.count("flash_attention_backward") == cfg.layers
    gemms = sum(labels.count(x) for x in ("dot_general", "dot_general_relu", "dot_general_add", "dot_general_relu_backward"))
    assert gemms == 3 * (4 * cfg.layers + 1)
    # 16-bit models fold the residual adds and the relu's backward into GEMM epilogues
    assert labels.count("dot_general_add") == 2 * cfg.layers and labels.count("dot_general_relu_backward") == cfg.layers
    assert "residual_add" not in labels and "relu_backward" not in labels
    # the per-parameter updates are horizontally fused: one launch per run between the buckets' waits
    fused = [x for x in labels if x.startswith("sgd_update")]
    assert sum(int(x.rsplit("_x", 1)[1]) if "_x" in x else 1 for x in fused) == len(names) and len(fused) < len(names)
    assert compile_graph(g, donate, horizontal=False).labels.count("sgd_update") == len(names)
    assert labels.count("all_reduce") == len(plan.buckets) == labels.count("device_wait")
    # every weight gradient is all-reduced, from one contiguous arena at the start of the workspace
    assert len(plan.comms) == len(names)
    spans = sorted((c.view.buffer.offset, c.view.buffer.nbytes) for c in plan.comms)
    assert spans[0][0] == 0 and all(a[0] + -(-a[1] // 256) * 256 == b[0] for a, b in zip(spans, spans[1:]))
    assert plan.arena_bytes >= sum(n for _, n in spans)
    assert plan.workspace_bytes % 256 == 0


def test_reshape_views():
    assert reshape_view((6, 4), (12, 1), (2, 3, 2, 2)) == (36, 12, 2, 1)
    assert reshape_view((6, 4), (4, 1), (24,)) == (1,)
    assert reshape_view((6, 4), (12, 1), (24,)) is None
    assert reshape_view((2, 3, 4), (12, 4, 1), (6, 4)) == (4, 1)
    assert reshape_view((5, 1, 4), (4, 4, 1), (5, 4)) == (4, 1)


def test_adamw_step_matches_float64_from_the_same_gradients():
    """The AdamW training step on the oracle: its updated weights and moments equal the float64 AdamW formulas
    (examples/optim.py:63-80) applied to the gradients the same graph returns, for the first and for a later step."""
    cfg = T.Config(vocab=64, d_model=32, heads=2, hidden=64, layers=1, seq=16, optimizer="adamw", lr=1e-2, weight_decay=0.1)
    g, names, donate = T.trace_train_step(cfg, 2, with_grads=True)
    n = len(names)
    assert donate == {1 + k: 2 + k for k in range(3 * n)}
    params = T.init_params(cfg, 0)
    ids, targets = batch_of(cfg, 2)
    rng = np.random.default_rng(1)
    for step, warm in ((1.0, False), (7.0, True)):
        m = [(1e-3 * rng.standard_normal(params[k].shape)).astype(np.float32) if warm else np.zeros(params[k].shape, np.float32) for k in names]
        v = [rng.uniform(0, 1e-6, params[k].shape).astype(np.float32) if warm else np.zeros(params[k].shape, np.float32) for k in names]
        out = oracle.run(g, [ids, targets] + [params[k] for k in names] + m + v + [np.array(step, np.float32)])
        assert len(out) == 1 + 4 * n
        b1, b2 = 0.9, 0.999
        for k, name in enumerate(names):
            grad = out[1 + 3 * n + k].astype(np.float64)
            m64, v64 = b1 * m[k] + (1 - b1) * grad, b2 * v[k] + (1 - b2) * grad * grad
            want = params[name].astype(np.float64) * (1 - cfg.lr * cfg.weight_decay) - cfg.lr * (m64 / (1 - b1**step)) / (np.sqrt(v64 / (1 - b2**step)) + 1e-8)
            np.testing.assert_allclose(out[1 + n + k], m64, rtol=1e-5, atol=1e-10, err_msg=name)
            np.testing.assert_allclose(out[1 + 2 * n + k], v64, rtol=1e-5, atol=1e-14, err_msg=name)
            np.testing.assert_allclose(out[1 + k], want, rtol=2e-5, atol=1e-6, err_msg=name)


def test_runtime_learning_rate_traces_the_same_arithmetic():
    """The step traced with the learning rate as a 0-d float32 input (the reference's run-time optimizer scalars,
    lumen/codegen/devices/cuda/mod.rs:197-200) gives, on the oracle, bit for bit what the step with the constant gives;
    another rate gives what a step traced with that constant gives."""
    cfg = T.Config(vocab=64, d_model=32, heads=2, hidden=64, layers=1, seq=16)
    params = T.init_params(cfg, 0)
    ids, targets = batch_of(cfg, 2)
    for dtype in ("float32", "bfloat16"):
        cfg.dtype = dtype
        cast = (lambda a: a.astype(BF16)) if dtype == "bfloat16" else (lambda a: a)
        g_rt, names, _ = T.trace_train_step(cfg, 2, runtime_lr=True)
        args = [ids, targets] + [cast(params[n]) for n in names]
        for lr in (cfg.lr, 0.37):
            fixed = T.Config(**{**cfg.__dict__, "lr": lr})
            g_const, _, _ = T.trace_train_step(fixed, 2)
            want = run_oracle(g_const, args)
            got = run_oracle(g_rt, args + [np.float32(lr)])
            for a, b in zip(got, want):
                assert np.asarray(a).tobytes() == np.asarray(b).tobytes()
    with pytest.raises(ValueError):
        T.trace_train_step(T.Config(vocab=64, d_model=32, heads=2, hidden=64, layers=1, seq=16, optimizer="adamw"), 2, runtime_lr=True)


def test_the_backend_accepts_the_plan_without_a_gpu():
    """`lb_plan_create` parses the plan text and generates + compiles (NVRTC) every fused kernel in it - the
    horizontally fused update and the collective steps included - with no device present."""
    import ctypes

    from lumen_b200 import _lib
    from lumen_b200.plan import _bind

    lib = _bind()
    small = dict(vocab=64, d_model=32, heads=2, hidden=64, layers=1, seq=16)
    for cfg, world, runtime_lr in ((T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=1, seq=128, dtype="bfloat16"), 2, False),
                                   (T.Config(**small), 1, False),
                                   (T.Config(**small), 1, True),                        # the learning rate as a 0-d operand
                                   (T.Config(**small, optimizer="adamw"), 1, False)):   # the step count as a 0-d operand
        g, names, donate = T.trace_train_step(cfg, 2, world=world, runtime_lr=runtime_lr)
        plan = compile_graph(g, donate, bucket_bytes=100_000)
        if world == 1:  # the per-parameter updates are ONE horizontally fused step, 0-d operands included
            assert sum(label.startswith(("sgd_update_x", "adamw_update_x")) for label in plan.labels) == 1
        handle = ctypes.c_void_p()
        _lib.check(lib.lb_plan_create(plan.text.encode(), ctypes.byref(handle)))
        assert lib.lb_plan_num_steps(handle) == len(plan.labels)
        assert lib.lb_plan_num_collectives(handle) == len(plan.buckets)
        lib.lb_plan_destroy(handle)
