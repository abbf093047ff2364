"""The backend's own runtime layer on a GPU: the region allocator (one reservation, first fit, coalescing, hold /
release), streams and events, pinned copies, and running a fused kernel on region memory with torch out of the
picture for the product call (lumen/allocator/region.rs, lumen/runtime/stream/cuda.rs)."""

import numpy as np
import pytest

from lumen_b200 import _lib, device as D
from lumen_b200.runtime import Fusion

pytestmark = pytest.mark.gpu


def test_region_reserves_once_and_reuses_freed_blocks(cuda):
    free_before, _ = D.memory_info()
    region = D.Region(64 << 20)
    assert D.memory_info()[0] == free_before  # nothing reserved until the first block is taken
    a = region.alloc(1000)
    free_reserved, _ = D.memory_info()
    assert free_before - free_reserved >= 64 << 20
    b = region.alloc(5 << 20)
    c = region.alloc(300, alignment=4096)
    assert a % 256 == 0 and b % 256 == 0 and c % 4096 == 0 and len({a, b, c}) == 3
    assert D.memory_info()[0] == free_reserved  # later blocks are host bookkeeping only
    stats = region.stats()
    assert stats["live_bytes"] == 1024 + (5 << 20) + 512 and stats["capacity"] == 64 << 20
    region.free(b)
    again = region.alloc(4 << 20)
    assert again == b  # first fit: the freed hole is reused
    region.free(again), region.free(a), region.free(c)
    assert region.stats()["live_bytes"] == 0 and region.stats()["largest_free"] == 64 << 20  # neighbours coalesced
    with pytest.raises(_lib.LumenError, match="out of memory"):
        region.alloc(65 << 20)
    with pytest.raises(_lib.LumenError, match="not a live block"):
        region.free(a)


def test_blocks_freed_on_hold_return_at_release(cuda):
    region = D.Region(8 << 20)
    a = region.alloc(4 << 20)
    region.hold()  # e.g. a recorded graph launches into `a`
    region.free(a)
    with pytest.raises(_lib.LumenError, match="out of memory"):
        region.alloc(6 << 20)
    region.release()
    assert region.alloc(6 << 20) == a


def test_a_fused_kernel_runs_on_region_memory_with_native_streams_and_events(cuda):
    from bench import chain_graph, chain_inputs
    from oracle import oracle

    rows, cols = 512, 2048
    g = chain_graph(rows, cols, "float32")
    x, gg, b = chain_inputs(rows, cols, "float32")
    region = D.Region(64 << 20)
    stream = D.Stream()
    tensors = [region.empty(a.shape, "float32") for a in (x, gg, b)]
    pinned = D.HostBuffer(x.nbytes)
    pinned.array(np.float32, x.shape)[...] = x
    tensors[0].copy_from_host(pinned, stream)  # asynchronous from pinned memory
    tensors[1].copy_from_host(gg, stream)
    tensors[2].copy_from_host(b, stream)
    start, stop = D.Event(timing=True), D.Event(timing=True)
    start.record(stream)
    y, s = Fusion(g)(*tensors, stream=stream.handle)
    stop.record(stream)
    stream.synchronize()
    assert isinstance(y, D.Tensor) and 0.0 < start.elapsed_ms(stop) < 1000.0
    want_y, want_s = oracle.run(g, [x, gg, b])
    np.testing.assert_array_equal(y.numpy(), want_y)
    np.testing.assert_allclose(s.numpy(), want_s, rtol=1e-5)
    # the same memory seen by a harness framework, without a copy
    import torch

    seen = torch.as_tensor(y, device="cuda")
    assert seen.data_ptr() == y.data_ptr() and torch.equal(seen.cpu(), torch.from_numpy(want_y))


def test_horizontal_launch_matches_separate_launches(cuda):
    """`lb_fusion_launch_groups`: one kernel over several (parameter, gradient) pairs of different sizes gives what one
    launch per pair gives, bit for bit (bfloat16 SGD update, in place)."""
    import torch

    from lumen_b200 import transformer as T
    from lumen_b200.compiler import compile_graph
    from lumen_b200.plan import Plan

    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16", lr=0.1)
    g, names, donate = T.trace_train_step(cfg, 2)
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, cfg.vocab, (2, cfg.seq + 1)).astype(np.int64)
    results = []
    for horizontal in (False, True):
        compiled = compile_graph(g, donate, horizontal=horizontal)
        assert ("multi" in [line.split()[1] for line in compiled.text.splitlines() if line.startswith("s ")]) == horizontal
        params = [torch.from_numpy(T.init_params(cfg, 0)[n]).cuda().bfloat16() for n in names]
        loss = torch.zeros((), device="cuda")
        ids = torch.from_numpy(np.ascontiguousarray(tokens[:, :-1])).cuda()
        targets = torch.from_numpy(np.ascontiguousarray(tokens[:, 1:])).cuda()
        plan = Plan(compiled)
        for _ in range(2):
            plan.run([ids, targets, *params], [loss, *params])
        torch.cuda.synchronize()
        results.append((float(loss), [p.view(torch.int16).cpu() for p in params]))
        assert compiled.kernel_launches < 200
    assert results[0][0] == results[1][0]
    for a, b in zip(results[0][1], results[1][1]):
        assert torch.equal(a, b)


def test_autotuned_plan_gives_the_same_results(cuda):
    """`lb_plan_autotune` on a plan with one large GEMM (2^30 multiply-adds and a long K, so that K splits are among the
    candidates): it reports what it timed and picked, and the tuned plan's product equals the untuned one's to the
    order of float32 sums."""
    import torch

    from lumen_b200 import prims, tracer
    from lumen_b200.compiler import compile_graph
    from lumen_b200.plan import Plan

    m, n, k = 1024, 1024, 8192
    g = tracer.trace(lambda a, b: prims.dot_general(a, b, (((1,), (0,)), ((), ())), "float32", "float32"), ("bfloat16", (m, k)), ("bfloat16", (k, n)))
    gen = torch.Generator(device="cpu").manual_seed(0)
    a = (torch.randn((m, k), generator=gen) / k**0.5).bfloat16().cuda()
    b = torch.randn((k, n), generator=gen).bfloat16().cuda()
    outs = []
    for tune in (False, True):
        plan = Plan(compile_graph(g))
        out = torch.full((m, n), float("nan"), device="cuda")
        bound = plan.bind([a, b], [out])
        if tune:
            report = plan.autotune(bound)
            assert len(report) == 1 and report[0]["candidates"] >= 4 and report[0]["us"] <= report[0]["default_us"] * 1.01
            assert set(report[0]["picked"]) == {"kernel", "splits", "group_m"}
        plan.run_bound(bound)
        torch.cuda.synchronize()
        outs.append(out)
    want = a.float() @ b.float()
    for out in outs:
        torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-4)
