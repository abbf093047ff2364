"""Data parallelism on CPU ranks: the gradient buckets and the collective steps of the plan, and a world-size-2 gloo
run of the all-reduce + update semantics against the single-rank step on the whole batch."""

import os
import subprocess
import sys

import numpy as np

from lumen_b200 import transformer as T
from lumen_b200.compiler import compile_graph, gradient_buckets
from tests.test_train_step import batch_of

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_buckets_cover_the_arena_in_production_order():
    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=3, seq=128, dtype="bfloat16")
    g, names, donate = T.trace_train_step(cfg, 2, world=4)
    plan = compile_graph(g, donate, bucket_bytes=200_000)
    buckets = plan.buckets
    assert buckets == gradient_buckets(plan, bucket_bytes=200_000) or len(buckets) == len(gradient_buckets(plan, bucket_bytes=200_000))
    assert len(buckets) > 2
    spans = sorted((b["start"], b["end"]) for b in buckets)
    assert spans[0][0] == 0 and spans[-1][1] == plan.arena_bytes
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert [b["ready"] for b in buckets] == sorted(b["ready"] for b in buckets)
    # the head's gradient is produced first in the backward pass, the embedding's last
    assert buckets[0]["start"] == 0
    one = compile_graph(g, donate, bucket_bytes=1 << 40).buckets
    assert len(one) == 1 and one[0]["end"] == plan.arena_bytes


def plan_steps(plan):
    return [line.split() for line in plan.text.splitlines() if line.startswith("s ")]


def test_collectives_are_plan_steps_in_the_right_places():
    """One `all_reduce` step per bucket, queued after the step that produces the bucket's last gradient and before
    any step of the update; its `wait` comes before the first step that reads one of its gradients and after the
    collective; the per-parameter updates between two waits are ONE horizontally fused launch."""
    cfg = T.Config(vocab=64, d_model=128, heads=2, hidden=256, layers=3, seq=128, dtype="bfloat16")
    g, names, donate = T.trace_train_step(cfg, 2, world=4)
    plan = compile_graph(g, donate, bucket_bytes=200_000)
    steps = plan_steps(plan)
    kinds = [s[1] for s in steps]
    n = len(plan.buckets)
    assert kinds.count("all_reduce") == n and kinds.count("wait") == n
    reduce_at = [k for k, s in enumerate(steps) if s[1] == "all_reduce"]
    wait_at = {int(s[3]): k for k, s in enumerate(steps) if s[1] == "wait"}
    assert sorted(wait_at) == list(range(n))
    for number, at in enumerate(reduce_at):
        assert at < wait_at[number]  # a wait follows its own collective
    updates = [k for k, s in enumerate(steps) if "sgd_update" in s[2]]
    assert min(updates) > max(reduce_at)  # every collective is queued before the first update
    assert min(wait_at.values()) < min(updates)
    # horizontal fusion: far fewer update launches than parameters, every parameter updated exactly once
    groups = sum(int(s[4]) if s[1] == "multi" else 1 for s in steps if "sgd_update" in s[2])
    assert groups == len(names) and len(updates) <= n + 2
    # without collectives (one rank) every update is one launch
    single = compile_graph(*T.trace_train_step(cfg, 2)[::2])
    multi = [s for s in plan_steps(single) if s[1] == "multi"]
    assert len(multi) == 1 and int(multi[0][4]) == len(names)


def test_adamw_step_keeps_the_same_buckets():
    """The optimizer does not change what is reduced: the AdamW variant's gradient arena and buckets equal the SGD
    step's, and every parameter gets one update kernel that scales the summed gradient by 1 / world."""
    base = dict(vocab=64, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16")
    plans = {}
    for opt in ("sgd", "adamw"):
        g, names, donate = T.trace_train_step(T.Config(optimizer=opt, **base), 2, world=4)
        plans[opt] = compile_graph(g, donate, horizontal=False)
        assert plans[opt].labels.count(f"{opt}_update") == len(names)
    a, b = (gradient_buckets(plans[o], bucket_bytes=200_000) for o in ("sgd", "adamw"))
    assert plans["sgd"].arena_bytes == plans["adamw"].arena_bytes
    assert [(x["start"], x["end"], x["ready"]) for x in a] == [(x["start"], x["end"], x["ready"]) for x in b]


WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["LB_ROOT"])
from lumen_b200 import transformer as T
from oracle import oracle
from tests.test_train_step import batch_of

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = T.Config(vocab=32, d_model=32, heads=2, hidden=64, layers=1, seq=16, dtype="float32", lr=0.1)
batch = 4
params = T.init_params(cfg, 0)
ids, targets = batch_of(cfg, batch)
shard = slice(rank * batch // world, (rank + 1) * batch // world)
g, names, _ = T.trace_train_step(cfg, batch // world, with_grads=True)
outs = oracle.run(g, [ids[shard], targets[shard]] + [params[n] for n in names])
grads = outs[1 + len(names):]
# one flat arena, reduced in buckets, then the update scaled by 1 / world (sum semantics of all_reduce)
flat = torch.from_numpy(np.concatenate([x.ravel() for x in grads]))
half = flat.numel() // 2
for piece in (flat[:half], flat[half:]):
    dist.all_reduce(piece, op=dist.ReduceOp.SUM)
at, new = 0, {}
for n, x in zip(names, grads):
    gsum = flat[at:at + x.size].numpy().reshape(x.shape)
    at += x.size
    new[n] = (params[n] - (gsum * np.float32(1.0 / world)) * np.float32(cfg.lr)).astype(np.float32)
if rank == 0:
    np.savez(os.environ["LB_OUT"], **new)
dist.barrier()
dist.destroy_process_group()
"""


def test_two_gloo_ranks_match_the_full_batch_step(tmp_path):
    out = str(tmp_path / "dp.npz")
    port = 29500 + os.getpid() % 2000
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   LB_ROOT=ROOT, LB_OUT=out, OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, cwd=ROOT))
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = np.load(out)
    from oracle import oracle

    cfg = T.Config(vocab=32, d_model=32, heads=2, hidden=64, layers=1, seq=16, dtype="float32", lr=0.1)
    params = T.init_params(cfg, 0)
    ids, targets = batch_of(cfg, 4)
    g, names, _ = T.trace_train_step(cfg, 4)
    want = oracle.run(g, [ids, targets] + [params[n] for n in names])[1:]
    for n, w in zip(names, want):
        np.testing.assert_allclose(got[n], w, rtol=1e-5, atol=1e-7, err_msg=n)
