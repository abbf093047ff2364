"""The data-parallel training step on 2 GPUs (one process per GPU, the backend's own store and NCCL communicator, the
all-reduces as plan steps): both ranks end with the weights of the single-GPU step on the whole batch, with the
ranges between collectives replayed as CUDA graphs and without graphs. Skipped on a single-GPU box."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

WORKER = r"""
import os, sys
import numpy as np
sys.path.insert(0, os.environ["LB_ROOT"])
from lumen_b200 import device, distributed
from lumen_b200 import transformer as T
from lumen_b200.runtime import device_status


def batch_of(cfg, batch, seed=0):
    t = np.random.default_rng(seed).integers(0, cfg.vocab, (batch, cfg.seq + 1)).astype(np.int64)
    return np.ascontiguousarray(t[:, :-1]), np.ascontiguousarray(t[:, 1:])


assert "torch" not in sys.modules  # the step, its memory, its stream and its collectives are the backend's own
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
device.set_device(rank)
group = distributed.init_process_group(timeout=60.0) if world > 1 else None
cfg = T.Config(vocab=512, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16", lr=float(os.environ["LB_LR"]))
batch = 4
ids, targets = batch_of(cfg, batch)
per = batch // world
init = T.init_params(cfg, 0)
step = T.TrainStep(cfg, per, init, rank, world=world, process_group=group, bucket_bytes=100_000, graphs=os.environ["LB_GRAPHS"],
                   lowering=os.environ.get("LB_LOWERING", "native"))
step.load_batch(ids[rank * per:(rank + 1) * per], targets[rank * per:(rank + 1) * per])
for _ in range(3):
    step.step()
step.synchronize(timeout=60.0)
device_status()
out = {n: a.astype(np.float32) for n, a in step.state_dict().items()}
out["__buckets"] = np.array(len(step.buckets))
out["__loss"] = np.array(step.loss.item())
assert "torch" not in sys.modules
np.savez(os.environ["LB_OUT"] + f".{world}.{rank}.npz", **out)
if world > 1:
    distributed.destroy_process_group()
"""


LR = 0.25  # large on purpose: three steps move the weights far more than the comparison's tolerance


def launch(world, out, port, graphs="whole", lowering="native"):
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), LB_ROOT=ROOT, LB_OUT=out, LB_GRAPHS=graphs, LB_LR=str(LR), LB_LOWERING=lowering)
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, cwd=ROOT))
    try:
        for p in procs:
            assert p.wait(timeout=90) == 0
    finally:
        for p in procs:  # a rank that is still running after the deadline is ended, whatever it waits for
            if p.poll() is None:
                p.kill()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("graphs", ["off", "segments"])
def test_two_ranks_match_one(tmp_path, graphs):
    """The DELTAS (weights after three steps minus the initial weights) of the 2-rank run equal the 1-rank run's to
    bfloat16 rounding of the per-rank partial sums: a gradient that was summed but not averaged, or averaged twice,
    would be off by a factor of two."""
    from lumen_b200 import transformer as T
    from tests.helpers import bf16

    out = str(tmp_path / "dp")
    launch(1, out, 29650, graphs)
    launch(2, out, 29652, graphs)
    cfg = T.Config(vocab=512, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16")
    init = {n: bf16(a).astype(np.float32) for n, a in T.init_params(cfg, 0).items()}
    one = np.load(out + ".1.0.npz")
    for rank in range(2):
        two = np.load(out + f".2.{rank}.npz")
        assert int(two["__buckets"]) > 1
        assert abs(float(two["__loss"]) - float(one["__loss"])) < 0.5  # each rank reports its own shard's loss
        for name in init:
            want, got = one[name] - init[name], two[name] - init[name]
            scale = np.abs(want).max()
            if name.endswith("norm.w"):  # scales start at 1.0: their updates are below one bfloat16 step of 1.0
                np.testing.assert_allclose(got, want, atol=2.0**-7)
                continue
            assert scale > 1e-3, name  # the update is far above bfloat16 noise
            assert np.abs(got - want).max() <= 2.0**-5 * scale + 2.0**-7 * np.abs(one[name]).max(), (rank, name)
            assert (got * want).sum() >= 0.99 * np.linalg.norm(got) * np.linalg.norm(want), (rank, name)
    a, b = np.load(out + ".2.0.npz"), np.load(out + ".2.1.npz")
    for name in init:
        np.testing.assert_array_equal(a[name], b[name])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_on_the_native_lowering(tmp_path):
    """The 2-rank step lowered by `lb_compile` (the backend's C++ lowering: gradient arena, buckets, `all_reduce` and
    `wait` steps, fused updates): both ranks end with the weights the 2-rank step of the Python lowering ends with,
    bit for bit (the same kernels and the same collectives in the same order)."""
    from lumen_b200 import transformer as T

    out_py, out_native = str(tmp_path / "py"), str(tmp_path / "native")
    launch(2, out_py, 29654, "segments", "optimising")
    launch(2, out_native, 29656, "segments", "native")
    cfg = T.Config(vocab=512, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16")
    for rank in range(2):
        a, b = np.load(out_py + f".2.{rank}.npz"), np.load(out_native + f".2.{rank}.npz")
        assert int(b["__buckets"]) == int(a["__buckets"]) > 1
        assert float(a["__loss"]) == float(b["__loss"])
        for name, _ in T.param_shapes(cfg):
            np.testing.assert_array_equal(a[name], b[name], err_msg=name)
