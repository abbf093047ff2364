"""The data-parallel training step on 2 GPUs (one process per GPU, NCCL): both ranks end with the weights of the
single-GPU step on the whole batch. Skipped on a single-GPU box."""

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
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["LB_ROOT"])
from lumen_b200 import transformer as T
from lumen_b200.runtime import device_status
from tests.test_train_step import batch_of

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
device = torch.device("cuda", rank)
if world > 1:
    dist.init_process_group("nccl", device_id=device)
cfg = T.Config(vocab=512, d_model=128, heads=2, hidden=256, layers=2, seq=128, dtype="bfloat16", lr=1e-2)
batch = 4
ids, targets = batch_of(cfg, batch)
per = batch // world
step = T.TrainStep(cfg, per, T.init_params(cfg, 0), device, world=world, bucket_bytes=100_000)
step.load_batch(torch.from_numpy(ids[rank * per:(rank + 1) * per]), torch.from_numpy(targets[rank * per:(rank + 1) * per]))
for _ in range(2):
    step.step()
device_status()
out = {n: p.float().cpu().numpy() for n, p in zip(step.names, step.params)}
out["__buckets"] = np.array(len(step.buckets))
np.savez(os.environ["LB_OUT"] + f".{world}.{rank}.npz", **out)
if world > 1:
    dist.barrier()
    dist.destroy_process_group()
"""


def launch(world, out, port):
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), LB_ROOT=ROOT, LB_OUT=out)
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, cwd=ROOT))
    for p in procs:
        assert p.wait(timeout=600) == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_match_one(tmp_path):
    out = str(tmp_path / "dp")
    launch(1, out, 29650)
    launch(2, out, 29651)
    one = np.load(out + ".1.0.npz")
    for rank in range(2):
        two = np.load(out + f".2.{rank}.npz")
        assert int(two["__buckets"]) > 1
        for name in one.files:
            if name.startswith("__"):
                continue
            # the same mean gradient up to bf16 rounding of per-rank partial sums; updates are lr * g ~ 1e-4
            np.testing.assert_allclose(two[name], one[name], rtol=2**-7, atol=2e-4, err_msg=f"rank {rank} {name}")
    a, b = np.load(out + ".2.0.npz"), np.load(out + ".2.1.npz")
    for name in a.files:
        np.testing.assert_array_equal(a[name], b[name])
