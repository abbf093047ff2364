"""The rendezvous store and the host side of the process group, among CPU processes: every wait has a deadline, so a
rank that never arrives, or that leaves between steps, makes its peers return LB_ERR_TIMEOUT instead of hanging
(lumen/distributed/store.rs:43-72: `wait_for(keys, timeout)`)."""

import os
import subprocess
import sys
import time

import pytest

from lumen_b200 import _lib
from lumen_b200.distributed import LB_ERR_TIMEOUT, ProcessGroup, TCPStore

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_set_get_add_wait_delete():
    master = TCPStore("127.0.0.1", 0, True, timeout=5.0)
    client = TCPStore("127.0.0.1", master.port, False, timeout=5.0)
    master.set("a", b"hello")
    assert client.get("a") == b"hello"
    assert client.add("n", 2) == 2 and master.add("n", 3) == 5
    assert client.get("n") == b"5"
    client.set("b", b"")
    master.wait(["a", "b", "n"], timeout=1.0)
    client.delete("a")
    t0 = time.monotonic()
    with pytest.raises(_lib.LumenError) as err:
        master.get("a", timeout=0.3)
    assert err.value.status == LB_ERR_TIMEOUT and 0.25 < time.monotonic() - t0 < 3.0
    with pytest.raises(_lib.LumenError) as err:
        client.wait(["b", "never"], timeout=0.2)
    assert err.value.status == LB_ERR_TIMEOUT and "never" in str(err.value)
    client.close()
    master.close()


def test_a_waiter_wakes_when_the_key_arrives():
    import threading

    master = TCPStore("127.0.0.1", 0, True, timeout=5.0)
    client = TCPStore("127.0.0.1", master.port, False, timeout=5.0)
    threading.Timer(0.2, lambda: master.set("late", b"x")).start()
    t0 = time.monotonic()
    assert client.get("late", timeout=5.0) == b"x"
    assert time.monotonic() - t0 < 2.0
    client.close()
    master.close()


def test_no_master_times_out():
    t0 = time.monotonic()
    with pytest.raises(_lib.LumenError) as err:
        TCPStore("127.0.0.1", 1, False, timeout=0.3)  # nothing listens on port 1
    assert err.value.status == LB_ERR_TIMEOUT and time.monotonic() - t0 < 3.0


WORKER = r"""
import os, sys, time
sys.path.insert(0, os.environ["LB_ROOT"])
from lumen_b200 import _lib
from lumen_b200.distributed import ProcessGroup, TCPStore

rank, world, port = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LB_PORT"])
mode = os.environ["LB_MODE"]
store = TCPStore("127.0.0.1", port, rank == 0, timeout=10.0)
group = ProcessGroup(store, rank, world, timeout=10.0, device_collectives=False)
group.barrier()
if mode == "steps":
    # three "steps", a host barrier before each; rank 1 leaves after the first one, between steps
    for step in range(3):
        if rank == 1 and step == 1:
            sys.exit(0)
        try:
            group.barrier(timeout=1.0)
        except _lib.LumenError as e:
            print(f"rank {rank} step {step}: status {e.status}", flush=True)
            sys.exit(40 + e.status)
    sys.exit(0)
if mode == "ok":
    total = store.add("sum", rank + 1)
    group.barrier()
    assert int(store.get("sum")) == world * (world + 1) // 2
    group.barrier()
    sys.exit(0)
"""


def launch(mode, world, absent=()):
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = {}
    for rank in range(world):
        if rank in absent:
            continue
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LB_PORT=str(port), LB_MODE=mode, LB_ROOT=ROOT)
        procs[rank] = subprocess.Popen([sys.executable, "-c", WORKER], env=env, cwd=ROOT, stdout=subprocess.PIPE, text=True)
    return {rank: (p.wait(timeout=120), p.stdout.read()) for rank, p in procs.items()}


def test_two_ranks_meet_at_barriers():
    results = launch("ok", 2)
    assert all(rc == 0 for rc, _ in results.values()), results


def test_a_rank_that_never_joins_times_the_others_out():
    """World of 2, only rank 0 starts: its first barrier gives up at its deadline with LB_ERR_TIMEOUT (exit code 1 from
    the uncaught LumenError), within seconds."""
    t0 = time.monotonic()
    env = dict(os.environ, RANK="0", WORLD_SIZE="2", LB_PORT="0", LB_MODE="ok", LB_ROOT=ROOT)
    code = WORKER.replace('timeout=10.0', 'timeout=1.0')
    p = subprocess.run([sys.executable, "-c", code], env=env, cwd=ROOT, capture_output=True, text=True, timeout=60)
    assert p.returncode != 0 and "1 of 2 ranks arrived" in p.stderr, p.stderr[-500:]
    assert time.monotonic() - t0 < 30


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    """Rank 1 exits after the first step. Rank 0's barrier before the next step returns LB_ERR_TIMEOUT after its one
    second deadline: it learns of the loss on the host, before it would queue the next launch."""
    results = launch("steps", 2)
    assert results[1][0] == 0
    assert results[0][0] == 40 + LB_ERR_TIMEOUT, results
    assert "step 1: status 4" in results[0][1]


def test_process_group_without_a_gpu_keeps_to_the_host():
    store = TCPStore("127.0.0.1", 0, True, timeout=2.0)
    group = ProcessGroup(store, 0, 1, timeout=2.0, device_collectives=False)
    group.barrier()
    assert not group.comm
    store.close()
