"""Process groups over the backend's own store and NCCL communicator (ctypes over the C ABI): the names of the
reference's `lumen.distributed` (`TCPStore`, `init_process_group`, `get_rank`, `get_world_size`, `barrier`,
`destroy_process_group`; lumen/distributed/__init__.py:21-66, lumen/distributed/store.rs, lumen/distributed/nccl.rs)
for the one thing this path needs: the data-parallel all-reduce of weight gradients, which a compiled plan runs as its
own steps (`lb_plan_set_comm`).

Rendezvous follows the usual launcher variables (`RANK`, `WORLD_SIZE`, `MASTER_ADDR`, `MASTER_PORT`). The store listens
on `LUMEN_STORE_PORT` when set, else on `MASTER_PORT + 1`: a launcher such as torchrun keeps `MASTER_PORT` itself for
its own agent store. Every wait on the store has a deadline; a rank that never arrives makes the others raise
`LumenError` with status `LB_ERR_TIMEOUT` instead of hanging.
"""

from __future__ import annotations

import ctypes
import os

from lumen_b200 import _lib

LB_ERR_TIMEOUT = 4


def _load_nccl() -> None:
    """Loads `libnccl.so.2` from the nvidia-nccl wheel when one is installed, before the backend opens NCCL by its
    soname: a process that later imports another framework built against that (newer) wheel must find its symbols in the
    copy already loaded (the reference does the same, lumen/distributed/__init__.py:106-120). Without the wheel the
    system's libnccl is used."""
    import importlib.util
    import sys

    if sys.platform != "linux":
        return
    spec = importlib.util.find_spec("nvidia.nccl") if importlib.util.find_spec("nvidia") else None
    for root in (spec.submodule_search_locations if spec else []):
        path = os.path.join(root, "lib", "libnccl.so.2")
        if os.path.exists(path):
            ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            return


def _bound():
    lib = _lib.lib()
    if getattr(lib, "_dist_bound", False):
        return lib
    _load_nccl()
    vp, P = ctypes.c_void_p, ctypes.POINTER
    lib.lb_store_create.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, P(vp)]
    lib.lb_store_destroy.argtypes = [vp]
    lib.lb_store_destroy.restype = None
    lib.lb_store_port.argtypes = [vp]
    lib.lb_store_set.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.lb_store_get.argtypes = [vp, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t, P(ctypes.c_size_t), ctypes.c_int]
    lib.lb_store_add.argtypes = [vp, ctypes.c_char_p, ctypes.c_int64, P(ctypes.c_int64)]
    lib.lb_store_wait.argtypes = [vp, P(ctypes.c_char_p), ctypes.c_int, ctypes.c_int]
    lib.lb_store_delete.argtypes = [vp, ctypes.c_char_p]
    lib.lb_comm_create.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, P(vp)]
    lib.lb_comm_destroy.argtypes = [vp]
    lib.lb_comm_destroy.restype = None
    lib.lb_comm_all_reduce.argtypes = [vp, vp, vp, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, vp]
    lib.lb_comm_broadcast.argtypes = [vp, vp, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, vp]
    lib.lb_comm_barrier.argtypes = [vp, ctypes.c_int]
    lib.lb_comm_check.argtypes = [vp]
    lib.lb_comm_synchronize.argtypes = [vp, vp, ctypes.c_int]
    lib.lb_comm_abort.argtypes = [vp]
    lib.lb_nccl_version.restype = ctypes.c_char_p
    lib._dist_bound = True
    return lib


class TCPStore:
    """A keyed store over TCP: the master rank's process serves it, every rank is a client
    (lumen/distributed/store.rs:100-230). `timeout` (seconds) bounds the connection and is the default of every wait."""

    def __init__(self, host: str, port: int, is_master: bool, timeout: float = 30.0):
        self.lib = _bound()
        self.handle = ctypes.c_void_p()
        _lib.check(self.lib.lb_store_create(host.encode(), int(port), int(is_master), int(timeout * 1000), ctypes.byref(self.handle)))
        self.host, self.timeout = host, timeout

    @property
    def port(self) -> int:
        return int(self.lib.lb_store_port(self.handle))

    def set(self, key: str, value: bytes) -> None:
        _lib.check(self.lib.lb_store_set(self.handle, key.encode(), bytes(value), len(value)))

    def get(self, key: str, timeout: float | None = None) -> bytes:
        """The value under `key`, waiting until it is set; `LumenError` (LB_ERR_TIMEOUT) at the deadline."""
        buf = ctypes.create_string_buffer(1 << 16)
        n = ctypes.c_size_t()
        _lib.check(self.lib.lb_store_get(self.handle, key.encode(), buf, len(buf), ctypes.byref(n), int((timeout or 0) * 1000)))
        return buf.raw[: n.value]

    def add(self, key: str, amount: int = 1) -> int:
        out = ctypes.c_int64()
        _lib.check(self.lib.lb_store_add(self.handle, key.encode(), int(amount), ctypes.byref(out)))
        return int(out.value)

    def wait(self, keys, timeout: float | None = None) -> None:
        arr = (ctypes.c_char_p * len(keys))(*[k.encode() for k in keys])
        _lib.check(self.lib.lb_store_wait(self.handle, arr, len(keys), int((timeout or 0) * 1000)))

    def delete(self, key: str) -> None:
        _lib.check(self.lib.lb_store_delete(self.handle, key.encode()))

    def close(self) -> None:
        if self.handle:
            self.lib.lb_store_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


REDUCE_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}


class ProcessGroup:
    """This process's membership of a group of `world` ranks: the store, and (on a GPU) the NCCL communicator."""

    def __init__(self, store: TCPStore, rank: int, world: int, timeout: float = 30.0, device_collectives: bool = True):
        self.lib = _bound()
        self.store, self.rank, self.world, self.timeout = store, rank, world, timeout
        self.comm = ctypes.c_void_p()
        self.rounds = 0
        if device_collectives:
            _lib.check(self.lib.lb_comm_create(store.handle, rank, world, int(timeout * 1000), ctypes.byref(self.comm)))

    def barrier(self, timeout: float | None = None) -> None:
        """Host barrier through the store; `LumenError` (LB_ERR_TIMEOUT) when a rank does not arrive in time."""
        wait_ms = int((timeout or self.timeout) * 1000)
        if self.comm:
            _lib.check(self.lib.lb_comm_barrier(self.comm, wait_ms))
            return
        # CPU ranks (no communicator): the same protocol on the store
        round_key = f"barrier/host/{self.rounds}"
        self.rounds += 1
        arrived = self.store.add(round_key + "/count", 1)
        if arrived == self.world:
            self.store.set(round_key + "/done", b"1")
        try:
            self.store.wait([round_key + "/done"], wait_ms / 1000)
        except _lib.LumenError as e:
            raise _lib.LumenError(e.status, f"barrier: {arrived} of {self.world} ranks arrived: {e}") from None

    def all_reduce(self, tensor, op: str = "sum", stream=None) -> None:
        """In-place all-reduce of a dense device tensor on `stream` (queued, not waited for)."""
        from lumen_b200.runtime import desc

        d = desc(tensor)
        count = 1
        for k in range(d.rank):
            count *= d.shape[k]
        _lib.check(self.lib.lb_comm_all_reduce(self.comm, d.ptr, d.ptr, count, d.dtype, REDUCE_OPS[op], _stream_handle(stream)))

    def broadcast(self, tensor, src: int = 0, stream=None) -> None:
        from lumen_b200.runtime import desc

        d = desc(tensor)
        count = 1
        for k in range(d.rank):
            count *= d.shape[k]
        _lib.check(self.lib.lb_comm_broadcast(self.comm, d.ptr, count, d.dtype, int(src), _stream_handle(stream)))

    def check(self) -> None:
        """Raises if NCCL has reported an asynchronous error on this communicator (a peer died, a link failed)."""
        _lib.check(self.lib.lb_comm_check(self.comm))

    def synchronize(self, stream=None, timeout: float | None = None) -> None:
        """Waits for `stream` with a deadline while polling the communicator's error state; on an error or at the
        deadline the communicator is aborted and `LumenError` raised - the host never waits on a dead peer forever."""
        _lib.check(self.lib.lb_comm_synchronize(self.comm, _stream_handle(stream), int((timeout or self.timeout) * 1000)))

    def destroy(self) -> None:
        if self.comm:
            self.lib.lb_comm_destroy(self.comm)
            self.comm = ctypes.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def _stream_handle(stream) -> int:
    if stream is None:
        return 0
    return getattr(stream, "handle", None) or getattr(stream, "cuda_stream", None) or int(stream)


_default: ProcessGroup | None = None


def store_port() -> int:
    if "LUMEN_STORE_PORT" in os.environ:
        return int(os.environ["LUMEN_STORE_PORT"])
    return int(os.environ.get("MASTER_PORT", "29500")) + 1


def init_process_group(rank: int | None = None, world_size: int | None = None, timeout: float = 60.0,
                       device_collectives: bool = True) -> ProcessGroup:
    """Joins the default group from the launcher's variables; rank 0 hosts the store. With `device_collectives` the
    current CUDA device (set it first: `lumen_b200.device.set_device(LOCAL_RANK)`) gets an NCCL communicator."""
    global _default
    if _default is not None:
        raise RuntimeError("the default process group is already initialised")
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    store = TCPStore(host, store_port(), rank == 0, timeout)
    _default = ProcessGroup(store, rank, world, timeout, device_collectives)
    return _default


def is_initialized() -> bool:
    return _default is not None


def default_group() -> ProcessGroup:
    if _default is None:
        raise RuntimeError("init_process_group() has not been called")
    return _default


def get_rank() -> int:
    return default_group().rank


def get_world_size() -> int:
    return default_group().world


def barrier(timeout: float | None = None) -> None:
    default_group().barrier(timeout)


def destroy_process_group() -> None:
    """Leaves the default group. Rank 0 serves the store, so it waits (bounded) for the others to arrive here first
    (the reference holds an exiting rank 0 the same way, lumen/distributed/__init__.py:122-127)."""
    global _default
    if _default is None:
        return
    group, _default = _default, None
    try:
        group.barrier(min(group.timeout, 10.0))
    except _lib.LumenError:
        pass
    group.destroy()
    group.store.close()


def nccl_version() -> str:
    return _bound().lb_nccl_version().decode()
