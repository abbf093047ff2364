"""ctypes front of the CPU oracle (oracle/oracle.cpp). TEST INFRASTRUCTURE ONLY: imported by tests/,
`__graft_entry__.smoke()` and bench.py's CPU-baseline legs, never by the lumen_b200 package."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

try:
    import ml_dtypes

    BF16 = np.dtype(ml_dtypes.bfloat16)
except ImportError:  # pragma: no cover - the image ships ml_dtypes
    BF16 = None

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")

NUMPY = {
    "bool": np.dtype(np.bool_), "int8": np.dtype(np.int8), "int16": np.dtype(np.int16), "int32": np.dtype(np.int32),
    "int64": np.dtype(np.int64), "uint8": np.dtype(np.uint8), "uint16": np.dtype(np.uint16),
    "uint32": np.dtype(np.uint32), "uint64": np.dtype(np.uint64), "float16": np.dtype(np.float16),
    "bfloat16": BF16, "float32": np.dtype(np.float32), "float64": np.dtype(np.float64),
}  # fmt: skip


def build(force: bool = False) -> str:
    """Compiles liboracle.so when missing or older than its source."""
    src = os.path.join(HERE, "oracle.cpp")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_run.restype = ctypes.c_int
        _lib.oracle_round.restype = ctypes.c_double
        _lib.oracle_round.argtypes = [ctypes.c_double, ctypes.c_char_p]
    return _lib


def threads() -> int:
    """OpenMP threads the oracle's loops use (OMP_NUM_THREADS as it was when the library was loaded)."""
    return int(lib().oracle_threads())


def set_threads(n: int) -> None:
    """Runs the oracle's loops on `n` threads from now on (torchrun exports OMP_NUM_THREADS=1 to its workers)."""
    lib().oracle_set_threads(int(n))


def round_to(x: float, dtype: str) -> float:
    return lib().oracle_round(float(x), dtype.encode())


def run(graph, inputs):
    """Evaluates `graph` (a lumen_b200.graph.Graph) on numpy `inputs`; returns its outputs as numpy arrays."""
    text = graph.to_text().encode()
    arrays = []
    for v, a in zip(graph.inputs, inputs):
        t = graph.types[v]
        a = np.require(a, requirements="C")  # ascontiguousarray would turn a 0-d array into a 1-d one
        if a.dtype != NUMPY[t.dtype] or tuple(a.shape) != t.shape:
            raise TypeError(f"input %{v} must be {t}, got {a.dtype}{list(a.shape)}")
        arrays.append(a)
    if len(arrays) != len(graph.inputs):
        raise TypeError(f"the graph takes {len(graph.inputs)} inputs, got {len(arrays)}")
    outs = [np.empty(graph.types[v].shape, NUMPY[graph.types[v].dtype]) for v in graph.outputs]
    in_ptrs = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    out_ptrs = (ctypes.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
    err = ctypes.create_string_buffer(1024)
    rc = lib().oracle_run(text, len(arrays), in_ptrs, len(outs), out_ptrs, err, 1024)
    if rc != 0:
        raise RuntimeError(err.value.decode())
    return outs
