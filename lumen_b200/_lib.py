"""ctypes binding of liblumen_b200.so (the C ABI of include/lumen_b200.h). There is no Python or CPU fallback: a
missing library or a failed call raises."""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblumen_b200.so")

DTYPE_CODES = {
    "bool": 0, "int8": 1, "int16": 2, "int32": 3, "int64": 4, "uint8": 5, "uint16": 6, "uint32": 7, "uint64": 8,
    "float16": 9, "bfloat16": 10, "float32": 11, "float64": 12,
}  # fmt: skip
MAX_RANK = 8


class LbTensor(ctypes.Structure):
    _fields_ = [
        ("ptr", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("shape", ctypes.c_int64 * MAX_RANK),
        ("stride", ctypes.c_int64 * MAX_RANK),
    ]


class LbGemmOut(ctypes.Structure):
    _fields_ = [("product", LbTensor), ("epilogue", ctypes.c_int32), ("reserved", ctypes.c_int32), ("aux", LbTensor)]


class LbGemmCfg(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_int32), ("reserved", ctypes.c_int32), ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
                ("splits", ctypes.c_int32), ("group_m", ctypes.c_int32)]


class LbAttnDesc(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_float), ("causal", ctypes.c_int32), ("causal_offset", ctypes.c_int64)]


class LumenError(RuntimeError):
    """A failed call into liblumen_b200.so; `status` is the lb_status code."""

    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(make -C lumen_b200/csrc). lumen_b200 has no fallback path."
            )
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.lb_last_error.restype = ctypes.c_char_p
        _lib.lb_version.restype = ctypes.c_char_p
        _lib.lb_fusion_source.restype = ctypes.c_char_p
        _lib.lb_fusion_source.argtypes = [ctypes.c_void_p]
        _lib.lb_fusion_scratch_bytes.restype = ctypes.c_size_t
        _lib.lb_fusion_scratch_bytes.argtypes = [ctypes.c_void_p]
        _lib.lb_fusion_num_inputs.argtypes = [ctypes.c_void_p]
        _lib.lb_fusion_num_outputs.argtypes = [ctypes.c_void_p]
        _lib.lb_fusion_compile.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
        _lib.lb_fusion_check.argtypes = [ctypes.c_char_p]
        _lib.lb_fusion_launch.argtypes = [
            ctypes.c_void_p, ctypes.POINTER(LbTensor), ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
        ]  # fmt: skip
        _lib.lb_launch_fused.argtypes = [
            ctypes.c_char_p, ctypes.POINTER(LbTensor), ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
        ]  # fmt: skip
        _lib.lb_gemm.argtypes = [
            ctypes.POINTER(LbTensor), ctypes.POINTER(LbTensor), ctypes.POINTER(LbGemmOut), ctypes.POINTER(LbGemmCfg),
            ctypes.c_void_p,
        ]  # fmt: skip
        _lib.lb_gemm_scratch_bytes.argtypes = [ctypes.c_int64] * 4
        _lib.lb_gemm_scratch_bytes.restype = ctypes.c_size_t
        T = ctypes.POINTER(LbTensor)
        _lib.lb_attention_fwd.argtypes = [ctypes.POINTER(LbAttnDesc), T, T, T, T, T, ctypes.c_void_p]
        _lib.lb_attention_bwd.argtypes = [ctypes.POINTER(LbAttnDesc)] + [T] * 10 + [ctypes.c_void_p]
        _lib.lb_attention_bwd_atomic.argtypes = [ctypes.POINTER(LbAttnDesc)] + [T] * 11 + [ctypes.c_void_p]
        _lib.lb_attention_bwd_static.argtypes = [ctypes.POINTER(LbAttnDesc)] + [T] * 9 + [ctypes.c_void_p]
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise LumenError(status, lib().lb_last_error().decode(errors="replace"))


def dense(ptr: int, dtype: str, shape) -> LbTensor:
    """A dense row-major tensor descriptor over device memory at `ptr`."""
    t = LbTensor()
    t.ptr = ptr
    t.dtype = DTYPE_CODES[dtype]
    t.rank = len(shape)
    stride = 1
    for d in range(len(shape) - 1, -1, -1):
        t.shape[d] = shape[d]
        t.stride[d] = stride
        stride *= shape[d]
    return t


def strided(ptr: int, dtype: str, shape, strides) -> LbTensor:
    t = LbTensor()
    t.ptr = ptr
    t.dtype = DTYPE_CODES[dtype]
    t.rank = len(shape)
    for d in range(len(shape)):
        t.shape[d] = shape[d]
        t.stride[d] = strides[d]
    return t
