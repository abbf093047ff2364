"""Device memory, streams, events and pinned host buffers of the backend itself (ctypes over the C ABI): what a plan
needs to run without any other CUDA framework in the process. Mirrors the reference's runtime layer - the region
allocator (lumen/allocator/region.rs, lumen/allocator/cuda.rs), the stream and its events (lumen/runtime/stream/
cuda.rs) - at the size this path needs.

`Tensor` is a typed view of region memory. It answers `data_ptr()`, `shape`, `stride()`, `dtype` like the arrays of
other frameworks, so every entry point of `lumen_b200.runtime` takes it, and it exports `__cuda_array_interface__`
so that a harness can look at the same memory without a copy.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np

from lumen_b200 import _lib

ITEMSIZE = {"bool": 1, "int8": 1, "int16": 2, "int32": 4, "int64": 8, "uint8": 1, "uint16": 2, "uint32": 4, "uint64": 8,
            "float16": 2, "bfloat16": 2, "float32": 4, "float64": 8}  # fmt: skip


def _bound():
    lib = _lib.lib()
    if getattr(lib, "_device_bound", False):
        return lib
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    P = ctypes.POINTER
    lib.lb_set_device.argtypes = [ctypes.c_int]
    lib.lb_device_memory.argtypes = [P(sz), P(sz)]
    lib.lb_region_create.argtypes = [sz, P(vp)]
    lib.lb_region_destroy.argtypes = [vp]
    lib.lb_region_destroy.restype = None
    lib.lb_region_alloc.argtypes = [vp, sz, sz, P(vp)]
    lib.lb_region_free.argtypes = [vp, vp]
    lib.lb_region_hold.argtypes = [vp]
    lib.lb_region_release.argtypes = [vp]
    lib.lb_region_stats.argtypes = [vp, P(sz), P(sz), P(sz), P(sz)]
    lib.lb_stream_create.argtypes = [P(vp)]
    for name in ("lb_stream_destroy", "lb_stream_synchronize", "lb_event_destroy", "lb_event_synchronize", "lb_host_free"):
        getattr(lib, name).argtypes = [vp]
    lib.lb_event_create.argtypes = [ctypes.c_int, P(vp)]
    lib.lb_event_record.argtypes = [vp, vp]
    lib.lb_stream_wait_event.argtypes = [vp, vp]
    lib.lb_event_elapsed_ms.argtypes = [vp, vp, P(ctypes.c_float)]
    lib.lb_host_alloc.argtypes = [sz, P(vp)]
    for name in ("lb_copy_to_device", "lb_copy_to_host", "lb_copy_on_device"):
        getattr(lib, name).argtypes = [vp, vp, sz, vp]
    lib.lb_fill_bytes.argtypes = [vp, ctypes.c_int, sz, vp]
    lib._device_bound = True
    return lib


def set_device(index: int) -> None:
    """Makes GPU `index` current for this thread (fails unless it is an sm_100 part)."""
    _lib.check(_bound().lb_set_device(int(index)))


def device_count() -> int:
    return int(_bound().lb_device_count())


def synchronize() -> None:
    _lib.check(_bound().lb_device_synchronize())


def memory_info() -> tuple[int, int]:
    """(free, total) bytes of the current device."""
    free, total = ctypes.c_size_t(), ctypes.c_size_t()
    _lib.check(_bound().lb_device_memory(ctypes.byref(free), ctypes.byref(total)))
    return free.value, total.value


class Stream:
    """A CUDA stream owned by the backend; `Stream.default()` is the legacy default stream (handle 0)."""

    def __init__(self, handle=None):
        self.lib = _bound()
        self.owned = handle is None
        if handle is None:
            h = ctypes.c_void_p()
            _lib.check(self.lib.lb_stream_create(ctypes.byref(h)))
            handle = h.value
        self.handle = handle or 0

    @staticmethod
    def default() -> "Stream":
        return Stream(0)

    def synchronize(self) -> None:
        _lib.check(self.lib.lb_stream_synchronize(self.handle))

    def wait(self, event: "Event") -> None:
        _lib.check(self.lib.lb_stream_wait_event(self.handle, event.handle))

    def __del__(self):
        try:
            if self.owned and self.handle:
                self.lib.lb_stream_destroy(self.handle)
        except Exception:
            pass


class Event:
    def __init__(self, timing: bool = False):
        self.lib = _bound()
        h = ctypes.c_void_p()
        _lib.check(self.lib.lb_event_create(int(timing), ctypes.byref(h)))
        self.handle = h.value

    def record(self, stream: Stream | None = None) -> "Event":
        _lib.check(self.lib.lb_event_record(self.handle, stream.handle if stream else 0))
        return self

    def synchronize(self) -> None:
        _lib.check(self.lib.lb_event_synchronize(self.handle))

    def elapsed_ms(self, later: "Event") -> float:
        ms = ctypes.c_float()
        _lib.check(self.lib.lb_event_elapsed_ms(self.handle, later.handle, ctypes.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            if self.handle:
                self.lib.lb_event_destroy(self.handle)
        except Exception:
            pass


class Region:
    """One reservation of device memory, handed out in 256-byte aligned blocks (first fit, coalescing frees)."""

    def __init__(self, capacity_bytes: int):
        self.lib = _bound()
        h = ctypes.c_void_p()
        _lib.check(self.lib.lb_region_create(int(capacity_bytes), ctypes.byref(h)))
        self.handle = h

    def alloc(self, nbytes: int, alignment: int = 256) -> int:
        out = ctypes.c_void_p()
        _lib.check(self.lib.lb_region_alloc(self.handle, int(nbytes), int(alignment), ctypes.byref(out)))
        return out.value

    def free(self, ptr: int) -> None:
        _lib.check(self.lib.lb_region_free(self.handle, ptr))

    def hold(self) -> None:
        """Blocks freed from now on return to the region only at `release()`: a recorded graph may launch into them."""
        _lib.check(self.lib.lb_region_hold(self.handle))

    def release(self) -> None:
        _lib.check(self.lib.lb_region_release(self.handle))

    def stats(self) -> dict:
        vals = [ctypes.c_size_t() for _ in range(4)]
        _lib.check(self.lib.lb_region_stats(self.handle, *[ctypes.byref(v) for v in vals]))
        return dict(zip(("capacity", "live_bytes", "peak_bytes", "largest_free"), (v.value for v in vals)))

    def empty(self, shape, dtype: str, stream: "Stream | None" = None) -> "Tensor":
        """A new tensor; `stream` is remembered as the stream its reads and copies are ordered on by default."""
        shape = tuple(int(n) for n in shape)
        nbytes = max(math.prod(shape) * ITEMSIZE[dtype], 1)
        return Tensor(self.alloc(nbytes), shape, dtype, owner=self, owned=True, stream=stream)

    def zeros(self, shape, dtype: str, stream: "Stream | None" = None) -> "Tensor":
        t = self.empty(shape, dtype, stream)
        t.fill_bytes(0, stream)
        return t

    def __del__(self):
        try:
            if self.handle:
                self.lib.lb_region_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def dense_strides(shape):
    strides, step = [], 1
    for n in reversed(shape):
        strides.append(step)
        step *= n
    return tuple(reversed(strides))


class Tensor:
    """A typed view of device memory: pointer, dtype name, shape, element strides. Owned blocks go back to their region
    when the tensor is collected; views keep their base alive."""

    def __init__(self, ptr: int, shape, dtype: str, strides=None, owner=None, owned: bool = False, stream=None):
        self.ptr, self.shape, self.dtype = int(ptr), tuple(shape), dtype
        self.strides = tuple(strides) if strides is not None else dense_strides(self.shape)
        self.owner, self.owned = owner, owned
        # the stream whose work produces this tensor: copies and reads that name no stream are ordered after it
        self.stream = stream
        self.lib = _bound()

    # the protocol lumen_b200.runtime.desc reads
    def data_ptr(self) -> int:
        return self.ptr

    def stride(self):
        return self.strides

    @property
    def is_cuda(self) -> bool:
        return True

    def numel(self) -> int:
        return math.prod(self.shape)

    def element_size(self) -> int:
        return ITEMSIZE[self.dtype]

    def item(self):
        """The one element of a one-element tensor as a Python number (synchronous copy)."""
        if self.numel() != 1:
            raise ValueError("item(): a tensor of one element")
        return self.copy_to_host().reshape(()).item()

    @property
    def nbytes(self) -> int:
        return self.numel() * ITEMSIZE[self.dtype]

    @property
    def __cuda_array_interface__(self):
        # bfloat16 has no NumPy type string: exported as its bit pattern (uint16)
        kinds = {"bool": "|b1", "int8": "|i1", "int16": "<i2", "int32": "<i4", "int64": "<i8", "uint8": "|u1", "uint16": "<u2",
                 "uint32": "<u4", "uint64": "<u8", "float16": "<f2", "bfloat16": "<u2", "float32": "<f4", "float64": "<f8"}  # fmt: skip
        size = ITEMSIZE[self.dtype]
        return {"shape": self.shape, "typestr": kinds[self.dtype], "data": (self.ptr, False), "version": 3,
                "strides": tuple(s * size for s in self.strides)}

    def view(self, shape, dtype: str | None = None, byte_offset: int = 0) -> "Tensor":
        """A dense view of the same memory (the caller answers for it fitting)."""
        return Tensor(self.ptr + byte_offset, shape, dtype or self.dtype, owner=self, stream=self.stream)

    def _handle(self, stream) -> int:
        stream = stream if stream is not None else self.stream
        return stream.handle if stream is not None else 0

    def fill_bytes(self, byte: int, stream: Stream | None = None) -> None:
        _lib.check(self.lib.lb_fill_bytes(self.ptr, byte, self.nbytes, self._handle(stream)))

    def copy_from_host(self, array, stream: Stream | None = None) -> None:
        """Copies a NumPy array or a `HostBuffer` of the same byte size in (asynchronous only from pinned memory)."""
        src, nbytes, keep = _host_pointer(array)
        if nbytes != self.nbytes:
            raise ValueError(f"copy_from_host: {nbytes} bytes into a tensor of {self.nbytes}")
        _lib.check(self.lib.lb_copy_to_device(self.ptr, src, nbytes, self._handle(stream)))
        if not isinstance(array, HostBuffer):
            _lib.check(self.lib.lb_stream_synchronize(self._handle(stream)))  # pageable memory: finish before `keep` goes
        del keep

    def copy_to_host(self, out=None, stream: Stream | None = None):
        """Copies out into `out` (a `HostBuffer`, asynchronous) or into a new NumPy array (synchronous)."""
        if isinstance(out, HostBuffer):
            if out.nbytes < self.nbytes:
                raise ValueError("copy_to_host: the host buffer is too small")
            _lib.check(self.lib.lb_copy_to_host(out.ptr, self.ptr, self.nbytes, self._handle(stream)))
            return out
        if self.strides != dense_strides(self.shape):
            raise ValueError("copy_to_host: only dense tensors")
        np_dtype = numpy_dtype(self.dtype)
        host = np.empty(self.shape, np_dtype)
        _lib.check(self.lib.lb_copy_to_host(host.ctypes.data, self.ptr, self.nbytes, self._handle(stream)))
        _lib.check(self.lib.lb_stream_synchronize(self._handle(stream)))
        return host

    def numpy(self):
        return self.copy_to_host()

    def __del__(self):
        try:
            if self.owned and self.owner is not None and self.owner.handle:
                self.owner.free(self.ptr)
        except Exception:
            pass


def numpy_dtype(name: str):
    if name == "bfloat16":
        import ml_dtypes

        return np.dtype(ml_dtypes.bfloat16)
    return np.dtype(name if name != "bool" else np.bool_)


class HostBuffer:
    """Page-locked host memory for asynchronous copies; `array(dtype, shape)` views it as NumPy."""

    def __init__(self, nbytes: int):
        self.lib = _bound()
        p = ctypes.c_void_p()
        _lib.check(self.lib.lb_host_alloc(int(nbytes), ctypes.byref(p)))
        self.ptr, self.nbytes = p.value, int(nbytes)

    def array(self, dtype, shape):
        dt = np.dtype(dtype)
        n = math.prod(shape)
        if n * dt.itemsize > self.nbytes:
            raise ValueError("HostBuffer.array: view larger than the buffer")
        buf = (ctypes.c_char * self.nbytes).from_address(self.ptr)
        return np.frombuffer(buf, dtype=dt, count=n).reshape(shape)

    def __del__(self):
        try:
            if self.ptr:
                self.lib.lb_host_free(self.ptr)
                self.ptr = None
        except Exception:
            pass


def _host_pointer(array):
    if isinstance(array, HostBuffer):
        return array.ptr, array.nbytes, array
    a = np.ascontiguousarray(array)
    return a.ctypes.data, a.nbytes, a
