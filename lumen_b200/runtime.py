"""Host-side handles over the C ABI: fused kernels compiled from fusion bodies, GEMM, attention, scatter-add, launched
on device memory the caller holds. Tensors are duck-typed: the backend's own `lumen_b200.device.Tensor`, or any array
of another framework that answers `data_ptr()`, `shape`, `stride()` and `dtype` (a harness may pass torch CUDA
tensors; torch is never imported by this module unless the caller already did). Every kernel that runs is
liblumen_b200's."""

from __future__ import annotations

import ctypes
import sys

from lumen_b200 import _lib
from lumen_b200.graph import Graph


class _TorchDtypes(dict):
    """dtype name -> torch dtype, filled on first use so that importing this module does not import torch."""

    def __missing__(self, key):
        import torch

        self.update({
            "bool": torch.bool, "int8": torch.int8, "int16": torch.int16, "int32": torch.int32, "int64": torch.int64,
            "uint8": torch.uint8, "uint16": torch.uint16, "uint32": torch.uint32, "uint64": torch.uint64,
            "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "float64": torch.float64,
        })  # fmt: skip
        return dict.__getitem__(self, key)


TORCH_DTYPES = _TorchDtypes()


def dtype_name(dtype) -> str:
    """The lumen dtype name of a tensor's `dtype` attribute (a name already, or another framework's dtype object)."""
    if isinstance(dtype, str):
        return dtype
    name = str(dtype).rsplit(".", 1)[-1]  # "torch.bfloat16" -> "bfloat16"
    if name not in _lib.DTYPE_CODES:
        raise TypeError(f"no lumen dtype for {dtype!r}")
    return name


def require_cuda() -> None:
    if _lib.lib().lb_device_count() <= 0:
        raise RuntimeError("lumen_b200 runs on a B200 GPU only: no CUDA device is available and there is no CPU fallback")


def desc(t) -> _lib.LbTensor:
    """The lb_tensor descriptor of a device tensor (shape, element strides, data pointer)."""
    if not getattr(t, "is_cuda", True):
        raise ValueError("expected a CUDA tensor")
    return _lib.strided(t.data_ptr(), dtype_name(t.dtype), tuple(t.shape), tuple(t.stride()))


_current = [0]


def set_current_stream(stream) -> None:
    """The stream launches go to when none is given and torch is not in the process (a `lumen_b200.device.Stream`)."""
    _current[0] = getattr(stream, "handle", stream) or 0


def current_stream() -> int:
    """The caller's current stream: torch's when the process uses torch (a harness), else the one set with
    `set_current_stream` (the legacy default stream by default)."""
    torch = sys.modules.get("torch")
    if torch is not None and _current[0] == 0 and torch.cuda.is_initialized():
        return torch.cuda.current_stream().cuda_stream
    return _current[0]


class Fusion:
    """One generated kernel for a fusion body (`lb_fusion_compile` / `lb_fusion_launch`)."""

    def __init__(self, body: Graph | str):
        text = body if isinstance(body, str) else body.to_text()
        handle = ctypes.c_void_p()
        _lib.check(_lib.lib().lb_fusion_compile(text.encode(), ctypes.byref(handle)))
        self.handle = handle
        self.n_inputs = _lib.lib().lb_fusion_num_inputs(handle)
        self.n_outputs = _lib.lib().lb_fusion_num_outputs(handle)
        self.scratch_bytes = _lib.lib().lb_fusion_scratch_bytes(handle)
        self.body = body if isinstance(body, Graph) else None
        self._scratch = None

    @property
    def source(self) -> str:
        return _lib.lib().lb_fusion_source(self.handle).decode()

    def launch_raw(self, descs, scratch_ptr=None, stream=None) -> None:
        arr = (_lib.LbTensor * len(descs))(*descs)
        _lib.check(
            _lib.lib().lb_fusion_launch(
                self.handle, arr, len(descs), scratch_ptr, current_stream() if stream is None else stream
            )
        )

    def __call__(self, *inputs, out=None, stream=None):
        """Runs the kernel on CUDA tensors; allocates the outputs unless `out` gives them."""
        require_cuda()
        if self.body is None:
            raise RuntimeError("calling a Fusion built from text needs explicit outputs: use launch_raw")
        if out is None:
            out = [_empty_like_input(inputs[0], self.body.types[v].shape, self.body.types[v].dtype) for v in self.body.outputs]
        scratch = None
        if self.scratch_bytes:
            if self._scratch is None or self._scratch.numel() < self.scratch_bytes:
                self._scratch = _empty_like_input(inputs[0], (self.scratch_bytes,), "uint8")
            scratch = self._scratch.data_ptr()
        self.launch_raw([desc(t) for t in (*inputs, *out)], scratch, stream)
        return out


_scratch_region = []


def _empty_like_input(like, shape, dtype: str):
    """A new dense device tensor of `shape`/`dtype` in the framework `like` comes from: torch for a torch tensor (the
    harness's convenience), else the backend's own region (grown in 256 MiB reservations)."""
    if type(like).__module__.startswith("torch"):
        import torch

        return torch.empty(tuple(shape), dtype=TORCH_DTYPES[dtype], device=like.device)
    from lumen_b200.device import ITEMSIZE, Region

    import math

    nbytes = max(math.prod(shape) * ITEMSIZE[dtype], 1)
    for region in _scratch_region:
        try:
            return region.empty(shape, dtype)
        except _lib.LumenError:
            continue
    _scratch_region.append(Region(max(nbytes + 4096, 256 << 20)))
    return _scratch_region[-1].empty(shape, dtype)


GEMM_KERNELS = {"auto": 0, "tcgen05": 1, "simt": 2, "tcgen05_1cta": 3}
EPILOGUES = {None: 0, "none": 0, "relu": 1, "add": 2, "mask_positive": 3}


def gemm(a, b, out, epilogue=None, kernel="auto", stream=None, scratch=None, aux=None):
    """`out[.., M, N] = a[.., M, K] @ b[.., K, N]` with float32 accumulation through `lb_gemm`. `a` and `b` may be
    transposed views (any unit-stride major); `out` is float32 or the operands' dtype, row-major. `scratch` (a
    uint8 tensor of `gemm_scratch_bytes` bytes) lets few-tile, long-K problems split K. Epilogues: "relu";
    "add" (`round(product) + aux`) and "mask_positive" (`aux > 0 ? round(product) : 0`) with `aux` shaped like `out`."""
    require_cuda()
    o = _lib.LbGemmOut()
    o.product = desc(out)
    o.epilogue = EPILOGUES[epilogue]
    if aux is not None:
        o.aux = desc(aux)
    cfg = _lib.LbGemmCfg()
    cfg.kernel = GEMM_KERNELS[kernel]
    if scratch is not None:
        cfg.scratch, cfg.scratch_bytes = scratch.data_ptr(), scratch.numel() * scratch.element_size()
    da, db = desc(a), desc(b)
    _lib.check(
        _lib.lib().lb_gemm(
            ctypes.byref(da), ctypes.byref(db), ctypes.byref(o), ctypes.byref(cfg),
            current_stream() if stream is None else stream,
        )
    )  # fmt: skip
    return out


def device_status() -> None:
    """Synchronises and raises if a kernel's bounded wait gave up (`lb_device_status`)."""
    _lib.check(_lib.lib().lb_device_status())


def attention_forward(q, k, v, scale=None, causal=False, out=None, lse=None, stream=None):
    """Flash attention forward through `lb_attention_fwd`: `q` [B, Sq, N, H], `k`/`v` [B, Sk, Nkv, H] bfloat16 views;
    returns `(o, lse)` with `o` [B, Sq, N, H] bfloat16 and `lse` [B, N, Sq] float32."""
    require_cuda()
    b, sq, n, h = q.shape
    sk = k.shape[1]
    if out is None:
        out = _empty_like_input(q, (b, sq, n, h), dtype_name(q.dtype))
    if lse is None:
        lse = _empty_like_input(q, (b, n, sq), "float32")
    d = _lib.LbAttnDesc()
    d.scale = float(scale if scale is not None else h**-0.5)
    d.causal = int(bool(causal))
    d.causal_offset = sk - sq
    dq, dk, dv, do, dl = desc(q), desc(k), desc(v), desc(out), desc(lse)
    _lib.check(
        _lib.lib().lb_attention_fwd(
            ctypes.byref(d), ctypes.byref(dq), ctypes.byref(dk), ctypes.byref(dv), ctypes.byref(do), ctypes.byref(dl),
            current_stream() if stream is None else stream,
        )
    )  # fmt: skip
    return out, lse


def attention_backward(q, k, v, o, d_o, lse, scale=None, causal=False, delta=None, stream=None, deterministic=True):
    """Flash attention backward; returns `(dq, dk, dv)` shaped like `q`, `k`, `v`. `deterministic` (the default here)
    runs `lb_attention_bwd`, the dK/dV + dQ kernel pair that is bit-identical from run to run; without it
    `lb_attention_bwd_atomic` runs the reference backend's default mode, one kernel adding dQ atomically into a float32
    accumulator."""
    require_cuda()
    b, sq, n, h = q.shape
    sk = k.shape[1]
    dq, dk, dv = (_empty_like_input(t, tuple(t.shape), dtype_name(t.dtype)) for t in (q, k, v))
    if delta is None:
        delta = _empty_like_input(q, (b, n, sq), "float32")
    d = _lib.LbAttnDesc()
    d.scale = float(scale if scale is not None else h**-0.5)
    d.causal = int(bool(causal))
    d.causal_offset = sk - sq
    tensors = [q, k, v, o, d_o, lse, delta, dq, dk, dv]
    entry = _lib.lib().lb_attention_bwd
    if not deterministic:
        tensors.insert(7, _empty_like_input(q, (b, sq, n, h), "float32"))
        entry = _lib.lib().lb_attention_bwd_atomic
    descs = [desc(t) for t in tensors]
    _lib.check(entry(ctypes.byref(d), *[ctypes.byref(x) for x in descs], current_stream() if stream is None else stream))
    return dq, dk, dv


def gemm_scratch_bytes(m: int, n: int, k: int, batch: int = 1) -> int:
    """Bytes of scratch with which `gemm` splits K for this problem (0: it would not split)."""
    return _lib.lib().lb_gemm_scratch_bytes(m, n, k, batch)


def scatter_add_rows(x, ids, updates, deterministic=True, stream=None):
    """`x` `[rows, width]` with `updates[t]` added into row `ids[t]` (clamped into range), through
    `lb_scatter_add_rows`. Deterministic form: a row hit more than once adds its updates in update order, rounding
    after each add, like the reference interpreter; otherwise float32 atomics in arrival order and one rounding."""
    require_cuda()
    lib = _lib.lib()
    lib.lb_scatter_add_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
    lib.lb_scatter_add_scratch_bytes.restype = ctypes.c_size_t
    T = ctypes.POINTER(_lib.LbTensor)
    lib.lb_scatter_add_rows.argtypes = [T, T, T, T, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    rows, width = x.shape
    nbytes = lib.lb_scatter_add_scratch_bytes(rows, width, ids.numel(), int(deterministic))
    scratch = _empty_like_input(x, (max(nbytes, 4),), "uint8")
    out = _empty_like_input(x, tuple(x.shape), dtype_name(x.dtype))
    dx, di, du, do = desc(x), desc(ids), desc(updates.reshape(-1, width)), desc(out)
    _lib.check(lib.lb_scatter_add_rows(ctypes.byref(dx), ctypes.byref(di), ctypes.byref(du), ctypes.byref(do), scratch.data_ptr(),
                                       nbytes, int(deterministic), current_stream() if stream is None else stream))
    return out
