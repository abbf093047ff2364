"""A compiled plan bound to the C ABI: `lb_plan_create` once, then `lb_plan_run` per call over device memory (inputs,
outputs and the one workspace). Mirrors the reference's Python `Plan` (`run_in`, `steps`, `workspace_bytes`;
lumen/graph_compiler/python.rs:38-191). The workspace comes from the backend's own region allocator
(`lumen_b200.device`) unless the caller hands one over; inputs and outputs are anything with `data_ptr()`."""

from __future__ import annotations

import ctypes
import json

from lumen_b200 import _lib
from lumen_b200.compiler import CompiledPlan
from lumen_b200.runtime import current_stream, require_cuda


def _bind():
    lib = _lib.lib()
    if getattr(lib, "_plan_bound", False):
        return lib
    lib.lb_plan_create.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.lb_plan_destroy.argtypes = [ctypes.c_void_p]
    lib.lb_plan_workspace_bytes.argtypes = [ctypes.c_void_p]
    lib.lb_plan_workspace_bytes.restype = ctypes.c_size_t
    lib.lb_plan_workspace_alignment.argtypes = [ctypes.c_void_p]
    lib.lb_plan_workspace_alignment.restype = ctypes.c_size_t
    lib.lb_plan_num_steps.argtypes = [ctypes.c_void_p]
    lib.lb_plan_steps_json.argtypes = [ctypes.c_void_p]
    lib.lb_plan_steps_json.restype = ctypes.c_char_p
    lib.lb_plan_text.argtypes = [ctypes.c_void_p]
    lib.lb_plan_text.restype = ctypes.c_char_p
    lib.lb_plan_run.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
    ]  # fmt: skip
    lib.lb_plan_capture.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
    ]  # fmt: skip
    lib.lb_graph_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.lb_graph_destroy.argtypes = [ctypes.c_void_p]
    lib.lb_plan_set_comm.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.lb_plan_num_collectives.argtypes = [ctypes.c_void_p]
    lib.lb_plan_kernel_launches.argtypes = [ctypes.c_void_p]
    lib.lb_plan_autotune.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
        ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t,
    ]  # fmt: skip
    lib._plan_bound = True
    return lib


class RecordedRange:
    """A step range of a plan recorded as a CUDA graph (`lb_plan_capture`); `launch()` replays it."""

    def __init__(self, plan: "Plan", bound, first=0, last=-1):
        self.lib = plan.lib
        self.keep = (plan, bound)  # the recording refers to their memory
        self.handle = ctypes.c_void_p()
        ins, n_in, outs, n_out = bound
        _lib.check(self.lib.lb_plan_capture(plan.handle, plan.workspace.data_ptr(), ins, n_in, outs, n_out, first, last, ctypes.byref(self.handle)))

    def launch(self, stream=None):
        _lib.check(self.lib.lb_graph_launch(self.handle, current_stream() if stream is None else stream))

    def __del__(self):
        try:
            if self.handle:
                self.lib.lb_graph_destroy(self.handle)
        except Exception:
            pass


class LbConfig(ctypes.Structure):
    _fields_ = [("deterministic", ctypes.c_int32), ("n_donate", ctypes.c_int32), ("donate", ctypes.POINTER(ctypes.c_int32)),
                ("bucket_bytes", ctypes.c_int64), ("reserved", ctypes.c_int32 * 2)]


def lower_native(graph, deterministic: bool = True, donate: dict[int, int] | None = None, bucket_bytes: int = 0) -> ctypes.c_void_p:
    """`lb_compile` on a graph that has been through the passes (its work in `fusion` nodes): the backend's own C++
    lowering to a plan. `donate` maps output indices to the inputs whose memory they are written into. Returns the plan
    handle; needs no GPU (kernels are generated and compiled, not loaded)."""
    lib = _bind()
    lib.lb_compile.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(LbConfig), ctypes.POINTER(ctypes.c_void_p)]
    pairs = [x for item in sorted((donate or {}).items()) for x in item]
    array = (ctypes.c_int32 * max(len(pairs), 1))(*pairs)
    config = LbConfig(deterministic=int(deterministic), n_donate=len(pairs) // 2, donate=array, bucket_bytes=int(bucket_bytes))
    handle = ctypes.c_void_p()
    _lib.check(lib.lb_compile(graph.to_text().encode(), -1, ctypes.byref(config), ctypes.byref(handle)))
    return handle


class Plan:
    def __init__(self, compiled: CompiledPlan, device=None, workspace=None, region=None, handle=None):
        """`workspace`: device memory of at least `workspace_bytes` (anything with `data_ptr()`), else it is taken from
        `region` (a `lumen_b200.device.Region`), else from a region made for it. `device` is accepted for callers that
        name one; the plan runs on the current device. `handle`: a plan the backend has already built (`lower_native`)."""
        require_cuda()
        self.compiled = compiled
        self.lib = _bind()
        self.handle = handle if handle is not None else ctypes.c_void_p()
        if handle is None:
            _lib.check(self.lib.lb_plan_create(compiled.text.encode(), ctypes.byref(self.handle)))
        self.workspace_bytes = self.lib.lb_plan_workspace_bytes(self.handle)
        if workspace is None:
            from lumen_b200.device import Region

            self.region = region if region is not None else Region(max(self.workspace_bytes, 256) + 256)
            workspace = self.region.empty((max(self.workspace_bytes, 256),), "uint8")
        self.workspace = workspace
        if self.workspace.data_ptr() % self.lib.lb_plan_workspace_alignment(self.handle):
            raise ValueError("the workspace must be 256-byte aligned")
        self.num_steps = self.lib.lb_plan_num_steps(self.handle)
        self.num_collectives = self.lib.lb_plan_num_collectives(self.handle)

    @classmethod
    def native(cls, graph, deterministic: bool = True, donate: dict[int, int] | None = None, **kwargs) -> "Plan":
        """The plan `lb_compile` (the backend's C++ lowering) makes of a graph that has been through the passes."""
        handle = lower_native(graph, deterministic, donate)
        lib = _bind()
        labels = [s["label"] for s in json.loads(lib.lb_plan_steps_json(handle).decode())]
        compiled = CompiledPlan(lib.lb_plan_text(handle).decode(), lib.lb_plan_workspace_bytes(handle), len(graph.inputs),
                                len(graph.outputs), labels=labels, kernel_launches=lib.lb_plan_kernel_launches(handle))
        return cls(compiled, handle=handle, **kwargs)

    def set_comm(self, group) -> None:
        """Binds the communicator the plan's `all_reduce` steps use (a `lumen_b200.distributed.ProcessGroup`)."""
        self.group = group
        _lib.check(self.lib.lb_plan_set_comm(self.handle, group.comm if group is not None else None))

    def steps(self):
        return json.loads(self.lib.lb_plan_steps_json(self.handle).decode())

    def bind(self, inputs, outputs):
        """Pointer arrays for a fixed set of input/output tensors (reuse them across runs)."""
        ins = (ctypes.c_void_p * len(inputs))(*[t.data_ptr() for t in inputs])
        outs = (ctypes.c_void_p * len(outputs))(*[t.data_ptr() for t in outputs])
        return ins, len(inputs), outs, len(outputs)

    def run_bound(self, bound, first=0, last=-1, stream=None):
        ins, n_in, outs, n_out = bound
        _lib.check(
            self.lib.lb_plan_run(
                self.handle, self.workspace.data_ptr(), ins, n_in, outs, n_out, first, last,
                current_stream() if stream is None else stream,
            )
        )  # fmt: skip

    def autotune(self, bound, stream=None) -> list:
        """Times the candidate configurations of the plan's large GEMM steps on its own buffers and keeps the fastest
        (`lb_plan_autotune`). Call before the first real run: the workspace and the outputs are overwritten. Returns the
        report: one entry per tuned step (shape, candidates, what was picked, microseconds picked / default)."""
        ins, n_in, outs, n_out = bound
        report = ctypes.create_string_buffer(1 << 20)
        _lib.check(self.lib.lb_plan_autotune(self.handle, self.workspace.data_ptr(), ins, n_in, outs, n_out,
                                             current_stream() if stream is None else stream, report, len(report)))
        return json.loads(report.value.decode() or "[]")

    def profile(self, bound, stream=None, repeats=2) -> list:
        """Times every step of the plan launched alone (events around each single-step run on `stream`, the last of
        `repeats` passes kept): `[(label, milliseconds)]` in plan order - the counterpart of the reference's per-step
        profile (lumen/plan/run.rs:247-427 brackets each step the same way). Collective steps need their communicator
        and every rank calling in; single launches run at higher clocks than a power-capped whole step."""
        from lumen_b200 import device as D

        s = stream if stream is not None else None
        times = []
        for rep in range(repeats):
            times = []
            for i, label in enumerate(self.compiled.labels):
                e0, e1 = D.Event(timing=True), D.Event(timing=True)
                e0.record(s)
                self.run_bound(bound, i, i + 1, s.handle if s is not None else None)
                e1.record(s)
                e1.synchronize()
                times.append((label, e0.elapsed_ms(e1)))
        return times

    def record(self, bound, first=0, last=-1) -> RecordedRange:
        """Records steps [first, last) over `bound` as a CUDA graph. Run the range once beforehand."""
        return RecordedRange(self, bound, first, last)

    def run(self, inputs, outputs, first=0, last=-1, stream=None):
        self.run_bound(self.bind(inputs, outputs), first, last, stream)

    def workspace_view(self, view):
        """A `lumen_b200.device.Tensor` over a dense workspace region of the plan (e.g. a gradient in the arena)."""
        from lumen_b200.device import Tensor

        start = view.buffer.offset + view.offset
        return Tensor(self.workspace.data_ptr() + start, view.shape, view.dtype, owner=self.workspace)

    def __del__(self):
        try:
            if self.handle:
                self.lib.lb_plan_destroy(self.handle)
        except Exception:
            pass
