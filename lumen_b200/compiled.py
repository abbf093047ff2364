"""`compile(fn, device="cuda")`: the call surface of `lumen.compile` (lumen/graph/tracer.py:693-751) for this backend.

`fn` is traced into a graph on its first call with each input signature (the tensor arguments' dtypes and shapes),
the passes clean it, match attention and group its prims into fusions, `lb_compile` (the backend's C++ lowering) turns
the result into a plan with one workspace, and every call then runs the plan (`lowering="optimising"` selects the
Python lowering instead, which emits the same plan format). As in the reference the compiled function owns its memory: the workspace and the result tensors are allocated
once per signature, and each call returns the same result tensors, which the next call overwrites (`.clone()` one
to keep it). Tensor arguments that already live on the device are read in place; host tensors are copied in.
Non-tensor arguments are static: they are part of the signature.
"""

from __future__ import annotations

from lumen_b200 import tracer
from lumen_b200.compiler import compile_graph
from lumen_b200.device import Tensor as DeviceTensor
from lumen_b200.plan import Plan
from lumen_b200.runtime import _empty_like_input, dtype_name, require_cuda


def _is_torch(a) -> bool:
    return type(a).__module__.startswith("torch") and hasattr(a, "data_ptr")


def _is_tensor(a) -> bool:
    return isinstance(a, DeviceTensor) or _is_torch(a)


class _Signature:
    def __init__(self, fn, args, device, lowering="native"):
        tensor_at = [k for k, a in enumerate(args) if _is_tensor(a)]
        types = [(dtype_name(args[k].dtype), tuple(args[k].shape)) for k in tensor_at]

        def traced(*tensors):
            full = list(args)
            for k, t in zip(tensor_at, tensors):
                full[k] = t
            return fn(*full)

        self.graph = tracer.trace(traced, *types)
        if lowering == "native":
            from lumen_b200.attention_pass import match_attention
            from lumen_b200.fusion_pass import fuse
            from lumen_b200.simplify import clean

            self.plan = Plan.native(fuse(match_attention(clean(self.graph))), device=device)
            self.compiled = self.plan.compiled
        elif lowering == "optimising":
            self.compiled = compile_graph(self.graph)
            self.plan = Plan(self.compiled, device)
        else:
            raise ValueError("lowering must be \"native\" or \"optimising\"")
        like = args[tensor_at[0]] if tensor_at else DeviceTensor(0, (), "uint8")
        if _is_torch(like) and not like.is_cuda:
            like = like.to(device)
        # results live in the arguments' framework: torch tensors for a torch caller, the backend's own otherwise
        self.results = [_empty_like_input(like, self.graph.types[v].shape, self.graph.types[v].dtype) for v in self.graph.outputs]
        self.recorded = None
        self.bound_to = None


class Compiled:
    """What `compile` returns: called as `fn` is. `str()` gives the latest signature's traced program, `steps()`
    its plan steps (kind and label), `workspace_bytes` its workspace size."""

    def __init__(self, fn, device="cuda", use_graphs: bool = False, lowering: str = "native"):
        if not str(device).startswith("cuda"):
            raise ValueError("lumen_b200 compiles for device=\"cuda\" only (there is no CPU fallback)")
        self.fn, self.device, self.use_graphs, self.lowering = fn, device, use_graphs, lowering
        self.signatures: dict = {}
        self.latest: _Signature | None = None

    def __call__(self, *args):
        require_cuda()
        # any array that speaks DLPack (the reference's tensors import and export it, lumen/tensor/dlpack.rs) is taken
        # in place, without a copy when it already lives on this device
        if any(not _is_tensor(a) and hasattr(a, "__dlpack__") for a in args):
            import torch  # the DLPack importer of a harness that passes foreign arrays

            args = tuple(torch.from_dlpack(a) if not _is_tensor(a) and hasattr(a, "__dlpack__") else a for a in args)
        key = tuple((dtype_name(a.dtype), tuple(a.shape)) if _is_tensor(a) else ("static", a) for a in args)
        sig = self.signatures.get(key)
        if sig is None:
            sig = self.signatures[key] = _Signature(self.fn, args, self.device, self.lowering)
        self.latest = sig
        inputs = [a.to(self.device).contiguous() if _is_torch(a) else a for a in args if _is_tensor(a)]
        pointers = tuple(t.data_ptr() for t in inputs)
        if self.use_graphs and sig.bound_to == pointers and sig.recorded is not None:
            sig.recorded.launch()  # the same argument memory as the recorded call: one graph launch
        else:
            bound = sig.plan.bind(inputs, sig.results)
            sig.plan.run_bound(bound)
            if self.use_graphs and sig.bound_to == pointers:
                sig.recorded = sig.plan.record(bound)  # second call with these pointers: record for the next ones
            sig.bound_to, sig.keep = pointers, (inputs, bound)
        outs = sig.results
        return outs[0] if len(outs) == 1 else tuple(outs)

    def __str__(self) -> str:
        return self.latest.graph.to_text() if self.latest else "<not traced yet>"

    def steps(self):
        return self.latest.plan.steps() if self.latest else []

    def dump_code(self, directory: str) -> list[str]:
        """Writes the latest signature's traced program (`program.txt`), its plan (`plan.txt`) and the generated CUDA
        source of every fused kernel the plan runs, in the order it runs them (`NN_label.cu`), like the reference's
        `compiled.dump_code` (lumen/graph/tracer.py:739-741). Returns the paths written."""
        import ctypes
        import os
        import re

        from lumen_b200 import _lib

        if self.latest is None:
            raise RuntimeError("dump_code: the function has not been called yet")
        os.makedirs(directory, exist_ok=True)
        text = self.latest.compiled.text
        written = []
        for name, content in (("program.txt", self.latest.graph.to_text()), ("plan.txt", text)):
            path = os.path.join(directory, name)
            with open(path, "w") as f:
                f.write(content)
            written.append(path)
        modules = [m.split("\n", 1)[1].rsplit("endmodule", 1)[0] for m in re.findall(r"^module.*?^endmodule$", text, flags=re.S | re.M)]
        k = 0
        for line in text.split("\n"):
            tok = line.split()
            if len(tok) > 3 and tok[0] == "s" and tok[1] == "fusion":
                handle = ctypes.c_void_p()
                _lib.check(_lib.lib().lb_fusion_compile(modules[int(tok[3])].encode(), ctypes.byref(handle)))
                path = os.path.join(directory, f"{k:02d}_{tok[2]}.cu")
                with open(path, "w") as f:
                    f.write(_lib.lib().lb_fusion_source(handle).decode())
                written.append(path)
                k += 1
        return written

    @property
    def workspace_bytes(self) -> int:
        return self.latest.plan.workspace_bytes if self.latest else 0


def compile(fn, device="cuda", use_graphs: bool = False, lowering: str = "native") -> Compiled:  # noqa: A001 (the reference's name)
    """`fn` compiled for this backend: traced, fused, lowered to a plan on the first call with each input signature,
    which every call then runs (`lumen.compile`, lumen/graph/tracer.py:693-751). With `use_graphs`, calls that pass
    the same argument memory again replay a recorded CUDA graph. `lowering`: "native" (`lb_compile`) or "optimising"
    (the Python lowering)."""
    return Compiled(fn, device, use_graphs, lowering)
