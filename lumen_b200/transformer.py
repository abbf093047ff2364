"""The decoder transformer training step of the baseline configs as a traced lumen graph, and its runner.

Architecture (the reference's example, examples/transformer.py:88-170, with the baseline's choices): learned token
and position embeddings, pre-LayerNorm blocks (scale and bias, eps 1e-5) of causal multi-head flash attention and a
ReLU MLP, no linear biases, an untied head, mean next-token cross entropy, SGD (`p - lr * g`,
examples/optim.py:18-24). With bfloat16 parameters the matmuls accumulate in float32, LayerNorm statistics, softmax
and cross entropy run in float32, and the logits are float32.

One graph holds forward, backward and update: inputs `ids`, `targets`, then the parameters; outputs the loss, then
the updated parameters, donated into the parameters' buffers. In data-parallel runs every weight gradient is
all-reduced (sum) before the update, which then scales it by 1 / world size (lumen/distributed/__init__.py:171-178,
tests/distributed/test_placements.py:277-284).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from lumen_b200 import graph as G
from lumen_b200 import nn, prims
from lumen_b200.prims import TracedTensor


@dataclass
class Config:
    vocab: int = 256
    d_model: int = 128
    heads: int = 4
    hidden: int = 512
    layers: int = 2
    seq: int = 64
    dtype: str = "float32"
    lr: float = 1e-2
    logits_dtype: str = "float32"  # dtype the output head writes; the cross entropy always computes in float32
    optimizer: str = "sgd"         # "sgd" (examples/optim.py:7-24) or "adamw" (examples/optim.py:27-80)
    weight_decay: float = 1e-2     # AdamW only

    @staticmethod
    def baseline_small():
        """Config 1: the 2-layer float32 parity anchor."""
        return Config()

    @staticmethod
    def baseline_large():
        """Config 5: the 12-layer bfloat16 data-parallel training step. Logits are a bfloat16 activation like every other
        activation of the model (float32 accumulation in the head's GEMM, one rounding); the cross entropy widens them
        back to float32 in registers."""
        return Config(vocab=32768, d_model=1024, heads=16, hidden=4096, layers=12, seq=2048, dtype="bfloat16", logits_dtype="bfloat16")


def param_shapes(cfg: Config) -> list[tuple[str, tuple[int, ...]]]:
    d = cfg.d_model
    shapes = [("embed.tokens", (cfg.vocab, d)), ("embed.positions", (cfg.seq, d))]
    for layer in range(cfg.layers):
        p = f"layers.{layer}."
        shapes += [
            (p + "attn.norm.w", (d,)), (p + "attn.norm.b", (d,)), (p + "attn.wqkv", (3 * d, d)), (p + "attn.wo", (d, d)),
            (p + "mlp.norm.w", (d,)), (p + "mlp.norm.b", (d,)), (p + "mlp.w1", (cfg.hidden, d)), (p + "mlp.w2", (d, cfg.hidden)),
        ]  # fmt: skip
    shapes += [("norm.w", (d,)), ("norm.b", (d,)), ("head", (cfg.vocab, d))]
    return shapes


def init_params(cfg: Config, seed: int = 0) -> dict[str, np.ndarray]:
    """Weights N(0, 0.02) float32 (LayerNorm scale 1, bias 0), from `numpy.random.default_rng(seed)`."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in param_shapes(cfg):
        if name.endswith("norm.w"):
            out[name] = np.ones(shape, np.float32)
        elif name.endswith("norm.b"):
            out[name] = np.zeros(shape, np.float32)
        else:
            out[name] = (0.02 * rng.standard_normal(shape)).astype(np.float32)
    return out


def flops_per_step(cfg: Config, batch: int) -> float:
    """Matmul FLOPs (6 per parameter per token) plus causal attention (3.5 x forward) of one training step."""
    tokens = batch * cfg.seq
    matmul_params = cfg.layers * (4 * cfg.d_model**2 + 2 * cfg.d_model * cfg.hidden) + cfg.vocab * cfg.d_model
    attention = cfg.layers * 3.5 * (4 * batch * cfg.seq**2 * cfg.d_model / 2)
    return 6.0 * matmul_params * tokens + attention


def trace_train_step(cfg: Config, batch: int, world: int = 1, with_grads: bool = False, update: bool = True,
                     runtime_lr: bool = False):
    """The training step graph. Returns `(graph, names, donate)`: parameter names in input order (after `ids`,
    `targets`) and the output -> input donation map. With `with_grads` the (reduced) gradients are extra outputs.
    `update=False` traces forward and backward only: the outputs are the loss and the gradients, nothing is donated.
    With `cfg.optimizer == "adamw"` the float32 moments `m`, `v` of every parameter and the 0-d float32 step count
    follow the parameters as inputs, and the updated moments follow the updated parameters as outputs. With `runtime_lr`
    (SGD) the learning rate is the LAST input, a 0-d float32 tensor read by the update kernels, instead of a constant."""
    if runtime_lr and (cfg.optimizer != "sgd" or not update):
        raise ValueError("runtime_lr applies to the SGD update")
    if cfg.optimizer not in ("sgd", "adamw"):
        raise ValueError(f"optimizer must be \"sgd\" or \"adamw\", got {cfg.optimizer!r}")
    g = G.Graph()
    prims.push_graph(g)
    try:
        ids = TracedTensor(g, g.add_input("int64", (batch, cfg.seq)))
        targets = TracedTensor(g, g.add_input("int64", (batch, cfg.seq)))
        names = [n for n, _ in param_shapes(cfg)]
        params = {n: TracedTensor(g, g.add_input(cfg.dtype, s)) for n, s in param_shapes(cfg)}
        adamw = cfg.optimizer == "adamw"
        if adamw:
            m_in = {n: TracedTensor(g, g.add_input("float32", s)) for n, s in param_shapes(cfg)}
            v_in = {n: TracedTensor(g, g.add_input("float32", s)) for n, s in param_shapes(cfg)}
            count = TracedTensor(g, g.add_input("float32", ()))
        rate = TracedTensor(g, g.add_input("float32", ())) if runtime_lr else cfg.lr
        tape = nn.Tape()
        x = nn.embedding(tape, params["embed.tokens"], params["embed.positions"], ids)
        for layer in range(cfg.layers):
            p = f"layers.{layer}."
            h = nn.layer_norm(tape, x, params[p + "attn.norm.w"], params[p + "attn.norm.b"])
            qkv = nn.linear(tape, h, params[p + "attn.wqkv"])
            a = nn.attention(tape, qkv, batch, cfg.heads)
            x = nn.linear(tape, a, params[p + "attn.wo"], residual=x)
            h = nn.layer_norm(tape, x, params[p + "mlp.norm.w"], params[p + "mlp.norm.b"])
            u = nn.linear(tape, h, params[p + "mlp.w1"], relu=True)
            x = nn.linear(tape, u, params[p + "mlp.w2"], residual=x)
        x = nn.layer_norm(tape, x, params["norm.w"], params["norm.b"])
        logits = nn.linear(tape, x, params["head"], output_dtype=cfg.logits_dtype)
        loss = nn.cross_entropy_mean(tape, logits, targets.reshape(batch * cfg.seq), cfg.dtype)
        grads = tape.backward(loss)
        updated, reduced, new_m, new_v = [], [], [], []
        # Updates are traced in the order the backward pass produces the gradients (the head's first, the embeddings'
        # last), so that each gradient bucket's updates can run as soon as that bucket's all-reduce has landed; the
        # outputs keep the parameters' order.
        for n in reversed(names):
            gr = grads[params[n].var]
            if world > 1:
                gr = prims.device_wait(prims.all_reduce(gr, "sum", tuple(range(world))))
            reduced.append(gr)
            if not update:
                continue
            if adamw:
                p_new, mm, vv = nn.adamw_update(params[n], m_in[n], v_in[n], gr, count, lr=cfg.lr,
                                                weight_decay=cfg.weight_decay, grad_scale=1.0 / world)
                updated.append(p_new), new_m.append(mm), new_v.append(vv)
            else:
                updated.append(nn.sgd_update(params[n], gr, rate, 1.0 / world))
    finally:
        prims.pop_graph()
    updated, reduced, new_m, new_v = (lst[::-1] for lst in (updated, reduced, new_m, new_v))
    outputs = [loss, *updated, *new_m, *new_v] + (reduced if with_grads or not update else [])
    g.set_outputs([o.var for o in outputs])
    # output k is written into input donate[k]: parameters, then (AdamW) both moments
    donate = {1 + k: 2 + k for k in range(len(names) * (3 if adamw else 1))} if update else {}
    return g, names, donate


class TrainStep:
    """The compiled training step on one GPU (one rank of a data-parallel group), on the backend's own memory, stream
    and communicator: nothing here needs another CUDA framework.

    `device`: the GPU's index (or anything whose `.index` is it; `None` = the current device). `process_group`: a
    `lumen_b200.distributed.ProcessGroup` when `world > 1`; its NCCL communicator runs the plan's `all_reduce` steps on
    the plan's side stream while the rest of the backward pass continues, and each bucket's updates wait only for that
    bucket. `graphs`: "whole" replays the whole step as ONE recorded CUDA graph from the second step on; "segments"
    records the ranges between collectives and queues the collective steps themselves (the NCCL call and the event
    hand-offs) from the host; "off" queues every launch. `runtime_lr`: the SGD learning rate is a device scalar (`set_lr`)
    instead of a constant of the update kernel. `lowering`: "native" (the default: `lb_compile`, the backend's C++
    lowering of the module the passes leave) or "optimising" (`lumen_b200.compiler`, the same lowering on the Python side,
    which emits plan text); their plans give bit-identical results. A plan that holds collectives always runs as "segments":
    with NCCL 2.27.3 a step recorded WITH its all-reduces did not complete when replayed on two ranks (both ranks
    waited until the test's deadline; cause not established), so collectives are never recorded."""

    def __init__(self, cfg: Config, batch: int, params: dict[str, np.ndarray], device=None, world: int = 1, process_group=None,
                 bucket_bytes: int = 64 << 20, use_graphs: bool = True, deterministic: bool = True, graphs: str | None = None,
                 stream=None, autotune: bool = False, runtime_lr: bool = False, lowering: str = "native"):
        from lumen_b200 import device as D
        from lumen_b200.compiler import compile_graph
        from lumen_b200.plan import Plan

        index = getattr(device, "index", device)
        if index is not None:
            D.set_device(int(index))
        self.D = D
        self.cfg, self.batch, self.world, self.group = cfg, batch, world, process_group
        if world > 1 and process_group is None:
            raise ValueError("a data-parallel step (world > 1) needs a process group: lumen_b200.distributed.init_process_group()")
        self.graph, self.names, donate = trace_train_step(cfg, batch, world, runtime_lr=runtime_lr)
        # deterministic: colliding embedding-gradient rows are added in update order (bit-reproducible steps)
        native_handle = None
        if lowering == "native":
            # the backend's own C++ lowering (lb_compile) of the module the passes leave: same kernels, same placement
            # rules, the gradient buckets' collective steps included
            import json

            from lumen_b200.attention_pass import match_attention
            from lumen_b200.compiler import CompiledPlan
            from lumen_b200.fusion_pass import fuse
            from lumen_b200.plan import _bind, lower_native
            from lumen_b200.simplify import clean

            native_handle = lower_native(fuse(match_attention(clean(self.graph))), deterministic, donate, bucket_bytes)
            lib = _bind()
            steps = json.loads(lib.lb_plan_steps_json(native_handle).decode())
            self.compiled = CompiledPlan("", lib.lb_plan_workspace_bytes(native_handle), len(self.graph.inputs), len(self.graph.outputs),
                                         labels=[s["label"] for s in steps], kernel_launches=lib.lb_plan_kernel_launches(native_handle),
                                         buckets=[{} for _ in range(lib.lb_plan_num_collectives(native_handle))])
        elif lowering == "optimising":
            self.compiled = compile_graph(self.graph, donate, deterministic=deterministic, bucket_bytes=bucket_bytes)
        else:
            raise ValueError("lowering must be \"optimising\" or \"native\"")
        shapes = dict(param_shapes(cfg))
        itemsize = D.ITEMSIZE[cfg.dtype]
        state_bytes = sum(-(-int(np.prod(shapes[n])) * itemsize // 256) * 256 + 256 for n in self.names)
        if cfg.optimizer == "adamw":
            state_bytes += 2 * sum(-(-int(np.prod(shapes[n])) * 4 // 256) * 256 + 256 for n in self.names)
        # ONE reservation holds the workspace, the parameters, the optimizer state and the step's small buffers
        self.region = D.Region(max(self.compiled.workspace_bytes, 256) + state_bytes + 2 * batch * cfg.seq * 8 + (1 << 16))
        self.plan = Plan(self.compiled, region=self.region, handle=native_handle)
        # The step has a stream of its own (non-blocking): the legacy default stream would serialise it against every
        # blocking stream of the process, and NCCL work must never be ordered through stream 0.
        self.stream = stream if stream is not None else D.Stream()
        self.params = [self.region.empty(shapes[n], cfg.dtype, self.stream) for n in self.names]
        for n, p in zip(self.names, self.params):
            p.copy_from_host(_as_dtype(params[n], cfg.dtype), self.stream)
        self.loss = self.region.zeros((), "float32", self.stream)
        self.ids = self.region.zeros((batch, cfg.seq), "int64", self.stream)
        self.targets = self.region.zeros((batch, cfg.seq), "int64", self.stream)
        self.host_batch = D.HostBuffer(2 * batch * cfg.seq * 8)  # pinned staging for ids and targets
        self.moments, self.count = [], None
        if cfg.optimizer == "adamw":
            self.moments = [self.region.zeros(p.shape, "float32", self.stream) for p in self.params + self.params]
            self.count = self.region.zeros((), "float32", self.stream)
            self.count_host = 0.0
            self.count_ring = D.HostBuffer(64 * 4)  # pinned slots for the step count, one per queued step
        self.lr = None
        if runtime_lr:  # the learning rate as a device scalar the update kernels read: `set_lr` changes it between steps
            self.lr = self.region.zeros((), "float32", self.stream)
            self.lr_ring, self.lr_writes = D.HostBuffer(64 * 4), 0
            self.set_lr(cfg.lr)
        state = [*self.params, *self.moments]
        scalars = ([self.count] if self.count is not None else []) + ([self.lr] if self.lr is not None else [])
        self.bound = self.plan.bind([self.ids, self.targets, *state, *scalars], [self.loss, *state])
        if world > 1:
            self.plan.set_comm(process_group)
        self.buckets = list(self.compiled.buckets)
        # measured choice of each large GEMM's split count, tile raster and CTA pairing, on the step's own buffers
        self.tuning = self.plan.autotune(self.bound, self.stream.handle) if autotune else []
        # The first step runs launch by launch; later steps replay recorded CUDA graphs.
        self.graph_mode = graphs or ("whole" if use_graphs else "off")
        if self.graph_mode not in ("whole", "segments", "off"):
            raise ValueError("graphs must be \"whole\", \"segments\" or \"off\"")
        if self.graph_mode == "whole" and self.plan.num_collectives:
            self.graph_mode = "segments"
        self.use_graphs, self.steps_done, self.recorded = self.graph_mode != "off", 0, {}
        kinds = [s["kind"] for s in self.plan.steps()]
        # ranges for "segments": maximal runs of compute steps, and single collective / wait steps between them
        self.segments, start = [], 0
        for k, kind in enumerate(kinds + ["end"]):
            if kind in ("all_reduce", "wait", "end"):
                if k > start:
                    self.segments.append((start, k, True))
                if kind != "end":
                    self.segments.append((k, k + 1, False))
                start = k + 1
        self.stream.synchronize()

    def state_dict(self) -> dict[str, np.ndarray]:
        """The current parameters as host arrays by name (the form `init_params` gives and `save_file` takes); with
        AdamW also its moments and step count (`optimizer.m.<name>`, `optimizer.v.<name>`, `optimizer.step`)."""
        self.stream.synchronize()
        out = {}
        if self.count is not None:  # AdamW: both float32 moments of every parameter and the step count
            n = len(self.names)
            for k, name in enumerate(self.names):
                out[f"optimizer.m.{name}"] = self.moments[k].copy_to_host(stream=self.stream)
                out[f"optimizer.v.{name}"] = self.moments[n + k].copy_to_host(stream=self.stream)
            out["optimizer.step"] = self.count.copy_to_host(stream=self.stream)
        for name, p in zip(self.names, self.params):
            out[name] = p.copy_to_host(stream=self.stream)
        return out

    def load_state_dict(self, params: dict[str, np.ndarray]) -> None:
        """Overwrites the parameters in place (the plan keeps its bound buffers): every name, same shapes."""
        wanted = list(self.names)
        if self.count is not None:
            wanted += [f"optimizer.{k}.{n}" for k in "mv" for n in self.names] + ["optimizer.step"]
        missing = [n for n in wanted if n not in params]
        extra = [n for n in params if n not in wanted]
        if missing or extra:
            raise KeyError(f"load_state_dict: missing {missing}, unexpected {extra}")
        if self.count is not None:
            n = len(self.names)
            for k, name in enumerate(self.names):
                self.moments[k].copy_from_host(np.ascontiguousarray(params[f"optimizer.m.{name}"], np.float32), self.stream)
                self.moments[n + k].copy_from_host(np.ascontiguousarray(params[f"optimizer.v.{name}"], np.float32), self.stream)
            self.count_host = float(np.asarray(params["optimizer.step"], dtype=np.float32))
            self.count.copy_from_host(np.asarray(self.count_host, dtype=np.float32), self.stream)
        for name, p in zip(self.names, self.params):
            value = params[name]
            if tuple(value.shape) != tuple(p.shape):
                raise ValueError(f"load_state_dict: `{name}` has shape {tuple(value.shape)}, the model's is {tuple(p.shape)}")
            p.copy_from_host(_as_dtype(value, self.cfg.dtype), self.stream)

    def save_checkpoint(self, filename, metadata: dict[str, str] | None = None) -> None:
        """The parameters as a safetensors file, written through a temporary file renamed over `filename`."""
        from lumen_b200.safetensors import save_file

        save_file(self.state_dict(), filename, {"steps": str(self.steps_done), **(metadata or {})})

    def load_checkpoint(self, filename) -> None:
        from lumen_b200.safetensors import load_file

        self.load_state_dict(load_file(filename))

    def load_batch(self, ids, targets):
        """Copies this step's token ids and targets (`[batch, seq]` int64 host arrays) to the device through pinned
        memory, asynchronously on the step's stream. The previous copy must have been consumed (a step queued and, when
        the caller reuses the staging buffer every step, finished)."""
        n = self.batch * self.cfg.seq
        stage = self.host_batch.array(np.int64, (2, n))
        stage[0] = _host_array(ids).reshape(n)
        stage[1] = _host_array(targets).reshape(n)
        lib = self.ids.lib
        from lumen_b200 import _lib

        _lib.check(lib.lb_copy_to_device(self.ids.ptr, self.host_batch.ptr, n * 8, self.stream.handle))
        _lib.check(lib.lb_copy_to_device(self.targets.ptr, self.host_batch.ptr + n * 8, n * 8, self.stream.handle))

    def set_lr(self, value: float) -> None:
        """The learning rate of the steps queued from now on (`runtime_lr=True`): an asynchronous 4-byte copy from pinned
        memory on the step's stream, ordered after the steps already queued. Up to 64 changes may be in flight."""
        if self.lr is None:
            raise RuntimeError("this step was compiled with a constant learning rate: pass runtime_lr=True")
        from lumen_b200 import _lib

        slot = self.lr_writes % 64
        self.lr_writes += 1
        self.lr_ring.array(np.float32, (64,))[slot] = value
        _lib.check(self.lr.lib.lb_copy_to_device(self.lr.ptr, self.lr_ring.ptr + 4 * slot, 4, self.stream.handle))

    def _run(self, first, last, record=True):
        """Steps [first, last) on the step's stream: launch by launch on the first step, replayed afterwards."""
        if not self.use_graphs or self.steps_done == 0 or not record:
            self.plan.run_bound(self.bound, first, last, self.stream.handle)
            return
        key = (first, last)
        if key not in self.recorded:
            self.recorded[key] = self.plan.record(self.bound, first, last)
        self.recorded[key].launch(self.stream.handle)

    def step(self):
        """Queues one training step on the step's stream and returns the (device) loss. With several ranks, gradient
        buckets are all-reduced on the plan's side stream while the rest of the backward pass runs; each bucket's
        updates wait for that bucket only."""
        if self.count is not None:
            # AdamW's bias corrections are computed from the step count inside the update kernels
            self.count_host += 1.0
            slot = self.steps_done % 64  # asynchronous copy from pinned memory: up to 64 steps may be queued ahead
            self.count_ring.array(np.float32, (64,))[slot] = self.count_host
            from lumen_b200 import _lib

            _lib.check(self.count.lib.lb_copy_to_device(self.count.ptr, self.count_ring.ptr + 4 * slot, 4, self.stream.handle))
        if self.graph_mode == "segments" and self.plan.num_collectives:
            for first, last, compute in self.segments:
                self._run(first, last, record=compute)
        else:
            self._run(0, -1)
        self.steps_done += 1
        return self.loss

    def synchronize(self, timeout: float | None = None) -> None:
        """Waits for the queued steps; with a process group, with a deadline and NCCL's error state polled meanwhile."""
        if self.group is not None and self.world > 1:
            self.group.synchronize(self.stream, timeout)
        else:
            self.stream.synchronize()


def _host_array(x) -> np.ndarray:
    """A NumPy view of a host array of another framework (`.numpy()`) or of NumPy's own."""
    if isinstance(x, np.ndarray):
        return x
    if hasattr(x, "numpy"):
        return x.numpy()
    return np.asarray(x)


def _as_dtype(a: np.ndarray, dtype: str) -> np.ndarray:
    """`a` as a contiguous host array of the lumen dtype `dtype` (bfloat16 through ml_dtypes, one rounding)."""
    if dtype == "bfloat16":
        import ml_dtypes

        return np.ascontiguousarray(a if a.dtype == ml_dtypes.bfloat16 else np.asarray(a, np.float32).astype(ml_dtypes.bfloat16))
    return np.ascontiguousarray(a, dtype=np.dtype(dtype))
