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


def trace_train_step(cfg: Config, batch: int, world: int = 1, with_grads: bool = False, update: bool = True):
    """The training step graph. Returns `(graph, names, donate)`: parameter names in input order (after `ids`,
    `targets`) and the output -> input donation map. With `with_grads` the (reduced) gradients are extra outputs.
    `update=False` traces forward and backward only: the outputs are the loss and the gradients, nothing is donated.
    With `cfg.optimizer == "adamw"` the float32 moments `m`, `v` of every parameter and the 0-d float32 step count
    follow the parameters as inputs, and the updated moments follow the updated parameters as outputs."""
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
        for n in names:
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
                updated.append(nn.sgd_update(params[n], gr, cfg.lr, 1.0 / world))
    finally:
        prims.pop_graph()
    outputs = [loss, *updated, *new_m, *new_v] + (reduced if with_grads or not update else [])
    g.set_outputs([o.var for o in outputs])
    # output k is written into input donate[k]: parameters, then (AdamW) both moments
    donate = {1 + k: 2 + k for k in range(len(names) * (3 if adamw else 1))} if update else {}
    return g, names, donate


class TrainStep:
    """The compiled training step on one GPU (one rank of a data-parallel group)."""

    def __init__(self, cfg: Config, batch: int, params: dict[str, np.ndarray], device, world: int = 1, process_group=None,
                 bucket_bytes: int = 64 << 20, use_graphs: bool = True, deterministic: bool = True):
        import torch

        from lumen_b200.compiler import compile_graph
        from lumen_b200.plan import Plan
        from lumen_b200.runtime import TORCH_DTYPES

        self.torch = torch
        self.cfg, self.batch, self.world, self.group = cfg, batch, world, process_group
        self.graph, self.names, donate = trace_train_step(cfg, batch, world)
        # deterministic: colliding embedding-gradient rows are added in update order (bit-reproducible steps)
        self.compiled = compile_graph(self.graph, donate, deterministic=deterministic)
        self.plan = Plan(self.compiled, device)
        td = TORCH_DTYPES[cfg.dtype]
        self.params = [torch.from_numpy(params[n]).to(device).to(td).contiguous() for n in self.names]
        self.loss = torch.zeros((), dtype=torch.float32, device=device)
        self.ids = torch.zeros((batch, cfg.seq), dtype=torch.int64, device=device)
        self.targets = torch.zeros((batch, cfg.seq), dtype=torch.int64, device=device)
        self.moments, self.count = [], None
        if cfg.optimizer == "adamw":
            self.moments = [torch.zeros(p.shape, dtype=torch.float32, device=device) for p in self.params + self.params]
            self.count = torch.zeros((), dtype=torch.float32, device=device)
        state = [*self.params, *self.moments]
        self.bound = self.plan.bind([self.ids, self.targets, *state, *([self.count] if self.count is not None else [])],
                                    [self.loss, *state])
        # The first step runs launch by launch; later steps replay each step range (the ranges between the
        # host-issued collectives) as a recorded CUDA graph.
        self.use_graphs, self.steps_done, self.recorded = use_graphs, 0, {}
        self.buckets = []
        if world > 1:
            self.comm_stream = torch.cuda.Stream(device=device)
            self.buckets = self._buckets(bucket_bytes, td)

    def _buckets(self, bucket_bytes, td):
        """The gradient arena cut into buckets, each one flat tensor reduced as soon as its last gradient has been
        queued (alignment padding between gradients is reduced along with them and never read)."""
        from lumen_b200.compiler import gradient_buckets

        buckets = gradient_buckets(self.compiled, bucket_bytes)
        for b in buckets:
            b["tensor"] = self.plan.workspace[b["start"] : b["end"]].view(td)
        return buckets

    def state_dict(self) -> dict[str, np.ndarray]:
        """The current parameters as host arrays by name (the form `init_params` gives and `save_file` takes); with
        AdamW also its moments and step count (`optimizer.m.<name>`, `optimizer.v.<name>`, `optimizer.step`)."""
        self.torch.cuda.current_stream().synchronize()
        out = {}
        if self.count is not None:  # AdamW: both float32 moments of every parameter and the step count
            n = len(self.names)
            for k, name in enumerate(self.names):
                out[f"optimizer.m.{name}"] = self.moments[k].detach().cpu().numpy().copy()
                out[f"optimizer.v.{name}"] = self.moments[n + k].detach().cpu().numpy().copy()
            out["optimizer.step"] = self.count.detach().cpu().numpy().copy()
        for name, p in zip(self.names, self.params):
            host = p.detach().cpu().contiguous()
            if host.dtype == self.torch.bfloat16:
                import ml_dtypes

                out[name] = host.view(self.torch.uint16).numpy().view(ml_dtypes.bfloat16).copy()
            else:
                out[name] = host.numpy().copy()
        return out

    def load_state_dict(self, params: dict[str, np.ndarray]) -> None:
        """Overwrites the parameters in place (the plan keeps its bound buffers): every name, same shapes."""
        torch = self.torch
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
                self.moments[k].copy_(torch.from_numpy(np.ascontiguousarray(params[f"optimizer.m.{name}"])))
                self.moments[n + k].copy_(torch.from_numpy(np.ascontiguousarray(params[f"optimizer.v.{name}"])))
            self.count.copy_(torch.from_numpy(np.asarray(params["optimizer.step"], dtype=np.float32)))
        for name, p in zip(self.names, self.params):
            value = params[name]
            if tuple(value.shape) != tuple(p.shape):
                raise ValueError(f"load_state_dict: `{name}` has shape {tuple(value.shape)}, the model's is {tuple(p.shape)}")
            if value.dtype.name == "bfloat16":
                host = torch.from_numpy(np.ascontiguousarray(value).view(np.uint16).copy()).view(torch.bfloat16)
            else:
                host = torch.from_numpy(np.ascontiguousarray(value))
            p.copy_(host.to(p.dtype))

    def save_checkpoint(self, filename, metadata: dict[str, str] | None = None) -> None:
        """The parameters as a safetensors file, written through a temporary file renamed over `filename`."""
        from lumen_b200.safetensors import save_file

        save_file(self.state_dict(), filename, {"steps": str(self.steps_done), **(metadata or {})})

    def load_checkpoint(self, filename) -> None:
        from lumen_b200.safetensors import load_file

        self.load_state_dict(load_file(filename))

    def load_batch(self, ids, targets):
        self.ids.copy_(ids, non_blocking=True)
        self.targets.copy_(targets, non_blocking=True)

    def _run(self, first, last):
        """Steps [first, last) on the current stream: launch by launch on the first step, replayed afterwards."""
        if not self.use_graphs or self.steps_done == 0:
            self.plan.run_bound(self.bound, first, last)
            return
        key = (first, last)
        if key not in self.recorded:
            self.recorded[key] = self.plan.record(self.bound, first, last)
        self.recorded[key].launch()

    def step(self):
        """Queues one training step on the current stream. With several ranks, gradient buckets are all-reduced on
        a side stream while the rest of the backward pass runs; the update waits for them."""
        if self.count is not None:
            self.count.add_(1.0)  # AdamW's bias corrections are computed from the step count inside the update kernels
        self._step()
        self.steps_done += 1
        return self.loss

    def _step(self):
        torch = self.torch
        if not self.buckets:
            self._run(0, -1)
            return
        import torch.distributed as dist

        main = torch.cuda.current_stream()
        at = 0
        done = []
        for b in self.buckets:
            if b["ready"] > at:
                self._run(at, b["ready"])
                at = b["ready"]
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                dist.all_reduce(b["tensor"], op=dist.ReduceOp.SUM, group=self.group)
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                done.append(ev)
        # everything after the last gradient: wait for the reductions, then update
        update_from = max(c.ready_step for c in self.compiled.comms)
        if update_from > at:
            self._run(at, update_from)
            at = update_from
        for ev in done:
            main.wait_event(ev)
        self._run(at, -1)
