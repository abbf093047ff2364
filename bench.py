"""Benchmark of the lumen_b200 hot path. Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (synthetic inputs with the shapes, seeds and distributions the baseline configs name):
  fused_chain_f32 / fused_chain_bf16
      y = relu(x*g + b) and the row-wise sum of squares of y as ONE generated kernel; x [16384, 4096].
      Metric: GB/s of algorithmic bytes (x, g, b read; y, s written).

Timing: W warm-up steps, then K steps between a barrier + synchronize on both sides, CUDA events on the launching
stream, max over ranks. Each step touches more bytes than the 126 MB L2 and steps rotate over three buffer sets, so
no step finds its inputs in L2. `e2e` repeats the measurement through the same C-ABI call with pinned HOST buffers:
inputs copied to the device and outputs copied back inside the timed region, every step.
`--impl reference` times the CPU restatement of the reference interpreter (oracle/, kind "port": the reference is
Rust and cannot be built here) on a bounded sample of the same workload, on this machine's host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


# ---- workload: fused chain ------------------------------------------------------------------------------------
def chain_graph(rows, cols, dtype):
    from lumen_b200 import functional as F
    from lumen_b200 import prims, tracer

    def chain(x, g, b):
        y = F.relu(x * g + b)
        return y, prims.reduce_sum(y * y, (1,), "float32")

    return tracer.trace(chain, (dtype, (rows, cols)), (dtype, (cols,)), (dtype, (cols,)))


def chain_inputs(rows, cols, dtype, seed=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    g = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32)
    return x, g, b


def chain_bytes(rows, cols, dtype):
    size = 4 if dtype == "float32" else 2
    return rows * cols * size * 2 + 2 * cols * size + rows * 4


class FusedChain:
    rows, cols = 16384, 4096
    sets = 3

    def __init__(self, dtype):
        self.dtype = dtype
        self.name = "fused_chain_f32" if dtype == "float32" else "fused_chain_bf16"
        self.metric = "fused elementwise+row-reduction throughput (algorithmic bytes)"
        self.unit = "GB/s"
        self.arith = "f32" if dtype == "float32" else "bf16"
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from an ncu capture of this workload (part of y
        # is still in L2 when the kernel ends); a recorded figure, not measured by this run
        self.traffic = 487.3e6 if dtype == "float32" else 217.0e6
        self.traffic_source = "ncu capture of one launch of this workload (recorded constant, summary under profiles/)"

    def units_per_step(self):
        return chain_bytes(self.rows, self.cols, self.dtype) / 1e9

    def setup(self, device, host=True):
        """`host=False` skips the pinned host buffers of the end-to-end leg (device-only measurement)."""
        import torch

        from lumen_b200.runtime import TORCH_DTYPES, Fusion

        self.torch = torch
        self.fusion = Fusion(chain_graph(self.rows, self.cols, self.dtype))
        td = TORCH_DTYPES[self.dtype]
        x, g, b = chain_inputs(self.rows, self.cols, self.dtype)
        pin = (lambda t: t.pin_memory()) if host else (lambda t: t)
        self.host_in = [pin(torch.from_numpy(a).to(td)) for a in (x, g, b)]
        self.dev_in = []
        for k in range(self.sets):
            xs = self.host_in[0].to(device)
            if k:
                xs = xs.roll(k, 0).contiguous()
            self.dev_in.append([xs, self.host_in[1].to(device), self.host_in[2].to(device)])
        self.dev_out = [
            [torch.empty((self.rows, self.cols), dtype=td, device=device), torch.empty((self.rows,), dtype=torch.float32, device=device)]
            for _ in range(self.sets)
        ]
        self.host_out = [torch.empty((self.rows, self.cols), dtype=td).pin_memory(), torch.empty((self.rows,), dtype=torch.float32).pin_memory()] if host else []
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = sum(t.numel() * t.element_size() for t in self.host_out)
        self.launches_per_step = 1

    def step(self, i):
        k = i % self.sets
        self.fusion(*self.dev_in[k], out=self.dev_out[k])

    def e2e_step(self, i):
        k = i % self.sets
        for d, h in zip(self.dev_in[k], self.host_in):
            d.copy_(h, non_blocking=True)
        self.fusion(*self.dev_in[k], out=self.dev_out[k])
        for h, d in zip(self.host_out, self.dev_out[k]):
            h.copy_(d, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def cpu_sample(self, rows=None):
        """Times the oracle on `rows` rows of the same workload; returns (GB/s, cores, description)."""
        from oracle import oracle

        rows = rows or 4096
        g = chain_graph(rows, self.cols, self.dtype)
        x, gg, b = chain_inputs(rows, self.cols, self.dtype, seed=1)
        if self.dtype == "bfloat16":
            x, gg, b = (a.astype(oracle.BF16) for a in (x, gg, b))
        oracle.run(g, [x, gg, b])  # warm the library
        t0 = time.perf_counter()
        oracle.run(g, [x, gg, b])
        dt = time.perf_counter() - t0
        return chain_bytes(rows, self.cols, self.dtype) / 1e9 / dt, oracle.threads(), f"{rows} of {self.rows} rows, oracle interpreter, OpenMP"


class MatmulBackward:
    """F.matmul bf16 x bf16 -> float32 (float32 accumulation) and its transpose-rule backward
    (lumen/autograd/rules.py:463-486): dA = bf16(dY) . B^T and dB = A^T . bf16(dY), both rounded once to bf16.
    M = N = K = 8192: three GEMMs of 2 * 8192^3 FLOP per step."""

    n = 8192
    rows = cols = 8192

    def __init__(self):
        self.name = "matmul_bf16_8192_fwd_bwd"
        self.metric = "bf16 matmul (fp32 accumulate) forward + backward throughput"
        self.unit = "TFLOP/s"
        self.arith = "bf16"
        self.launches_per_step = 3

    def units_per_step(self):
        return 3 * 2 * self.n**3 / 1e12

    def setup(self, device, host=True):
        import torch

        from lumen_b200.runtime import gemm

        self.torch, self.gemm = torch, gemm
        n = self.n
        gen = torch.Generator(device="cpu").manual_seed(2)
        pin = (lambda t: t.pin_memory()) if host else (lambda t: t)
        self.host_in = [pin((torch.randn((n, n), generator=gen) / n**0.5).bfloat16()) for _ in range(2)]
        self.host_in.append(pin(torch.randn((n, n), generator=gen).bfloat16()))  # dY already narrowed to bf16
        self.a, self.b, self.dy = (t.to(device) for t in self.host_in)
        self.y = torch.empty((n, n), dtype=torch.float32, device=device)
        self.da = torch.empty((n, n), dtype=torch.bfloat16, device=device)
        self.db = torch.empty((n, n), dtype=torch.bfloat16, device=device)
        self.host_out = ([torch.empty((n, n), dtype=torch.float32).pin_memory()] + [torch.empty((n, n), dtype=torch.bfloat16).pin_memory() for _ in range(2)]) if host else []
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = sum(t.numel() * t.element_size() for t in self.host_out)

    def step(self, i):
        self.gemm(self.a, self.b, self.y)
        self.gemm(self.dy, self.b.t(), self.da)
        self.gemm(self.a.t(), self.dy, self.db)

    def e2e_step(self, i):
        for d, h in zip((self.a, self.b, self.dy), self.host_in):
            d.copy_(h, non_blocking=True)
        self.step(i)
        for h, d in zip(self.host_out, (self.y, self.da, self.db)):
            h.copy_(d, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def roofline(self, peaks, kernel_ms):
        achieved = 2 * self.n**3 / 1e12 / (kernel_ms / 1e3)
        return {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_tflops"], "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                "traffic": 1.43e9, "traffic_source": "ncu capture of the forward launch (recorded constant, summary under profiles/)",
                "kernel": "gemm_tcgen05_pair", "flops_per_launch": 2 * self.n**3}  # fmt: skip

    def cpu_sample(self, n=1024):
        """The oracle's dot_general (sequential fp32 accumulation, OpenMP over rows) on an n^3 sample."""
        from lumen_b200 import functional as F
        from lumen_b200 import tracer
        from oracle import oracle

        g = tracer.trace(lambda x, y: F.matmul(x, y, "float32", "float32"), ("bfloat16", (n, n)), ("bfloat16", (n, n)))
        rng = np.random.default_rng(2)
        a, b = ((rng.standard_normal((n, n)) / n**0.5).astype(np.float32).astype(oracle.BF16) for _ in range(2))
        t0 = time.perf_counter()
        oracle.run(g, [a, b])
        dt = time.perf_counter() - t0
        return 2 * n**3 / 1e12 / dt, oracle.threads(), f"one {n}^3 bf16 GEMM of the 3 x 8192^3 per step, oracle dot_general, OpenMP"


class FlashAttention:
    """Causal flash attention forward + backward, batch 8, 32 heads, sequence 4096, head dim 128, bf16 with fp32
    accumulation and fp32 log-sum-exp. FLOPs by the reference dashboard's convention (dashboard/bench.py:284-285):
    forward 4*B*H*S^2*D/2, backward 2.5x that."""

    def __init__(self, b=8, h=32, s=4096, d=128):
        self.b, self.h, self.s, self.d = b, h, s, d
        self.rows, self.cols = b * s, h * d
        self.name = f"flash_attention_causal_b{b}_h{h}_s{s}_d{d}_fwd_bwd"
        self.metric = "causal flash attention forward + backward throughput"
        self.unit = "TFLOP/s"
        self.arith = "bf16"
        # LUMEN_B200_DETERMINISTIC=0: the backward as one kernel with atomic dQ (head dim 64), the reference backend's default mode
        self.deterministic = os.environ.get("LUMEN_B200_DETERMINISTIC", "0") != "0"
        self.launches_per_step = 4  # forward, delta, dK/dV, dQ (or: forward, delta, the single-kernel backward, dQ rounding)

    def fwd_flops(self):
        return 4 * self.b * self.h * self.s * self.s * self.d / 2

    def units_per_step(self):
        return 3.5 * self.fwd_flops() / 1e12

    def setup(self, device, host=True):
        import torch

        from lumen_b200 import runtime

        self.torch, self.rt = torch, runtime
        shape = (self.b, self.s, self.h, self.d)
        gen = torch.Generator(device="cpu").manual_seed(3)
        pin = (lambda t: t.pin_memory()) if host else (lambda t: t)
        self.host_in = [pin(torch.randn(shape, generator=gen).bfloat16()) for _ in range(4)]  # q, k, v, dO
        self.q, self.k, self.v, self.do = (t.to(device) for t in self.host_in)
        self.o = torch.empty(shape, dtype=torch.bfloat16, device=device)
        self.lse = torch.empty((self.b, self.h, self.s), dtype=torch.float32, device=device)
        self.delta = torch.empty_like(self.lse)
        self.grads = None
        self.host_out = [torch.empty(shape, dtype=torch.bfloat16).pin_memory() for _ in range(4)] if host else []  # o, dq, dk, dv
        self.h2d = sum(t.numel() * t.element_size() for t in self.host_in)
        self.d2h = sum(t.numel() * t.element_size() for t in self.host_out)
        self.fwd_ms = self.bwd_ms = None

    def step(self, i):
        self.rt.attention_forward(self.q, self.k, self.v, causal=True, out=self.o, lse=self.lse)
        self.grads = self.rt.attention_backward(self.q, self.k, self.v, self.o, self.do, self.lse, causal=True, delta=self.delta,
                                                deterministic=self.deterministic)

    def e2e_step(self, i):
        for d, h in zip((self.q, self.k, self.v, self.do), self.host_in):
            d.copy_(h, non_blocking=True)
        self.step(i)
        for h, d in zip(self.host_out, (self.o, *self.grads)):
            h.copy_(d, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()

    def split_times(self, steps=5):
        """Forward and backward timed separately with CUDA events (after the main timed region)."""
        torch = self.torch
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        for _ in range(steps):
            self.rt.attention_forward(self.q, self.k, self.v, causal=True, out=self.o, lse=self.lse)
        ev[1].record()
        for _ in range(steps):
            self.rt.attention_backward(self.q, self.k, self.v, self.o, self.do, self.lse, causal=True, delta=self.delta,
                                       deterministic=self.deterministic)
        ev[2].record()
        torch.cuda.synchronize()
        self.fwd_ms, self.bwd_ms = ev[0].elapsed_time(ev[1]) / steps, ev[1].elapsed_time(ev[2]) / steps

    def roofline(self, peaks, kernel_ms):
        self.split_times()
        fwd = self.fwd_flops() / 1e12 / (self.fwd_ms / 1e3)
        bwd = 2.5 * self.fwd_flops() / 1e12 / (self.bwd_ms / 1e3)
        return {"bound": "tensor", "achieved": fwd, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": fwd / peaks["bf16_tflops"],
                "traffic": 1.063e9 if (self.b, self.h, self.s, self.d) == (8, 32, 4096, 128) else None,
                "traffic_source": "ncu capture of the forward launch at batch 8, 32 heads, 4096, 128 (recorded constant, summary under profiles/)",
                "kernel": f"attention_fwd_kernel<{self.d}>", "flops_per_launch": self.fwd_flops(),
                "forward_ms": self.fwd_ms, "backward_ms": self.bwd_ms, "backward_achieved": bwd,
                "backward_frac": bwd / peaks["bf16_tflops"]}  # fmt: skip

    def cpu_sample(self, s=512):
        """The oracle on the traced forward program for one (batch, head) slice of a shorter sequence."""
        from lumen_b200 import functional as F
        from lumen_b200 import tracer
        from oracle import oracle

        shape = (1, s, 1, self.d)
        g = tracer.trace(lambda q, k, v: F.attention_forward_prims(q, k, v, self.d**-0.5, True), *[("bfloat16", shape)] * 3)
        rng = np.random.default_rng(3)
        q, k, v = (rng.standard_normal(shape).astype(np.float32).astype(oracle.BF16) for _ in range(3))
        t0 = time.perf_counter()
        oracle.run(g, [q, k, v])
        dt = time.perf_counter() - t0
        return 4 * s * s * self.d / 2 / 1e12 / dt, oracle.threads(), f"forward only, one (batch, head) slice at sequence {s}, oracle interpreter of the traced program"


class TrainStepWorkload:
    """The 12-layer decoder transformer data-parallel training step (forward + loss.backward + SGD update), bf16
    weights/activations with fp32 matmul accumulation: d_model 1024, 16 heads x 64, MLP hidden 4096 ReLU,
    pre-LayerNorm, vocab 32768, seq 2048, GLOBAL batch 64 sequences sharded over the ranks (strong scaling), token ids
    uniform from seed 4, weights N(0, 0.02). Metric: tokens/s of the whole job."""

    def __init__(self, small=False):
        from lumen_b200 import transformer as T

        self.T = T
        self.small = small
        self.cfg = T.Config.baseline_small() if small else T.Config.baseline_large()
        self.global_batch = 8 if small else 64
        self.name = "train_step_2layer_f32" if small else "train_step_12layer_bf16_dp"
        self.metric = "transformer train-step throughput"
        self.unit = "tokens/s"
        self.arith = "f32" if small else "bf16"
        self.rows, self.cols = self.global_batch * self.cfg.seq, self.cfg.d_model
        self.scaling = "strong"
        self.tokens_per_rank = self.global_batch * self.cfg.seq
        # The reference backend's default mode: attention backward as one kernel that adds dQ atomically, scatter-add by
        # atomics (its `deterministic` option, off by default, selects the bit-reproducible forms:
        # lumen/codegen/attention/triton/mod.rs:458-466, lumen/codegen/scatter_add/README.md:23-39).
        # LUMEN_B200_DETERMINISTIC=1 runs those instead.
        self.deterministic = os.environ.get("LUMEN_B200_DETERMINISTIC", "0") != "0"

    def units_per_step(self):  # tokens per step per rank: set in setup (depends on the world size)
        return self.tokens_per_rank

    def setup(self, device, host=True):
        """Everything here is the backend's own: memory from its region allocator, its stream, its store and NCCL
        communicator. No other CUDA framework takes part in the step."""
        from lumen_b200 import device as D
        from lumen_b200 import distributed

        self.D = D
        group = distributed.default_group() if distributed.is_initialized() else None
        world = group.world if group else 1
        rank = group.rank if group else 0
        if self.global_batch % world:
            raise SystemExit(f"the global batch {self.global_batch} does not shard over {world} ranks")
        self.batch = self.global_batch // max(world, getattr(self, "shard_of", 0) or 1)
        self.tokens_per_rank = self.batch * self.cfg.seq
        params = self.T.init_params(self.cfg, seed=4)
        self.step_fn = self.T.TrainStep(self.cfg, self.batch, params, device, world=world, process_group=group,
                                        graphs=os.environ.get("LUMEN_B200_GRAPHS") or None,
                                        deterministic=self.deterministic,
                                        lowering=os.environ.get("LUMEN_B200_LOWERING", "native"),
                                        autotune=os.environ.get("LUMEN_B200_AUTOTUNE", "0") != "0")
        rng = np.random.default_rng(4)
        tokens = rng.integers(0, self.cfg.vocab, (self.global_batch, self.cfg.seq + 1))
        mine = tokens[rank * self.batch : (rank + 1) * self.batch]
        self.host_ids = np.ascontiguousarray(mine[:, :-1]).astype(np.int64)
        self.host_targets = np.ascontiguousarray(mine[:, 1:]).astype(np.int64)
        self.step_fn.load_batch(self.host_ids, self.host_targets)
        self.host_loss = D.HostBuffer(4)  # pinned: the loss is read back asynchronously
        self.h2d = 2 * self.host_ids.size * 8
        self.d2h = 4
        self.launches_per_step = self.step_fn.compiled.kernel_launches  # kernels, not plan steps
        self.workspace_gb = self.step_fn.compiled.workspace_bytes / 2**30
        self.world = world

    def step(self, i):
        self.step_fn.step()

    def e2e_step(self, i):
        self.step_fn.load_batch(self.host_ids, self.host_targets)  # through pinned staging, asynchronous
        loss = self.step_fn.step()
        loss.copy_to_host(self.host_loss, self.step_fn.stream)
        self.step_fn.stream.synchronize()

    def roofline(self, peaks, kernel_ms):
        """The step against the tensor-core roofline (its FLOPs over the sustained bf16 peak: the step runs for
        hundreds of milliseconds under the power cap), and the dominant kernel (the tcgen05 GEMM) timed alone on the
        step's largest shape."""
        import torch  # harness only: operands of the stand-alone GEMM timing below

        from lumen_b200.runtime import gemm

        step_ms = kernel_ms * self.launches_per_step
        flops = self.T.flops_per_step(self.cfg, self.batch)
        achieved = flops / 1e12 / (step_ms / 1e3)
        out = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
               "frac": achieved / peaks["bf16_tflops_sustained"], "frac_of_burst": achieved / peaks["bf16_tflops"],
               "traffic": None, "kernel": "whole step (gemm_tcgen05_pair dominates)", "flops_per_step_per_gpu": flops,
               "loss": float(self.step_fn.loss.item()), "gradient_buckets": len(self.step_fn.buckets), "deterministic": self.deterministic,
               "graphs": self.step_fn.graph_mode, "plan_steps": self.step_fn.plan.num_steps,
               "autotuned_gemm_steps": len(self.step_fn.tuning),
               "autotune_gain_us_per_step": float(sum(t["default_us"] - t["us"] for t in self.step_fn.tuning))}  # fmt: skip
        if self.step_fn.tuning:  # LUMEN_B200_AUTOTUNE=1: the tuner's isolated timings per GEMM shape of the step
            shapes = {}
            for t in self.step_fn.tuning:
                e = shapes.setdefault(f"{t['label']} [{t['m']}, {t['n']}, {t['k']}]", {"steps": 0, "default_us": 0.0, "tuned_us": 0.0, "flop": 2.0 * t["m"] * t["n"] * t["k"]})
                e["steps"] += 1
                e["default_us"] += t["default_us"]
                e["tuned_us"] += t["us"]
            out["gemm_shapes"] = {k: {"steps": e["steps"], "default_us": round(e["default_us"] / e["steps"], 1),
                                      "default_tflops": round(e["flop"] * e["steps"] / e["default_us"] / 1e6),
                                      "tuned_us": round(e["tuned_us"] / e["steps"], 1)} for k, e in shapes.items()}
        if not self.small:
            t, d, h = self.tokens_per_rank, self.cfg.d_model, self.cfg.hidden
            a = torch.randn((t, d), device="cuda").bfloat16()
            w = torch.randn((h, d), device="cuda").bfloat16()
            y = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
            for _ in range(3):
                gemm(a, w.t(), y)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            for _ in range(10):
                gemm(a, w.t(), y)
            ev[1].record()
            torch.cuda.synchronize()
            ms = ev[0].elapsed_time(ev[1]) / 10
            # traffic: ncu dram bytes of one launch at 131072 tokens (279 MB read + 1024 MB written; the algorithmic
            # figure is A + B + D = 1350 MB), scaled by the tokens of this rank
            out["dominant_kernel"] = {"name": "gemm_tcgen05_pair", "shape": [t, h, d], "ms": ms,
                                      "achieved": 2 * t * d * h / 1e12 / (ms / 1e3), "unit": "TFLOP/s",
                                      "traffic": 1.3025e9 * t / 131072, "algorithmic_bytes": 2.0 * (t * d + h * d + t * h)}  # fmt: skip
            out["traffic"] = out["dominant_kernel"]["traffic"]
            out["traffic_source"] = ("ncu capture of one gemm_tcgen05_pair launch at 131072 tokens (recorded constant, summary under "
                                     "profiles/), scaled by this rank's tokens")
        return out

    SAMPLE_TOKENS = 128

    def cpu_sample(self):
        """Times the oracle on a bounded sample of THIS workload and extrapolates to the whole step.

        12-layer configuration: forward + backward of the same architecture and shapes (d_model 1024, 16 heads x 64,
        hidden 4096, vocabulary 32768, bfloat16 with float32 accumulation) with ONE of the 12 layers plus the whole
        head, on 128 tokens of one sequence. The whole step's time is taken as the sample's time per token, times the
        ratio of the full model's FLOPs per token (12 layers, sequence 2048) to the sample's, times the step's tokens;
        the optimizer update (under 1 % of a CPU step at 131072 tokens) is left out. Returns the EXTRAPOLATED
        tokens/s, the threads used and a description carrying the measured seconds."""
        from lumen_b200 import transformer as T
        from oracle import oracle

        if self.small:
            cfg, batch, update = T.Config.baseline_small(), 8, True
        else:
            cfg, batch, update = T.Config.baseline_large(), 1, False
            cfg.layers, cfg.seq = 1, self.SAMPLE_TOKENS
        if getattr(self, "_cpu_graph", None) is None:
            g, names, _ = T.trace_train_step(cfg, batch, update=update)
            params = T.init_params(cfg, 4)
            t = np.random.default_rng(4).integers(0, cfg.vocab, (batch, cfg.seq + 1))
            cast = (lambda a: a.astype(oracle.BF16)) if cfg.dtype == "bfloat16" else (lambda a: a)
            self._cpu_graph = (g, [np.ascontiguousarray(t[:, :-1]), np.ascontiguousarray(t[:, 1:])] + [cast(params[n]) for n in names])
        g, inputs = self._cpu_graph
        t0 = time.perf_counter()
        oracle.run(g, inputs)
        dt = time.perf_counter() - t0
        self.cpu_sample_seconds = dt
        tokens = batch * cfg.seq
        if self.small:
            return tokens / dt, oracle.threads(), f"one full step of the 2-layer float32 configuration ({tokens} tokens) in {dt:.2f} s, oracle interpreter"
        ratio = (T.flops_per_step(self.cfg, 1) / self.cfg.seq) / (T.flops_per_step(cfg, 1) / cfg.seq)
        return tokens / (dt * ratio), oracle.threads(), (
            f"EXTRAPOLATED from a bounded sample: forward + backward of 1 of the 12 layers plus the head at the step's own "
            f"shapes on {tokens} tokens took {dt:.2f} s on the oracle interpreter; scaled by the FLOPs per token of the full "
            f"model over the sample's ({ratio:.2f}x); optimizer update not included")


WORKLOADS = {
    "train_step_12layer_bf16_dp": TrainStepWorkload,
    "train_step_2layer_f32": lambda: TrainStepWorkload(small=True),
    "flash_attention_fwd_bwd": FlashAttention,
    "flash_attention_d64_fwd_bwd": lambda: FlashAttention(b=64, h=16, s=2048, d=64),  # the training step's attention shape
    "matmul_bf16_8192_fwd_bwd": MatmulBackward,
    "fused_chain_f32": lambda: FusedChain("float32"),
    "fused_chain_bf16": lambda: FusedChain("bfloat16"),
}
DEFAULT_WORKLOAD = "train_step_12layer_bf16_dp"


# ---- clocks ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons every 200 ms while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index):
        self.index, self.samples, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5,
                ).stdout.strip()  # fmt: skip
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        self.thread.join(timeout=6)

    def summary(self):
        mhz = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {
            "sm_mhz": float(np.median(mhz)) if mhz else None,
            "sm_max_mhz": float(self.samples[0][1]) if self.samples and self.samples[0][1].replace(".", "").isdigit() else None,
            "reasons": reasons,
            "samples": len(self.samples),
        }


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---- the other headline quantities, measured in the same run ----------------------------------------------------
def secondary_measurements(device, peaks, steps=6, warmup=3):
    """Fused-chain GB/s, 8192^3 matmul TFLOP/s and flash-attention TFLOP/s (the benchmark shape at head dim 128 and the
    training step's own attention shape at head dim 64), each timed on the device with CUDA events after warm-up, with
    inputs resident in HBM and larger than L2. Returns `{name: {value, unit, ms, frac, peak, ...}}`."""
    import torch

    out = {}

    def timed(fn, n):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for i in range(n):
            fn(i)
        ev[1].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) / n

    for make in (lambda: FusedChain("float32"), lambda: FusedChain("bfloat16")):
        w = make()
        w.setup(device, host=False)
        ms = timed(w.step, 3 * steps)
        gbs = w.units_per_step() / (ms / 1e3)
        out[w.name] = {"value": gbs, "unit": "GB/s", "ms": ms, "frac": gbs / peaks["hbm_gbs"], "peak": peaks["hbm_gbs"],
                       "bytes_per_launch": w.units_per_step() * 1e9, "kernel": "fused_kernel"}
        del w
        torch.cuda.empty_cache()
    w = MatmulBackward()
    w.setup(device, host=False)
    ms = timed(w.step, steps)
    tf = w.units_per_step() / (ms / 1e3)
    out[w.name] = {"value": tf, "unit": "TFLOP/s", "ms": ms, "frac": tf / peaks["bf16_tflops"], "peak": peaks["bf16_tflops"],
                   "launches_per_step": 3, "kernel": "gemm_tcgen05_pair"}
    del w
    torch.cuda.empty_cache()
    for shape in ((8, 32, 4096, 128), (64, 16, 2048, 64)):
        w = FlashAttention(*shape)
        w.setup(device, host=False)
        timed(w.step, 1)
        w.split_times(steps)
        fwd = w.fwd_flops() / 1e12 / (w.fwd_ms / 1e3)
        bwd = 2.5 * w.fwd_flops() / 1e12 / (w.bwd_ms / 1e3)
        total = 3.5 * w.fwd_flops() / 1e12 / ((w.fwd_ms + w.bwd_ms) / 1e3)
        out[w.name] = {"value": total, "unit": "TFLOP/s", "ms": w.fwd_ms + w.bwd_ms, "frac": total / peaks["bf16_tflops"],
                       "peak": peaks["bf16_tflops"], "forward": {"value": fwd, "ms": w.fwd_ms, "frac": fwd / peaks["bf16_tflops"]},
                       "backward": {"value": bwd, "ms": w.bwd_ms, "frac": bwd / peaks["bf16_tflops"]},
                       "kernels": "attention_fwd_kernel, attention_delta, attention_bwd_kernel x2"}
        del w
        torch.cuda.empty_cache()
    return out


# ---- reference arm ----------------------------------------------------------------------------------------------
def host_threads() -> int:
    """Cores this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def use_all_host_cores() -> None:
    """The CPU legs run the oracle on every core this process may use, also under torchrun (which exports
    OMP_NUM_THREADS=1 to its workers); the line reports the thread count actually set."""
    from oracle import oracle

    oracle.set_threads(host_threads())


def run_reference(args, workload):
    """The CPU arm: every step is one bounded sample of the workload on the oracle (all host cores), timed by wall
    clock; `ms_per_step` is the measured time of one sample, `value` the workload's metric that sample gives
    (extrapolated where the sample is smaller than the workload; `cpu_baseline.sample` says how)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_cores()
    for _ in range(args.warmup):
        workload.cpu_sample()
    values = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, cores, sample = workload.cpu_sample()
        values.append(v)
    ms = (time.perf_counter() - t0) * 1e3 / max(args.steps, 1)
    v = float(np.mean(values))
    line = {
        "impl": "reference", "metric": workload.metric, "value": v, "unit": workload.unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": getattr(workload, "scaling", "weak"), "vs_baseline": None, "dtype": workload.arith, "data": "synthetic",
        "config": {"workload": workload.name, "step": "one bounded CPU sample of the workload per step; ms_per_step is its measured wall time"},
        "cpu_baseline": {"value": v, "unit": workload.unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---- main -------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="lumen_b200", choices=["lumen_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the fused / matmul / attention measurements of the default line")
    ap.add_argument("--profile-steps", action="store_true",
                    help="diagnostic, one GPU: after the timed region, time every plan step of the training step launched alone "
                         "and add the per-label totals to the line (`step_profile`)")
    ap.add_argument("--shard-of", type=int, default=0, metavar="N",
                    help="diagnostic, one GPU: run ONE rank's share of an N-rank training step alone, without its collectives "
                         "(the compute-only time the N-rank step is compared with)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    workload = WORKLOADS[args.workload]()
    if args.shard_of:
        if not isinstance(workload, TrainStepWorkload) or int(os.environ.get("WORLD_SIZE", "1")) > 1:
            raise SystemExit("--shard-of applies to the training step on one GPU")
        workload.shard_of = args.shard_of

    if args.impl == "reference":
        run_reference(args, workload)
        return

    from lumen_b200 import device as D
    from lumen_b200 import distributed

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if D.device_count() <= 0:
        raise SystemExit("bench.py needs a B200 GPU: lumen_b200 has no CPU fallback")
    D.set_device(local_rank)
    group = distributed.init_process_group(timeout=300.0) if world > 1 else None  # the backend's own store + NCCL communicator
    torch_workload = not isinstance(workload, TrainStepWorkload)
    if torch_workload:  # the kernel micro-benchmarks hold their operands in torch tensors (harness only)
        import torch

        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
    else:
        device = local_rank

    workload.setup(device)
    # the stream the workload launches on: the training step's own stream, torch's current (default) stream otherwise
    launch_stream = workload.step_fn.stream if isinstance(workload, TrainStepWorkload) else None

    def barrier():
        """Every rank has finished its queued work (waited for with a deadline while NCCL's error state is polled),
        then every rank has arrived (host barrier through the store, with a deadline)."""
        if world > 1:
            group.synchronize(launch_stream, 120.0)
            group.barrier(120.0)
        D.synchronize()

    for i in range(args.warmup):
        workload.step(i)
    barrier()

    # timed region: K steps, CUDA events on the launching stream
    start, stop = D.Event(timing=True), D.Event(timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        start.record(launch_stream)
        for i in range(args.steps):
            workload.step(i)
        stop.record(launch_stream)
        barrier()
    ms = start.elapsed_ms(stop)

    # end to end through the same call with host buffers
    for i in range(2):
        workload.e2e_step(i)
    barrier()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_start, e2e_stop = D.Event(timing=True), D.Event(timing=True)
    e2e_start.record(launch_stream)
    for i in range(e2e_steps):
        workload.e2e_step(i)
    e2e_stop.record(launch_stream)
    barrier()
    e2e_ms = e2e_start.elapsed_ms(e2e_stop)

    if world > 1:  # the slowest rank's times
        region = D.Region(1 << 16)
        times = region.empty((2,), "float64")
        side = D.Stream()
        times.copy_from_host(np.array([ms, e2e_ms], np.float64), side)
        group.all_reduce(times, "max", side)
        group.synchronize(side, 120.0)
        ms, e2e_ms = times.copy_to_host(stream=side).tolist()

    if rank == 0:
        peaks, peak_kind = measured_peak()
        units = workload.units_per_step()  # GB per step per rank
        value = units * world * args.steps / (ms / 1e3)
        scaling = getattr(workload, "scaling", "weak")
        kernel_ms = ms / args.steps / workload.launches_per_step
        achieved = units / (kernel_ms / 1e3)
        line = {
            "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": workload.arith, "data": "synthetic",
            "config": {"workload": workload.name, "rows": workload.rows, "cols": workload.cols,
                       "l2": "each step moves more than the 126 MB L2 and steps rotate over 3 buffer sets",
                       "parallelism": (f"dp{world}" if scaling == "strong" else "replicas only") if world > 1 else "single GPU"},
            "roofline": workload.roofline(peaks, kernel_ms) if hasattr(workload, "roofline") else
                        {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": getattr(workload, "traffic", None),
                         "traffic_source": getattr(workload, "traffic_source", None),
                         "kernel": "fused_kernel", "bytes_per_launch": units * 1e9},
            "e2e": {"value": units * world * e2e_steps / (e2e_ms / 1e3), "unit": workload.unit,
                    "h2d_bytes_per_step": workload.h2d, "d2h_bytes_per_step": workload.d2h},
            "gpu_launches": args.steps * workload.launches_per_step,
            "clocks": clocks.summary(),
        }  # fmt: skip
        line["roofline"]["peak_kind"] = peak_kind
        if args.profile_steps and isinstance(workload, TrainStepWorkload) and world == 1:
            totals = {}
            for label, ms_one in workload.step_fn.plan.profile(workload.step_fn.bound, workload.step_fn.stream):
                entry = totals.setdefault(label, {"steps": 0, "ms": 0.0})
                entry["steps"] += 1
                entry["ms"] += ms_one
            line["step_profile"] = {k: {"steps": v["steps"], "ms": round(v["ms"], 3)} for k, v in sorted(totals.items(), key=lambda kv: -kv[1]["ms"])}
        if args.shard_of:
            line["config"]["parallelism"] = f"one rank's share of dp{args.shard_of}, run alone without collectives (diagnostic)"
        if args.workload == DEFAULT_WORKLOAD and world == 1 and not args.no_secondary and not args.shard_of:
            # the metric's other quantities (fused GB/s, matmul and flash-attention TFLOP/s) after the step's memory is released
            workload.step_fn = None
            import gc

            gc.collect()
            import torch  # harness only: the micro-benchmarks' operands

            torch.cuda.set_device(local_rank)
            line["secondary"] = secondary_measurements(torch.device("cuda", local_rank), peaks)
        if not args.no_cpu_baseline and world == 1 and not args.shard_of:  # rank 0 at N = 1 only
            use_all_host_cores()
            v, cores, sample = workload.cpu_sample()
            line["cpu_baseline"] = {"value": v, "unit": workload.unit, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        distributed.destroy_process_group()


if __name__ == "__main__":
    main()
