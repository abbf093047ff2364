"""Shared test helpers: seeded inputs, oracle evaluation, numpy <-> torch for bfloat16."""

import numpy as np
import torch

from oracle import oracle

BF16 = oracle.BF16


def to_torch(a: np.ndarray, device) -> torch.Tensor:
    if a.dtype == BF16:
        return torch.from_numpy(a.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    if a.dtype in (np.uint16, np.uint32, np.uint64):
        return torch.from_numpy(a.view(a.dtype.str.replace("u", "i")).copy()).view(getattr(torch, a.dtype.name)).to(device)
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().view(BF16)
    return t.numpy()


def bf16(a) -> np.ndarray:
    """float array rounded to bfloat16 (round to nearest even)."""
    return np.asarray(a, np.float32).astype(BF16)


def run_oracle(graph, inputs):
    return oracle.run(graph, inputs)


def max_rel_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    scale = np.maximum(np.abs(want).max(), 1e-30)
    return float(np.abs(got - want).max() / scale)
