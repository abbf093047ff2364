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


def attention_f64(q, k, v, causal, d_o=None):
    """Float64 attention one (batch, head) at a time, so that a 4096 x 4096 score matrix is the most held at once:
    returns `(o [B, Sq, N, H], lse [B, N, Sq])`, and with `d_o` also `(dq, dk, dv)` by the closed-form backward
    (dV = P^T dO; dS = P * (dO V^T - rowsum(dO * O)) * scale; dQ = dS K; dK = dS^T Q), grouped heads summed."""
    b, sq, n, h = q.shape
    sk, nkv = k.shape[1], k.shape[2]
    scale = 1.0 / np.sqrt(h)
    o = np.zeros((b, sq, n, v.shape[3]))
    lse = np.zeros((b, n, sq))
    grads = [np.zeros(a.shape) for a in (q, k, v)] if d_o is not None else None
    visible = None
    if causal:
        visible = np.arange(sk)[None, :] <= np.arange(sq)[:, None] + (sk - sq)
    for bi in range(b):
        for hi in range(n):
            kv = hi // (n // nkv)
            qh, kh, vh = (a.astype(np.float64) for a in (q[bi, :, hi], k[bi, :, kv], v[bi, :, kv]))
            s = (qh @ kh.T) * scale
            if visible is not None:
                s = np.where(visible, s, -np.inf)
            m = s.max(-1, keepdims=True)
            e = np.exp(s - m)
            total = e.sum(-1, keepdims=True)
            p = e / total
            o[bi, :, hi] = p @ vh
            lse[bi, hi] = (m + np.log(total))[:, 0]
            if d_o is not None:
                g = d_o[bi, :, hi].astype(np.float64)
                delta = (g * o[bi, :, hi]).sum(-1, keepdims=True)
                ds = p * (g @ vh.T - delta) * scale
                grads[0][bi, :, hi] = ds @ kh
                grads[1][bi, :, kv] += ds.T @ qh
                grads[2][bi, :, kv] += p.T @ g
    return (o, lse) if d_o is None else (o, lse, grads)
