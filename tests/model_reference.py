"""An independent float64 PyTorch (CPU autograd) statement of the transformer training step, used to check the
hand-derived backward of lumen_b200.nn: same architecture as lumen_b200.transformer, nothing shared with it."""

import math

import torch


def torch_step(cfg, params, ids, targets):
    """Returns (loss, grads by name) in float64."""
    p = {k: torch.tensor(v, dtype=torch.float64, requires_grad=True) for k, v in params.items()}
    ids_t, tg = torch.tensor(ids), torch.tensor(targets)
    b, s = ids.shape
    d, h = cfg.d_model, cfg.heads
    x = (p["embed.tokens"][ids_t] + p["embed.positions"]).reshape(b * s, d)

    def ln(a, w, bias):
        xc = a - a.mean(-1, keepdim=True)
        return xc / torch.sqrt((xc * xc).mean(-1, keepdim=True) + 1e-5) * w + bias

    mask = torch.tril(torch.ones(s, s, dtype=torch.bool))
    for layer in range(cfg.layers):
        q = f"layers.{layer}."
        hh = ln(x, p[q + "attn.norm.w"], p[q + "attn.norm.b"])
        qkv = hh @ p[q + "attn.wqkv"].T
        qq, kk, vv = (qkv[:, i * d : (i + 1) * d].reshape(b, s, h, d // h).permute(0, 2, 1, 3) for i in range(3))
        sc = qq @ kk.transpose(-1, -2) / math.sqrt(d // h)
        sc = sc.masked_fill(~mask, float("-inf"))
        a = (torch.softmax(sc, -1) @ vv).permute(0, 2, 1, 3).reshape(b * s, d)
        x = x + a @ p[q + "attn.wo"].T
        hh = ln(x, p[q + "mlp.norm.w"], p[q + "mlp.norm.b"])
        x = x + torch.relu(hh @ p[q + "mlp.w1"].T) @ p[q + "mlp.w2"].T
    x = ln(x, p["norm.w"], p["norm.b"])
    logits = x @ p["head"].T
    loss = torch.nn.functional.cross_entropy(logits, tg.reshape(-1))
    loss.backward()
    return loss.item(), {k: v.grad.numpy() for k, v in p.items()}
