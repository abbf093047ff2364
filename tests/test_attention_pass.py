"""The attention passes on CPU: programs that spell attention in bare prims are rewritten into `flash_attention` /
`flash_attention_backward` fusions whose bodies are the matched nodes, so the oracle's results do not change by a bit
(lumen/reference/README.md:15), and they lower to `attn_fwd` / `attn_bwd` plan steps
(lumen/graph_compiler/passes/attention/forward.rs:56-97, backward.rs:54-83)."""

import math

import numpy as np
import pytest

from lumen_b200 import functional as F
from lumen_b200 import tracer
from lumen_b200.attention_pass import match_attention
from lumen_b200.compiler import compile_graph
from oracle import oracle
from tests.helpers import bf16

B, S, N, H = 2, 128, 4, 64
FULL = ("bfloat16", (B, S, N, H))
GROUPED = ("bfloat16", (B, S, 2, H))


def softmax_and_two_matmuls(q, k, v):
    """Attention written by hand: `[B, S, N, H]` operands permuted to heads-first, F.softmax, two F.matmuls."""
    qt, kt, vt = q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1), v.permute(0, 2, 1, 3)
    s = F.matmul(qt, kt, "float32", "float32") * (1 / math.sqrt(H))
    p = F.softmax(s, -1).to("bfloat16")
    return F.matmul(p, vt, "float32", "bfloat16").permute(0, 2, 1, 3)


def heads_first_output(q, k, v):
    """The same, leaving the output heads-first `[B, N, S, H]` (the kernel writes it through a strided view)."""
    qt, kt, vt = q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1), v.permute(0, 2, 1, 3)
    p = F.softmax(F.matmul(qt, kt, "float32", "float32") * 0.125, -1).to("bfloat16")
    return F.matmul(p, vt, "float32", "bfloat16")


def forward_and_backward(q, k, v, do):
    o, lse = F.attention_forward_prims(q, k, v, 0.125, True)
    return (o, *F.attention_backward_prims(q, k, v, o, lse, do, 0.125, True))


def inputs_for(specs, seed=0):
    rng = np.random.default_rng(seed)
    return [bf16(rng.standard_normal(shape)) for _, shape in specs]


CASES = [
    (softmax_and_two_matmuls, [FULL] * 3, ["flash_attention"], {"causal": False, "heads_per_kv": 1, "o": "BSNH", "lse": False}),
    (heads_first_output, [FULL] * 3, ["flash_attention"], {"o": "BNSH"}),
    (lambda q, k, v: F.attention_forward_prims(q, k, v, 0.125, True), [FULL, GROUPED, GROUPED], ["flash_attention"],
     {"causal": True, "offset": 0, "heads_per_kv": 2, "lse": True}),
    (forward_and_backward, [FULL, GROUPED, GROUPED, FULL], ["flash_attention", "flash_attention_backward"], {"heads_per_kv": 2}),
    (forward_and_backward, [FULL] * 4, ["flash_attention", "flash_attention_backward"], {"heads_per_kv": 1}),
]


@pytest.mark.parametrize("fn,specs,names,expect", CASES)
def test_rewrite_finds_the_attention_and_changes_no_value(fn, specs, names, expect):
    g = tracer.trace(fn, *specs)
    args = inputs_for(specs)
    want = oracle.run(g, args)
    before = len(g.nodes)
    rewritten = match_attention(g)
    assert len(g.nodes) == before  # the traced graph itself is untouched
    fusions = [n for n in rewritten.nodes if n.op == "fusion"]
    assert [f.params["name"] for f in fusions] == names
    for key, value in expect.items():
        assert fusions[-1 if key == "heads_per_kv" else 0].params["attention"][key] == value
    assert fusions[0].params["attention"]["scale"] == pytest.approx(0.125)
    assert not any(n.op in ("exp", "dot_general", "reduce_max") for n in rewritten.nodes)  # nothing of it left outside
    got = oracle.run(rewritten, args)
    for a, b in zip(want, got):
        assert a.tobytes() == b.tobytes()


def test_the_rewritten_program_lowers_to_attention_steps():
    g = tracer.trace(forward_and_backward, FULL, GROUPED, GROUPED, FULL)
    plan = compile_graph(g)
    kinds = [line.split()[1] for line in plan.text.splitlines() if line.startswith("s ")]
    assert kinds == ["attn_fwd", "attn_bwd"]
    plan = compile_graph(tracer.trace(heads_first_output, FULL, FULL, FULL))
    assert [line.split()[1] for line in plan.text.splitlines() if line.startswith("s ")] == ["attn_fwd"]


def test_lookalikes_are_left_alone():
    """A softmax whose probabilities are also returned, scores scaled by a tensor, and a plain matmul chain: no match,
    the program runs as traced."""
    def returns_probabilities(q, k, v):
        qt, kt, vt = q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1), v.permute(0, 2, 1, 3)
        p = F.softmax(F.matmul(qt, kt, "float32", "float32") * 0.125, -1).to("bfloat16")
        return F.matmul(p, vt, "float32", "bfloat16"), p

    def scaled_by_a_tensor(q, k, v, t):
        qt, kt, vt = q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1), v.permute(0, 2, 1, 3)
        p = F.softmax(F.matmul(qt, kt, "float32", "float32") * t, -1).to("bfloat16")
        return F.matmul(p, vt, "float32", "bfloat16")

    for fn, specs in ((returns_probabilities, [FULL] * 3), (scaled_by_a_tensor, [FULL] * 3 + [("float32", (B, N, S, S))])):
        rewritten = match_attention(tracer.trace(fn, *specs))
        assert not [n for n in rewritten.nodes if n.op == "fusion"]
