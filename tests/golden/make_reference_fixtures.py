"""Generates tests/golden/reference_*.npz by RUNNING the reference's own NumPy model of this path.

The reference's test modules cannot be imported without its Rust extension (their top-level `import lumen` fails),
but the NumPy model they hold needs nothing of it. This script reads two of those test files as text, picks the
model's functions and constants out of the syntax tree, compiles exactly those definitions (nothing is retyped
here), and evaluates them on seeded inputs:

  tests/test_transformer_example.py : VOCAB .. LAYERS, BATCH; _bf16, _rms_norm, _matmul, _attention, _logits
  tests/functional/test_attention.py: reference() (float64 attention), CASES (its shapes)

The outputs pin the CPU oracle (tests/test_reference_fixtures.py). Run where the reference checkout is present:

    python tests/golden/make_reference_fixtures.py [--reference /path/to/lumen]

The fixtures are committed; the tests never read the reference checkout.
"""

from __future__ import annotations

import argparse
import ast
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def lift(path: str, functions: list[str], constants: list[str]) -> dict:
    """The named top-level functions and constant assignments of the file at `path`, compiled on their own."""
    with open(path) as f:
        tree = ast.parse(f.read(), path)
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in functions:
            keep.append(node)
        elif isinstance(node, ast.Assign):
            names = set()
            for target in node.targets:
                for leaf in ast.walk(target):
                    if isinstance(leaf, ast.Name):
                        names.add(leaf.id)
            if names and names <= set(constants):
                keep.append(node)
    found = {n.name for n in keep if isinstance(n, ast.FunctionDef)}
    missing = set(functions) - found
    if missing:
        raise SystemExit(f"{path}: functions {sorted(missing)} not found; the reference's layout changed")
    module = ast.Module(body=keep, type_ignores=[])
    namespace = {"np": np}
    exec(compile(module, path, "exec"), namespace)
    for c in constants:
        if c not in namespace:
            raise SystemExit(f"{path}: constant {c} not found")
    return namespace


def model_weights(ns: dict, seed: int) -> dict[str, np.ndarray]:
    """Weights for the names `_logits` reads, drawn as the reference's `_weights` draws them (norm scales near one,
    matrices N(0, 1) / sqrt(fan_in)); `_weights` itself walks a lumen module and cannot run here."""
    vocab, seq, dim, hidden, layers = (ns[k] for k in ("VOCAB", "SEQ", "DIM", "HIDDEN", "LAYERS"))
    shapes = [("embed.tokens", (vocab, dim)), ("embed.positions", (seq, dim))]
    for layer in range(layers):
        p = f"layers.{layer}."
        shapes += [(p + "attn.norm", (dim,))] + [(p + f"attn.w{n}", (dim, dim)) for n in "qkvo"]
        shapes += [(p + "mlp.norm", (dim,)), (p + "mlp.w1", (hidden, dim)), (p + "mlp.w2", (dim, hidden))]
    shapes += [("norm", (dim,)), ("head", (vocab, dim))]
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in shapes:
        if len(shape) == 1:
            out[name] = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)
        else:
            out[name] = (rng.standard_normal(shape) / np.sqrt(shape[1])).astype(np.float32)
    return out


def attention_case_inputs(i: int, shape):
    """Seeded float32 q [b, sq, n, h], k [b, sk, nkv, h], v [b, sk, nkv, hv] of attention case `i`."""
    b, sq, sk, n, nkv, h, hv = (int(x) for x in shape)
    rng = np.random.default_rng(1000 + i)
    return (rng.standard_normal((b, sq, n, h)).astype(np.float32), rng.standard_normal((b, sk, nkv, h)).astype(np.float32),
            rng.standard_normal((b, sk, nkv, hv)).astype(np.float32))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its tests/ directory is read)")
    args = ap.parse_args()

    model = lift(os.path.join(args.reference, "tests", "test_transformer_example.py"),
                 ["_bf16", "_rms_norm", "_matmul", "_attention", "_logits"],
                 ["VOCAB", "SEQ", "DIM", "HEADS", "HIDDEN", "LAYERS", "BATCH", "PASSES", "LR"])
    attn = lift(os.path.join(args.reference, "tests", "functional", "test_attention.py"), ["reference"], ["CASES", "TOL"])

    # 1. _bf16: random magnitudes over the whole exponent range plus ties, signed zeros, the largest finite value
    rng = np.random.default_rng(100)
    x = (rng.standard_normal(8192) * 10.0 ** rng.integers(-30, 30, 8192)).astype(np.float32)
    edge = np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 1.0078125, 1.00390624, 3.3895314e38, 1e-40, -1e-40,
                     65504.0, 2.0**-126, 2.0**-133], np.float32)
    x = np.concatenate([x, edge])
    np.savez_compressed(os.path.join(HERE, "reference_bf16.npz"), x=x, y=model["_bf16"](x))

    # 2. _rms_norm, 3. _matmul
    rng = np.random.default_rng(101)
    xn = rng.standard_normal((48, model["DIM"])).astype(np.float32)
    wn = (1.0 + 0.1 * rng.standard_normal(model["DIM"])).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_rms_norm.npz"), x=xn, w=wn, y=model["_rms_norm"](xn, wn))
    xm = rng.standard_normal((48, 96)).astype(np.float32)
    wm = (rng.standard_normal((40, 96)) / np.sqrt(96)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_matmul.npz"), x=xm, w=wm, y_bf16=model["_matmul"](xm, wm),
                        y_f32=model["_matmul"](xm, wm, out=lambda a: a))

    # 4. _attention: [B, S, D] values already rounded to bfloat16, HEADS heads, causal
    rng = np.random.default_rng(102)
    q, k, v = (model["_bf16"](rng.standard_normal((2, model["SEQ"], model["DIM"])).astype(np.float32)) for _ in range(3))
    np.savez_compressed(os.path.join(HERE, "reference_attention_bf16.npz"), q=q, k=k, v=v, heads=model["HEADS"],
                        o=model["_attention"](q, k, v))

    # 5. _logits: the whole forward model
    weights = model_weights(model, seed=0)
    ids = np.random.default_rng(1).integers(0, model["VOCAB"], (model["BATCH"], model["SEQ"])).astype(np.int64)
    logits = model["_logits"](weights, ids)
    np.savez_compressed(os.path.join(HERE, "reference_logits.npz"), ids=ids, logits=logits,
                        config=np.array([model[k] for k in ("VOCAB", "SEQ", "DIM", "HEADS", "HIDDEN", "LAYERS", "BATCH")]),
                        **{"w." + name: value for name, value in weights.items()})

    # 6. reference(): float64 attention on the reference's own case shapes (b, sq, sk, n, nkv, h, hv), causal flag.
    # The inputs are redrawn from the seed by the test (`attention_case_inputs`); their sums are stored to catch a
    # generator that draws differently. Outputs are stored as float32 (the tightest tolerance applied is 2e-6).
    out = {"cases": np.array([list(shape) + [int(causal)] for shape, causal in attn["CASES"]], np.int64),
           "tol_bfloat16": attn["TOL"]["bfloat16"], "tol_float32": attn["TOL"]["float32"]}
    for i, (shape, causal) in enumerate(attn["CASES"]):
        q, k, v = attention_case_inputs(i, shape)
        out[f"sums{i}"] = np.array([a.astype(np.float64).sum() for a in (q, k, v)])
        out[f"o{i}"] = attn["reference"](q, k, v, causal=causal).astype(np.float32)
        # the reference's bfloat16 tests compare with reference() of the ROUNDED tensors' values (test_attention.py:33-43)
        qb, kb, vb = (model["_bf16"](a) for a in (q, k, v))
        out[f"ob{i}"] = attn["reference"](qb, kb, vb, causal=causal).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_attention_f64.npz"), **out)
    for name in sorted(os.listdir(HERE)):
        if name.startswith("reference_") and name.endswith(".npz"):
            print(name, os.path.getsize(os.path.join(HERE, name)), "bytes")


if __name__ == "__main__":
    main()
