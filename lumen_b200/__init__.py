"""lumen_b200: a B200-native CUDA execution backend for lumen's compiled graphs."""


def compile(fn, device="cuda", use_graphs=False, lowering="native"):  # noqa: A001
    """`lumen.compile(fn, device="cuda")` for this backend (see `lumen_b200.compiled`)."""
    from lumen_b200.compiled import compile as _compile

    return _compile(fn, device, use_graphs, lowering)
