"""Weights in and out of the training step in the safetensors format, over NumPy arrays (the form parameters take on
either side of `lumen_b200.transformer.TrainStep`). The counterpart of `lumen.safetensors`
(lumen/safetensors/__init__.py:1-70, lumen/safetensors/mod.rs:490-606,672-760): an 8-byte little-endian header
length, a compact JSON header (`__metadata__` first, then each tensor's dtype name, shape and byte range), padded
with spaces to a multiple of 8, then the tensors' bytes packed back to back - widest dtypes first, then by name,
which keeps every tensor's offset a multiple of its element size. Headers are validated on read exactly as the
reference does: ranges tile the data section from 0, sizes match shape and dtype, names are unique."""

from __future__ import annotations

import json
import os
import tempfile

import numpy as np

try:  # the NumPy bfloat16 dtype
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except ImportError:  # bfloat16 tensors are then reported as unsupported
    _BF16 = None

MAX_HEADER_SIZE = 100_000_000

# the format's dtype names in the order the reference's enum gives them (lumen/safetensors/mod.rs:113-137): the sort key
_ORDER = ["BOOL", "F4", "F6_E2M3", "F6_E3M2", "U8", "I8", "F8_E5M2", "F8_E4M3", "F8_E8M0", "F8_E4M3FNUZ", "F8_E5M2FNUZ",
          "I16", "U16", "F16", "BF16", "I32", "U32", "F32", "C64", "F64", "I64", "U64"]  # fmt: skip
_BITS = dict(zip(_ORDER, [8, 4, 6, 6, 8, 8, 8, 8, 8, 8, 8, 16, 16, 16, 16, 32, 32, 32, 64, 64, 64, 64]))
_NUMPY = {
    "BOOL": np.dtype(np.bool_), "U8": np.dtype(np.uint8), "I8": np.dtype(np.int8), "I16": np.dtype("<i2"),
    "U16": np.dtype("<u2"), "F16": np.dtype("<f2"), "I32": np.dtype("<i4"), "U32": np.dtype("<u4"),
    "F32": np.dtype("<f4"), "F64": np.dtype("<f8"), "I64": np.dtype("<i8"), "U64": np.dtype("<u8"),
}  # fmt: skip
if _BF16 is not None:
    _NUMPY["BF16"] = _BF16
_NAME = {v: k for k, v in _NUMPY.items()}


def _flatten(tensors):
    """`(name, array)` pairs in data order, checked as the reference checks them (`_flatten`, `prepare`)."""
    if not isinstance(tensors, dict):
        raise ValueError(f"Expected a dict of [str, numpy.ndarray] but received {type(tensors)}")
    bases = {}
    for name, t in tensors.items():
        if not isinstance(t, np.ndarray):
            raise ValueError(f"Key `{name}` is invalid, expected numpy.ndarray but received {type(t)}")
        if t.dtype not in _NAME:
            raise ValueError(f"tensor `{name}` has dtype {t.dtype}, which safetensors does not support")
        if not t.flags["C_CONTIGUOUS"]:
            raise ValueError(f"tensor `{name}` is not contiguous")
        root = t
        while isinstance(root.base, np.ndarray):
            root = root.base
        if t.size:
            bases.setdefault(id(root), []).append(name)
    shared = [names for names in bases.values() if len(names) > 1]
    if shared:
        raise RuntimeError(
            f"Some tensors share memory, which would be written twice and loaded as separate tensors: {shared}."
            " Save one tensor of each storage."
        )
    return sorted(tensors.items(), key=lambda kv: (-_ORDER.index(_NAME[kv[1].dtype]), kv[0]))


def _header(order, metadata) -> bytes:
    parts = []
    if metadata is not None:
        for k, v in metadata.items():
            if not isinstance(k, str) or not isinstance(v, str):
                raise ValueError("metadata maps strings to strings")
        body = ",".join(f"{json.dumps(k, ensure_ascii=False)}:{json.dumps(v, ensure_ascii=False)}" for k, v in sorted(metadata.items()))
        parts.append('"__metadata__":{' + body + "}")
    offset = 0
    for name, t in order:
        shape = ",".join(str(d) for d in t.shape)
        parts.append(f'{json.dumps(name, ensure_ascii=False)}:{{"dtype":"{_NAME[t.dtype]}","shape":[{shape}],"data_offsets":[{offset},{offset + t.nbytes}]}}')
        offset += t.nbytes
    header = ("{" + ",".join(parts) + "}").encode()
    header += b" " * (-len(header) % 8)
    if len(header) > MAX_HEADER_SIZE:
        raise ValueError(f"header too large (over {MAX_HEADER_SIZE} bytes)")
    return header


def save(tensors, metadata=None) -> bytes:
    """`tensors` (`{name: contiguous array}`) as the bytes of a safetensors file, with optional string `metadata`."""
    order = _flatten(tensors)
    header = _header(order, metadata)
    return b"".join([len(header).to_bytes(8, "little"), header, *[t.tobytes() for _, t in order]])


def save_file(tensors, filename, metadata=None) -> None:
    """Writes `tensors` to `filename` through a temporary file renamed over it, so readers never see it half-written."""
    filename = os.fspath(filename)
    order = _flatten(tensors)
    header = _header(order, metadata)
    fd, tmp = tempfile.mkstemp(dir=os.path.dirname(os.path.abspath(filename)), prefix=".tmp-", suffix=".safetensors")
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(len(header).to_bytes(8, "little"))
            f.write(header)
            for _, t in order:
                f.write(t.reshape(-1).view(np.uint8).data if t.size else b"")  # raw bytes, no copy (bfloat16 has no buffer format)
        os.replace(tmp, filename)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def read_metadata(data) -> tuple[int, dict, list]:
    """The header of safetensors bytes: `(offset of the data section, metadata or None, [(name, dtype name, shape,
    (start, end))] in data order)`, validated (lumen/safetensors/mod.rs:290-322,672-730)."""
    if len(data) < 8:
        raise ValueError("header too small")
    n = int.from_bytes(bytes(data[:8]), "little")
    if n > MAX_HEADER_SIZE:
        raise ValueError(f"header too large (over {MAX_HEADER_SIZE} bytes)")
    if 8 + n > len(data):
        raise ValueError("invalid header length")
    try:
        header = json.loads(bytes(data[8 : 8 + n]).decode("utf-8"), object_pairs_hook=list)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise ValueError(f"invalid JSON in header: {e}") from None
    if not isinstance(header, list):
        raise ValueError("invalid header: not a JSON object")
    metadata, infos, seen = None, [], set()
    for name, value in header:
        if name == "__metadata__":
            metadata = {k: v for k, v in value}
            if not all(isinstance(v, str) for v in metadata.values()):
                raise ValueError("invalid header: metadata maps strings to strings")
            continue
        if name in seen:
            raise ValueError(f"invalid header: duplicate tensor `{name}`")
        seen.add(name)
        info = dict(value)
        dtype, shape, (start, end) = info["dtype"], [int(d) for d in info["shape"]], info["data_offsets"]
        if dtype not in _ORDER:
            raise ValueError(f"invalid header: unknown dtype {dtype} of tensor `{name}`")
        infos.append((name, dtype, shape, (int(start), int(end))))
    infos.sort(key=lambda i: i[3])
    at = 0
    for name, dtype, shape, (start, end) in infos:
        if start != at or end < start:
            raise ValueError(f"invalid offset for tensor `{name}`")
        at = end
        total = width = _BITS[dtype]
        for d in shape:
            total *= d
        if total % 8:
            raise ValueError("misaligned slice")
        if end - start != total // 8:
            raise ValueError(f"tensor `{name}`: byte range does not match its shape and dtype")
    if 8 + n + at != len(data):
        raise ValueError("metadata incomplete buffer" if 8 + n + at > len(data) else "data section longer than the header says")
    return 8 + n, metadata, infos


def _array(data, base, name, dtype, shape, span):
    if dtype not in _NUMPY:
        raise ValueError(f"tensor `{name}` has dtype {dtype}, which lumen does not support")
    start, end = span
    return np.frombuffer(bytes(data[base + start : base + end]), dtype=_NUMPY[dtype]).reshape(shape).copy()


def load(data) -> dict:
    """The tensors in safetensors bytes, as `{name: array}` (arrays own their memory)."""
    base, _, infos = read_metadata(data)
    return {name: _array(data, base, name, dtype, shape, span) for name, dtype, shape, span in infos}


class safe_open:  # noqa: N801 (the reference's name)
    """Header parsed up front, tensors read from the file on demand (lumen/safetensors/mod.rs:753-820)."""

    def __init__(self, filename):
        self._file = open(os.fspath(filename), "rb")
        head = self._file.read(8)
        n = int.from_bytes(head, "little") if len(head) == 8 else 0
        if len(head) < 8 or n > MAX_HEADER_SIZE:
            self._file.close()
            raise ValueError("header too small" if len(head) < 8 else f"header too large (over {MAX_HEADER_SIZE} bytes)")
        size = os.fstat(self._file.fileno()).st_size
        header = head + self._file.read(n)
        # validate against the file's size without reading the data section
        self._base, self._metadata, self._infos = read_metadata(_Sized(header, size))
        self._by_name = {i[0]: i for i in self._infos}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self._file.close()
        self._file = None

    def _open(self):
        if self._file is None:
            raise ValueError("the file is closed")
        return self._file

    def keys(self):
        self._open()
        return sorted(self._by_name)

    def offset_keys(self):
        self._open()
        return [i[0] for i in self._infos]

    def metadata(self):
        self._open()
        return self._metadata

    def get_tensor(self, name):
        f = self._open()
        if name not in self._by_name:
            raise KeyError(f"tensor `{name}` is missing from the file")
        _, dtype, shape, (start, end) = self._by_name[name]
        if dtype not in _NUMPY:
            raise ValueError(f"tensor `{name}` has dtype {dtype}, which lumen does not support")
        f.seek(self._base + start)
        return np.frombuffer(f.read(end - start), dtype=_NUMPY[dtype]).reshape(shape).copy()

    def get_tensors(self):
        return [(name, self.get_tensor(name)) for name in self.offset_keys()]


class _Sized:
    """Header bytes that answer `len()` with the whole file's size (read_metadata checks the data section's length)."""

    def __init__(self, head: bytes, size: int):
        self.head, self.size = head, size

    def __len__(self):
        return self.size

    def __getitem__(self, s):
        return self.head[s]


def load_file(filename) -> dict:
    """The tensors in safetensors file `filename`, as `{name: array}`."""
    with safe_open(filename) as f:
        return dict(f.get_tensors())
