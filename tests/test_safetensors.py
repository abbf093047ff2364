"""`lumen_b200.safetensors` (weights in and out of the training step) against the behaviour the reference's tests
pin for `lumen.safetensors` (tests/safetensors/test_safetensors.py:42-111): the documented header bytes, round trips
of every dtype, lazy reads, atomic file writes, and the errors."""

import numpy as np
import pytest

from lumen_b200 import transformer
from lumen_b200.safetensors import load, load_file, read_metadata, safe_open, save, save_file
from tests.helpers import BF16

DTYPES = ["bool", "uint8", "uint16", "uint32", "uint64", "int8", "int16", "int32", "int64", "float16", "bfloat16", "float32", "float64"]


def tensors():
    """A small 2 x 3 array of each supported dtype, keyed by dtype."""
    values = np.arange(6).reshape(2, 3) % 5
    return {d: (values != 0 if d == "bool" else values).astype(BF16 if d == "bfloat16" else d) for d in DTYPES}


def assert_same(expected, actual):
    assert sorted(expected) == sorted(actual)
    for name, t in expected.items():
        assert (actual[name].dtype, actual[name].shape) == (t.dtype, t.shape), name
        assert actual[name].tobytes() == t.tobytes(), name


def test_bytes_round_trip_and_documented_header():
    ts = tensors()
    assert_same(ts, load(save(ts)))
    data = save({"attn.0": np.array([[[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]], dtype=np.float32)})
    assert data[:8] == (64).to_bytes(8, "little")
    assert data[8:72] == b'{"attn.0":{"dtype":"F32","shape":[1,2,3],"data_offsets":[0,24]}}'
    padded = save({"w": np.zeros(3, np.uint8)})  # the header is padded with spaces to a multiple of 8
    n = int.from_bytes(padded[:8], "little")
    assert n % 8 == 0 and padded[8 : 8 + n].endswith(b" ") and len(padded) == 8 + n + 3
    assert load(save({"empty": np.zeros((0, 4), np.float32)}))["empty"].shape == (0, 4)


def test_files_safe_open_and_metadata(tmp_path):
    path = tmp_path / "model.safetensors"
    ts = tensors()
    save_file(ts, path, metadata={"format": "lumen"})
    assert_same(ts, load_file(path))
    with safe_open(path) as f:
        assert f.keys() == sorted(DTYPES)
        assert f.offset_keys()[0] in ("float64", "int64", "uint64")  # widest dtypes first, then by name
        assert f.offset_keys()[-1] == "bool"
        assert f.metadata() == {"format": "lumen"}
        assert f.get_tensor("float32").tolist() == [[0.0, 1.0, 2.0], [3.0, 4.0, 0.0]]
        with pytest.raises(KeyError, match="missing"):
            f.get_tensor("missing")
    with pytest.raises(ValueError, match="closed"):
        f.keys()
    assert [p.name for p in tmp_path.iterdir()] == ["model.safetensors"]  # no temporary file is left behind


def test_save_checks():
    w = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    with pytest.raises(ValueError, match="Expected a dict"):
        save([w])
    with pytest.raises(ValueError, match="expected numpy.ndarray"):
        save({"w": [1.0]})
    with pytest.raises(RuntimeError, match="share memory"):
        save({"a": w, "b": w[:1]})
    with pytest.raises(ValueError, match="not contiguous"):
        save({"t": w.T})
    with pytest.raises(ValueError, match="does not support"):
        save({"c": np.zeros(2, np.complex128)})


def test_load_errors(tmp_path):
    with pytest.raises(OSError):
        load_file(tmp_path / "missing.safetensors")
    with pytest.raises(ValueError, match="invalid JSON"):
        load(b"\x01\x00\x00\x00\x00\x00\x00\x00{")
    header = b'{"w":{"dtype":"F8_E4M3","shape":[2],"data_offsets":[0,2]}}'
    with pytest.raises(ValueError, match="F8_E4M3, which lumen does not support"):
        load(len(header).to_bytes(8, "little") + header + b"\x00\x00")

    def file(header, data):
        return len(header).to_bytes(8, "little") + header + data

    with pytest.raises(ValueError, match="invalid offset"):  # ranges have to tile the data section from 0
        load(file(b'{"w":{"dtype":"U8","shape":[2],"data_offsets":[1,3]}}', b"\x00\x00\x00"))
    with pytest.raises(ValueError, match="does not match"):
        load(file(b'{"w":{"dtype":"F32","shape":[2],"data_offsets":[0,4]}}', b"\x00" * 4))
    with pytest.raises(ValueError, match="duplicate"):
        load(file(b'{"w":{"dtype":"U8","shape":[1],"data_offsets":[0,1]},"w":{"dtype":"U8","shape":[1],"data_offsets":[1,2]}}', b"\x00\x00"))
    with pytest.raises(ValueError, match="incomplete"):
        load(file(b'{"w":{"dtype":"U8","shape":[4],"data_offsets":[0,4]}}', b"\x00"))
    with pytest.raises(ValueError, match="too large"):
        read_metadata((200_000_000).to_bytes(8, "little") + b"{}")


def test_transformer_parameters_round_trip(tmp_path):
    """The training step's parameters (bfloat16 and float32 configurations) through a file and back, bit for bit."""
    for cfg in (transformer.Config.baseline_small(), transformer.Config(vocab=64, d_model=32, heads=2, hidden=64, layers=1, seq=16, dtype="bfloat16")):
        params = transformer.init_params(cfg, seed=3)
        path = tmp_path / f"{cfg.dtype}.safetensors"
        save_file(params, path, metadata={"layers": str(cfg.layers)})
        back = load_file(path)
        assert list(sorted(back)) == sorted(params)
        for name, value in params.items():
            assert back[name].dtype == value.dtype and back[name].tobytes() == value.tobytes(), name
