"""Host side of the quantised-weight loader: the safetensors container, the name map and the row shards
(rusty-loader/src/lib.rs:97-218 is the reference interface).  No GPU."""
import json
import struct

import numpy as np
import pytest

from rusty_b200 import capi
from rusty_b200.loader import GROUP, LoaderError, WeightsContext, save_file


def _quantized(rng, shape):
    total = int(np.prod(shape))
    q = rng.integers(0, 256, size=shape, dtype=np.uint8)
    groups = (total + GROUP - 1) // GROUP
    s = rng.uniform(0.001, 0.02, size=groups).astype(np.float32)
    b = (-128.0 * s).astype(np.float32)
    return q, s, b


def _dequant(q, s, b):
    flat = q.reshape(-1).astype(np.float32)
    g = np.arange(flat.size) // GROUP
    return (flat * s[g] + b[g]).reshape(q.shape)


def test_container_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    q, s, b = _quantized(rng, (96, 128))
    emb = rng.standard_normal((10, 16)).astype(np.float32)
    half = rng.standard_normal((3, 5)).astype(np.float16)
    path = str(tmp_path / "model.safetensors")
    save_file(path, {"l0.q_proj.weight": q, "l0.q_proj.scales": s, "l0.q_proj.biases": b, "embed.weight": emb, "h": half},
              metadata={"format": "pt"})
    w = WeightsContext()
    w.load_file(path)
    assert set(w.names()) == {"l0.q_proj.weight", "l0.q_proj.scales", "l0.q_proj.biases", "embed.weight", "h"}
    assert w.get_tensor_info("l0.q_proj.weight") == ([96, 128], "U8")
    assert w.get_tensor_info("embed.weight") == ([10, 16], "F32")
    assert w.get_tensor_info("nope") is None
    assert np.array_equal(w.read_array("embed.weight"), emb)
    assert np.array_equal(w.read_array("h"), half)
    raw, shape = w.read_bytes("l0.q_proj.weight")
    assert shape == [96, 128] and raw.dtype == np.uint8 and np.array_equal(raw.reshape(shape), q)
    assert w.is_quantized("l0.q_proj") and not w.is_quantized("embed")
    with pytest.raises(LoaderError) as e:
        w.read_bytes("missing.weight")
    assert e.value.kind == "MissingWeight"


def test_header_is_the_published_layout(tmp_path):
    path = str(tmp_path / "t.safetensors")
    a = np.arange(6, dtype=np.int32).reshape(2, 3)
    save_file(path, {"a": a})
    blob = open(path, "rb").read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    assert header["a"] == {"dtype": "I32", "shape": [2, 3], "data_offsets": [0, 24]}
    assert blob[8 + n:] == a.tobytes() and (8 + n) % 8 == 0


@pytest.mark.parametrize("damage", ["short", "length", "json", "offsets", "dtype", "overlap"])
def test_malformed_files_are_rejected(tmp_path, damage):
    path = str(tmp_path / "bad.safetensors")
    good = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    if damage == "short":
        blob = b"\x01\x02"
    elif damage == "length":
        blob = struct.pack("<Q", 1 << 40) + b"{}"
    elif damage == "json":
        blob = struct.pack("<Q", 4) + b"{{{{"
    else:
        if damage == "offsets":
            good["a"]["data_offsets"] = [0, 12]
        elif damage == "overlap":
            good["b"] = {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}
        else:
            good["a"]["dtype"] = "Q4"
        hj = json.dumps(good).encode()
        blob = struct.pack("<Q", len(hj)) + hj + b"\0" * 8
    open(path, "wb").write(blob)
    with pytest.raises(LoaderError):
        WeightsContext().load_file(path)


def test_missing_file_is_an_io_error(tmp_path):
    with pytest.raises(LoaderError) as e:
        WeightsContext().load_file(str(tmp_path / "absent.safetensors"))
    assert e.value.kind == "Io"


def test_row_shards_reassemble_the_dequantised_matrix(tmp_path):
    rng = np.random.default_rng(1)
    n, k = 32, 192
    q, s, b = _quantized(rng, (n, k))
    path = str(tmp_path / "m.safetensors")
    save_file(path, {"w.weight": q, "w.scales": s, "w.biases": b})
    w = WeightsContext()
    w.load_file(path)
    full = _dequant(q, s, b)
    for world in (1, 2, 4):
        parts = []
        for rank in range(world):
            q2, s2, b2 = w.quantized_shard("w", capi.LAYOUT_NK, rank, world)
            assert q2.shape == (n // world, k) and s2.size == b2.size == n // world * k // GROUP
            parts.append(_dequant(q2, s2, b2))
        assert np.array_equal(np.concatenate(parts, axis=0), full)
    with pytest.raises(LoaderError):
        w.quantized_shard("w", capi.LAYOUT_KN, 0, 2)       # read as [in,out] = [32, 192]: 96 columns per rank are not whole groups
    with pytest.raises(LoaderError):
        w.quantized_shard("w", capi.LAYOUT_NK, 0, 3)       # 32 rows do not split three ways


def test_column_shards_of_in_out_storage_reassemble_the_dequantised_matrix(tmp_path):
    """rusty's own [in,out] storage: groups of 64 run along the output dimension, a rank keeps whole groups of every row."""
    rng = np.random.default_rng(5)
    k, n = 24, 512
    q, s, b = _quantized(rng, (k, n))
    path = str(tmp_path / "m.safetensors")
    save_file(path, {"w.weight": q, "w.scales": s, "w.biases": b})
    w = WeightsContext()
    w.load_file(path)
    full = _dequant(q, s, b)
    for world in (1, 2, 4, 8):
        parts = []
        for rank in range(world):
            q2, s2, b2 = w.quantized_shard("w", capi.LAYOUT_KN, rank, world)
            assert q2.shape == (k, n // world) and q2.flags["C_CONTIGUOUS"] and s2.size == b2.size == k * n // world // GROUP
            parts.append(_dequant(q2, s2, b2))
        assert np.array_equal(np.concatenate(parts, axis=1), full)
    with pytest.raises(LoaderError):
        w.quantized_shard("w", capi.LAYOUT_KN, 0, 16)      # 32 columns per rank: half a group
    with pytest.raises(LoaderError):
        w.quantized_shard("w", capi.LAYOUT_KN, 0, 3)


def test_too_few_scales_is_an_error(tmp_path):
    rng = np.random.default_rng(2)
    q, s, b = _quantized(rng, (4, 128))
    path = str(tmp_path / "m.safetensors")
    save_file(path, {"w.weight": q, "w.scales": s[:-1], "w.biases": b})
    w = WeightsContext()
    w.load_file(path)
    with pytest.raises(LoaderError):
        w.quantized_shard("w")
