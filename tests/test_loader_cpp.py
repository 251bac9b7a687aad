"""The C++ loader mirror (rusty_b200/host/rusty_loader.hpp) against the Python one on the same synthetic checkpoint:
header parsing, row shards (host only, no GPU), error variants; and on a GPU both upload paths."""
import os
import subprocess

import numpy as np
import pytest

from rusty_b200 import capi
from rusty_b200.loader import GROUP, WeightsContext, save_file

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "loader_test.cpp")


def _fnv(b: bytes) -> int:
    h = 1469598103934665603
    for c in b:
        h = ((h ^ c) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cpp") / "loader_test")
    pkg = os.path.join(ROOT, "rusty_b200")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I",
                           os.path.join(pkg, "host"), SRC, "-o", out, "-L", pkg, "-lrusty_cuda", f"-Wl,-rpath,{pkg}"])
    return out


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    rng = np.random.default_rng(8)
    n, k = 64, 192
    q = rng.integers(0, 256, size=(n, k), dtype=np.uint8)
    s = rng.uniform(0.001, 0.02, size=n * k // GROUP).astype(np.float32)
    b = (-128.0 * s).astype(np.float32)
    path = str(tmp_path_factory.mktemp("ckpt") / "model.safetensors")
    save_file(path, {"layers.0.q_proj.weight": q, "layers.0.q_proj.scales": s, "layers.0.q_proj.biases": b,
                     "norm.weight": rng.standard_normal(k).astype(np.float32)}, metadata={"format": "pt", "note": "a \"quoted\" value"})
    return path


def test_header_and_name_map(exe, checkpoint):
    r = subprocess.run([exe, "info", checkpoint, "layers.0.q_proj.weight", "norm.weight", "absent.weight"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.splitlines() == ["layers.0.q_proj.weight U8 64 192 quantized=1", "norm.weight F32 192 quantized=0",
                                     "absent.weight missing"]


@pytest.mark.parametrize("world", [1, 2, 4])
def test_row_shards_match_the_python_loader(exe, checkpoint, world):
    w = WeightsContext()
    w.load_file(checkpoint)
    for rank in range(world):
        q2, s, b = w.quantized_shard("layers.0.q_proj", capi.LAYOUT_NK, rank, world)
        want = f"{q2.shape[0]} {q2.shape[1]} {s.size} {_fnv(q2.tobytes())} {_fnv(s.tobytes())} {_fnv(b.tobytes())}"
        r = subprocess.run([exe, "shard", checkpoint, "layers.0.q_proj", str(rank), str(world)], capture_output=True, text=True,
                           timeout=60)
        assert r.returncode == 0 and r.stdout.strip() == want, r.stdout + r.stderr


@pytest.mark.parametrize("world", [1, 3])
def test_column_shards_of_in_out_storage_match_the_python_loader(exe, checkpoint, world):
    """The same tensor read as [in,out] = [64, 192]: three column shards of one 64-group each."""
    w = WeightsContext()
    w.load_file(checkpoint)
    for rank in range(world):
        q2, s, b = w.quantized_shard("layers.0.q_proj", capi.LAYOUT_KN, rank, world)
        want = f"{q2.shape[0]} {q2.shape[1]} {s.size} {_fnv(q2.tobytes())} {_fnv(s.tobytes())} {_fnv(b.tobytes())}"
        r = subprocess.run([exe, "shard_kn", checkpoint, "layers.0.q_proj", str(rank), str(world)], capture_output=True, text=True,
                           timeout=60)
        assert r.returncode == 0 and r.stdout.strip() == want, r.stdout + r.stderr
    r = subprocess.run([exe, "shard_kn", checkpoint, "layers.0.q_proj", "0", "2"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Safetensors"     # 96 columns are not whole groups


def test_error_variants(exe, checkpoint, tmp_path):
    r = subprocess.run([exe, "info", str(tmp_path / "absent.safetensors")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Io"
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((4).to_bytes(8, "little") + b"{{{{")
    r = subprocess.run([exe, "info", str(bad)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Json"
    # a crafted shape whose element count wraps around 2^64: [2^32, 2^32] over zero bytes must be refused, not
    # accepted as an empty tensor with huge dimensions
    import json
    hdr = json.dumps({"w.weight": {"dtype": "U8", "shape": [2 ** 32, 2 ** 32], "data_offsets": [0, 0]}}).encode()
    wrap = tmp_path / "wrap.safetensors"
    wrap.write_bytes(len(hdr).to_bytes(8, "little") + hdr)
    r = subprocess.run([exe, "info", str(wrap), "w.weight"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Safetensors", r.stdout + r.stderr
    # two tensors over the same bytes
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}).encode()
    lap = tmp_path / "overlap.safetensors"
    lap.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    r = subprocess.run([exe, "info", str(lap), "a"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Safetensors", r.stdout + r.stderr
    r = subprocess.run([exe, "shard", checkpoint, "norm", "0", "1"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError MissingWeight"   # norm has no quantised parts
    r = subprocess.run([exe, "shard", checkpoint, "layers.0.q_proj", "0", "3"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "LoaderError Safetensors"     # 64 rows do not split three ways


@pytest.mark.gpu
def test_both_upload_paths_on_the_device(exe, checkpoint):
    r = subprocess.run([exe, "gpu", checkpoint, "layers.0.q_proj"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
