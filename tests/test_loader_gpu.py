"""GPU tests of the quantised-weight loader: a synthetic safetensors checkpoint in the reference's on-disk layout
(rusty-loader/src/lib.rs:155-218) goes to the device both ways: dequantised to f32 as the reference does, and kept
at one byte per weight as a fused linear, whole and as two row shards."""
import numpy as np
import pytest

from parity import TOL_FP32, assert_bits_equal, rel_err
from rusty_b200 import UnifiedTensor, capi
from rusty_b200.loader import GROUP, WeightsContext, save_file

pytestmark = pytest.mark.gpu


def _checkpoint(tmp_path):
    rng = np.random.default_rng(5)
    tensors = {}
    raw = {}
    for name, shape in [("model.layers.0.q_proj", (256, 192)), ("model.layers.0.down_proj", (320, 128))]:
        q = rng.integers(0, 256, size=shape, dtype=np.uint8)
        groups = q.size // GROUP
        s = rng.uniform(0.001, 0.02, size=groups).astype(np.float32)
        b = (-128.0 * s).astype(np.float32)
        tensors[f"{name}.weight"], tensors[f"{name}.scales"], tensors[f"{name}.biases"] = q, s, b
        raw[name] = (q, s, b)
    tensors["model.norm.weight"] = rng.standard_normal(192).astype(np.float32)
    path = str(tmp_path / "model.safetensors")
    save_file(path, tensors)
    w = WeightsContext()
    w.load_file(path)
    return w, raw


def test_upload_quantized_is_the_reference_dequantisation(ctx, engine, oracle, tmp_path):
    w, raw = _checkpoint(tmp_path)
    for name, (q, s, b) in raw.items():
        t = w.upload_quantized(name, ctx, engine)
        assert t.shape == list(q.shape)
        assert_bits_equal(t.to_vec(ctx), oracle.affine_dequantize(q.reshape(-1), s, b))


@pytest.mark.parametrize("M", [1, 7, 48])
def test_upload_qlinear_matches_dequantise_then_matmul(ctx, engine, oracle, tmp_path, M):
    w, raw = _checkpoint(tmp_path)
    rng = np.random.default_rng(M)
    for name, (q, s, b) in raw.items():
        for layout in (capi.LAYOUT_KN, capi.LAYOUT_NK):
            N, K = q.shape if layout == capi.LAYOUT_NK else q.shape[::-1]
            x = rng.standard_normal((M, K)).astype(np.float32)
            ql = w.upload_qlinear(name, ctx, layout=layout)
            assert (ql.N, ql.K) == (N, K)
            xt = UnifiedTensor.new(ctx, x, [M, K])
            y = UnifiedTensor.empty(ctx, [M, N])
            engine.qlinear(ctx, xt, ql, y)
            ref = oracle.qlinear_affine(x, q.reshape(-1), s, b, q.shape, layout_nk=layout == capi.LAYOUT_NK)
            assert rel_err(y.to_vec(ctx).reshape(M, N), ref) <= TOL_FP32


def test_row_shards_give_the_columns_of_the_whole(ctx, engine, tmp_path):
    w, raw = _checkpoint(tmp_path)
    name = "model.layers.0.q_proj"
    q = raw[name][0]
    N, K = q.shape
    M = 5
    x = np.random.default_rng(9).standard_normal((M, K)).astype(np.float32)
    xt = UnifiedTensor.new(ctx, x, [M, K])
    whole = UnifiedTensor.empty(ctx, [M, N])
    engine.qlinear(ctx, xt, w.upload_qlinear(name, ctx, layout=capi.LAYOUT_NK), whole)
    want = whole.to_vec(ctx).reshape(M, N)
    for world in (2, 4):
        cols = []
        for rank in range(world):
            ql = w.upload_qlinear(name, ctx, layout=capi.LAYOUT_NK, rank=rank, world=world)
            y = UnifiedTensor.empty(ctx, [M, N // world])
            engine.qlinear(ctx, xt, ql, y)
            cols.append(y.to_vec(ctx).reshape(M, N // world))
        assert_bits_equal(np.concatenate(cols, axis=1), want)
