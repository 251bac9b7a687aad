"""GPU parity of the four unfused operators (and the buffer layer) against the
oracle, through the C ABI.  Written the way tests of rusty-backend's
ComputeEngine would read."""
import numpy as np
import pytest

from parity import TOL_FP32, assert_bits_equal, rel_err
from rusty_b200 import BackendError, DType, UnifiedTensor

pytestmark = pytest.mark.gpu


def test_adapter_info(ctx):
    info = ctx.adapter_info()
    assert "CUDA sm_100" in info, info


def test_ops_test_matmul_identity(ctx, engine, kat):
    a = UnifiedTensor.new(ctx, [1.0, 2.0, 3.0, 4.0], [2, 2])
    b = UnifiedTensor.new(ctx, [1.0, 0.0, 0.0, 1.0], [2, 2])
    out = UnifiedTensor.empty(ctx, [2, 2])
    engine.matmul(ctx, a, b, out)
    assert out.to_vec(ctx).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_matmul_tails_bit_exact_vs_fma_oracle(ctx, engine, kat):
    for i in range(int(kat["mm_count"])):
        a, b = kat[f"mm{i}_a"], kat[f"mm{i}_b"]
        M, K = a.shape
        N = b.shape[1]
        ta, tb = UnifiedTensor.new(ctx, a, [M, K]), UnifiedTensor.new(ctx, b, [K, N])
        out = UnifiedTensor.empty(ctx, [M, N])
        engine.matmul(ctx, ta, tb, out)
        got = out.to_vec(ctx).reshape(M, N)
        assert_bits_equal(got, kat[f"mm{i}_out_fma"])          # shader order under FMA contraction
        assert rel_err(got, kat[f"mm{i}_out"]) <= TOL_FP32     # and within tolerance of the uncontracted text
        tbt = UnifiedTensor.new(ctx, np.ascontiguousarray(b.T), [N, K])
        out2 = UnifiedTensor.empty(ctx, [M, N])
        engine.matmul_bt(ctx, ta, tbt, out2)
        assert_bits_equal(out2.to_vec(ctx).reshape(M, N), kat[f"mm{i}_bt_out_fma"])


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (33, 1000, 257), (128, 512, 640)])
def test_matmul_larger_vs_oracle(ctx, engine, oracle, M, K, N):
    rng = np.random.default_rng(M * 7 + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    ta, tb = UnifiedTensor.new(ctx, a, [M, K]), UnifiedTensor.new(ctx, b, [K, N])
    out = UnifiedTensor.empty(ctx, [M, N])
    engine.matmul(ctx, ta, tb, out)
    got = out.to_vec(ctx).reshape(M, N)
    rows = slice(0, min(M, 4))  # the scalar oracle on a few rows; all of them for M=1
    assert_bits_equal(got[rows], oracle.matmul_tiled(a[rows], b, fma=True))
    assert rel_err(got[rows], oracle.matmul_tiled(a[rows], b)) <= TOL_FP32
    assert rel_err(got, a.astype(np.float64) @ b.astype(np.float64)) <= TOL_FP32


def test_dequantize_kats(ctx, engine, kat):
    raw = kat["deq_in"]
    t_in = UnifiedTensor.from_bytes_with_dtype(ctx, raw, [raw.size], DType.U8)
    out = UnifiedTensor.empty(ctx, [raw.size])
    engine.dequantize(ctx, t_in, out)
    assert_bits_equal(out.to_vec(ctx), kat["deq_out"])
    big = kat["deq_big_in"]
    t_in = UnifiedTensor.from_bytes_with_dtype(ctx, big, [big.size], DType.U8)
    out = UnifiedTensor.empty(ctx, [big.size])
    engine.dequantize(ctx, t_in, out)
    assert_bits_equal(out.to_vec(ctx), kat["deq_big_out"])


def test_dequantize_ragged(ctx, engine, kat):
    raw = kat["deq_in"]
    # 7 outputs only: the shader's per-store guard drops the 8th value
    t_in = UnifiedTensor.from_bytes_with_dtype(ctx, raw[:8], [7], DType.U8)
    out = UnifiedTensor.new(ctx, np.full(7, -1.0, np.float32), [7])
    engine.dequantize(ctx, t_in, out)
    assert_bits_equal(out.to_vec(ctx), kat["deq_out_n7"])
    # input buffer holds 2 words but the shape claims 12 bytes: outputs past the input stay untouched
    t_in = UnifiedTensor.from_bytes_with_dtype(ctx, raw[:8], [12], DType.U8)
    out = UnifiedTensor.new(ctx, np.full(12, -1.0, np.float32), [12])
    engine.dequantize(ctx, t_in, out)
    assert_bits_equal(out.to_vec(ctx), kat["deq_out_short_in"])


def test_dequantize_config1_weight_exact(ctx, engine, oracle):
    """Every byte of the 4096x4096 weight unpacks bit-exactly (16.7 M values)."""
    rng = np.random.default_rng(0)
    raw = rng.integers(0, 256, size=4096 * 4096, dtype=np.uint8)
    t_in = UnifiedTensor.from_bytes_with_dtype(ctx, raw, [4096, 4096], DType.U8)
    out = UnifiedTensor.empty(ctx, [4096, 4096])
    engine.dequantize(ctx, t_in, out)
    got = out.to_vec(ctx)
    assert np.array_equal(got.view(np.uint32), raw.astype(np.float32).view(np.uint32))
    assert_bits_equal(got[:4096], oracle.dequantize(raw[:4096]))


def test_affine_dequantize_kat_bit_exact(ctx, engine, kat):
    u, s, b = kat["aff_u"], kat["aff_s"], kat["aff_b"]
    w = UnifiedTensor.from_bytes_with_dtype(ctx, np.concatenate([u, np.zeros(5, np.uint8)]), [u.size], DType.U8)
    out = UnifiedTensor.empty(ctx, [u.size])
    engine.affine_dequantize(ctx, w, UnifiedTensor.new(ctx, s, [s.size]), UnifiedTensor.new(ctx, b, [b.size]), out)
    assert_bits_equal(out.to_vec(ctx), kat["aff_out"])


def test_affine_dequantize_beyond_reference_dispatch_limit(ctx, engine, oracle):
    """n > 4 194 240: the reference's dispatch leaves the tail unwritten; this
    implementation writes every element with the intended arithmetic."""
    n = 4096 * 4096
    rng = np.random.default_rng(11)
    u = rng.integers(0, 256, size=n, dtype=np.uint8)
    s = rng.uniform(0.001, 0.02, size=n // 64).astype(np.float32)
    b = rng.uniform(-2, 2, size=n // 64).astype(np.float32)
    w = UnifiedTensor.from_bytes_with_dtype(ctx, u, [4096, 4096], DType.U8)
    out = UnifiedTensor.empty(ctx, [4096, 4096])
    engine.affine_dequantize(ctx, w, UnifiedTensor.new(ctx, s, [s.size]), UnifiedTensor.new(ctx, b, [b.size]), out)
    got = out.to_vec(ctx)
    assert_bits_equal(got, oracle.affine_dequantize(u, s, b, mt=True))


def test_add(ctx, engine):
    a = UnifiedTensor.new(ctx, [1.0, 2.0, 3.0, 4.0], [4])
    b = UnifiedTensor.new(ctx, [5.0, 6.0, 7.0, 8.0], [4])
    out = UnifiedTensor.empty(ctx, [4])
    engine.add(ctx, a, b, out)
    assert out.to_vec(ctx).tolist() == [6.0, 8.0, 10.0, 12.0]


# ---- buffer layer: pool bins, views, copy_tensor, errors ----

def test_pool_returns_exact_size_bins(ctx):
    ctx.pool_clear()
    nbytes = 12345 * 4
    t = UnifiedTensor.empty(ctx, [12345])
    p = t.device_ptr()
    assert ctx.pool_idle_count(nbytes) == 0
    del t
    assert ctx.pool_idle_count(nbytes) == 1
    t2 = UnifiedTensor.empty(ctx, [12345])           # same size: same buffer comes back
    assert t2.device_ptr() == p and ctx.pool_idle_count(nbytes) == 0
    t3 = UnifiedTensor.empty(ctx, [12346])           # other size: other bin
    assert t3.device_ptr() != p
    del t2, t3
    fresh = UnifiedTensor.new(ctx, np.zeros(12345, np.float32), [12345])  # `new` is not pooled
    del fresh
    assert ctx.pool_idle_count(nbytes) == 1
    ctx.pool_clear()
    assert ctx.pool_idle_count(nbytes) == 0


def test_reshaped_shares_storage(ctx):
    t = UnifiedTensor.new(ctx, np.arange(12, dtype=np.float32), [3, 4])
    v = t.reshaped([2, 6])
    assert v.device_ptr() == t.device_ptr() and v.shape == [2, 6]
    with pytest.raises(AssertionError):
        t.reshaped([5, 5])
    del t
    assert v.to_vec(ctx).tolist() == list(range(12))


def test_copy_tensor_with_offset(ctx, engine):
    src = UnifiedTensor.new(ctx, [1.0, 2.0], [2])
    dst = UnifiedTensor.zeros(ctx, [5])
    engine.copy_tensor(ctx, src, dst, 8)
    assert dst.to_vec(ctx).tolist() == [0.0, 0.0, 1.0, 2.0, 0.0]
    with pytest.raises(BackendError) as e:
        engine.copy_tensor(ctx, src, dst, 16)
    assert e.value.kind == "BufferOperation"


def test_shape_errors_are_status_codes(ctx, engine):
    a = UnifiedTensor.new(ctx, np.zeros(6, np.float32), [2, 3])
    b = UnifiedTensor.new(ctx, np.zeros(6, np.float32), [3, 2])
    small = UnifiedTensor.empty(ctx, [1, 2])
    with pytest.raises(BackendError) as e:
        engine.matmul(ctx, a, b, small)
    assert e.value.kind == "InvalidDimensions"
    ctx.sync()  # the context is still usable


def test_release_while_a_capture_is_open_is_deferred(ctx, engine):
    """A host-language destructor may run at any time, also between graph_begin and graph_end; freeing device memory
    or synchronising there would invalidate the capture, so the release is parked until the capture has ended."""
    from rusty_b200 import QLinear
    from rusty_b200.backend import Graph
    from rusty_b200.workloads import sym_row_linear
    rng = np.random.default_rng(3)
    a = rng.standard_normal(1000).astype(np.float32)
    b = rng.standard_normal(1000).astype(np.float32)
    ta, tb, out = UnifiedTensor.new(ctx, a, [1000]), UnifiedTensor.new(ctx, b, [1000]), UnifiedTensor.empty(ctx, [1000])
    victim = UnifiedTensor.new(ctx, a, [1000])          # not pooled: its release is a cudaFree
    x, q, s = sym_row_linear(0, 1, 256, 64)
    ql_victim = QLinear.from_host(ctx, q, s)             # a whole fused linear dies inside the capture as well
    old = Graph(ctx)
    with old:
        engine.add(ctx, ta, tb, out)
    g = Graph(ctx)
    with g:
        engine.add(ctx, ta, tb, out)
        del victim
        del ql_victim
        del old                                          # a graph destroyed while another capture is open
        engine.add(ctx, out, tb, out)
    g.launch()
    ctx.sync()
    assert np.array_equal(out.to_vec(ctx), (a + b) + b)
    # the context is fully usable afterwards (allocations, eager launches, another capture)
    t2 = UnifiedTensor.new(ctx, b, [1000])
    engine.add(ctx, t2, t2, out)
    assert np.array_equal(out.to_vec(ctx), b + b)
    g2 = Graph(ctx)
    with g2:
        engine.add(ctx, ta, ta, out)
    g2.launch()
    assert np.array_equal(out.to_vec(ctx), a + a)
