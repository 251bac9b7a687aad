"""SwiGLU glue of the MLP (rusty-graph/src/lib.rs:317-323): the unfused `silu` and `mul` operators against the oracle's
restatement of the two shaders, and the fused form — a pair-interleaved gate|up weight whose kernels write
silu(x.gate) * (x.up) from their epilogue — against "two linears, silu, mul" composed from the oracle."""
import numpy as np
import pytest

from parity import TOL_BF16, TOL_FP32, rel_err
from rusty_b200 import BackendError, DType, QLinear, UnifiedTensor, capi
from rusty_b200.backend import interleave_pairs

pytestmark = pytest.mark.gpu


def test_silu_and_mul_match_the_shaders(ctx, engine, oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(1000).astype(np.float32) * 4, np.array([0.0, -0.0, 30.0, -30.0, 88.0, -88.0], np.float32)])
    y = rng.standard_normal(x.size).astype(np.float32)
    tx, ty = UnifiedTensor.new(ctx, x, [x.size]), UnifiedTensor.new(ctx, y, [x.size])
    out = UnifiedTensor.empty(ctx, [x.size])
    engine.silu(ctx, tx, out)
    got = out.to_vec(ctx)
    assert np.isfinite(got).all()
    assert rel_err(got, oracle.silu(x)) <= TOL_FP32
    engine.mul(ctx, tx, ty, out)
    assert np.array_equal(out.to_vec(ctx).view(np.uint32), oracle.mul(x, y).view(np.uint32))


def _pairs_case(seed, M, K, F):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    gq = rng.integers(-127, 128, size=(F, K), dtype=np.int8)
    uq = rng.integers(-127, 128, size=(F, K), dtype=np.int8)
    # scales chosen so that the gate lands in the curved part of silu
    gs = rng.uniform(0.0005, 0.002, size=F).astype(np.float32)
    us = rng.uniform(0.001, 0.02, size=F).astype(np.float32)
    return x, gq, gs, uq, us


def _reference(oracle, x, gq, gs, uq, us):
    g = oracle.qlinear_rowscale(x, gq, gs)
    u = oracle.qlinear_rowscale(x, uq, us)
    return oracle.mul(oracle.silu(g), u)


@pytest.mark.parametrize("M,K,F", [(1, 256, 64), (2, 1024, 96), (4, 512, 200), (5, 512, 64), (32, 4096, 1024),
                                   (32, 1024, 7168), (37, 256, 70), (64, 2048, 512), (100, 512, 192)])
def test_fused_pairs_match_two_linears_silu_mul(ctx, engine, oracle, M, K, F):
    x, gq, gs, uq, us = _pairs_case(M * 7 + F, M, K, F)
    ql = QLinear.from_gate_up(ctx, gq, gs, uq, us)
    assert ql.out_features == F and ql.plan(M) in ("gemv", "gemv_mma", "tcgen05")
    xt = UnifiedTensor.new(ctx, x, [M, K])
    y = UnifiedTensor.new(ctx, np.full(M * F, np.nan, np.float32), [M, F])
    engine.qlinear(ctx, xt, ql, y)
    got = y.to_vec(ctx).reshape(M, F)
    assert np.isfinite(got).all()
    assert rel_err(got, _reference(oracle, x, gq, gs, uq, us)) <= TOL_FP32


def test_fused_pairs_equal_the_unfused_operators_on_the_device(ctx, engine):
    """The same numbers as Linear, silu, mul run one after the other through the C ABI (f32 everywhere)."""
    M, K, F = 32, 2048, 640
    x, gq, gs, uq, us = _pairs_case(3, M, K, F)
    xt = UnifiedTensor.new(ctx, x, [M, K])
    fused = UnifiedTensor.empty(ctx, [M, F])
    engine.qlinear(ctx, xt, QLinear.from_gate_up(ctx, gq, gs, uq, us), fused)
    g, u, act, out = (UnifiedTensor.empty(ctx, [M, F]) for _ in range(4))
    engine.qlinear(ctx, xt, QLinear.from_host(ctx, gq, gs), g)
    engine.qlinear(ctx, xt, QLinear.from_host(ctx, uq, us), u)
    engine.silu(ctx, g, act)
    engine.mul(ctx, act, u, out)
    assert rel_err(fused.to_vec(ctx), out.to_vec(ctx)) <= 2e-6


def test_bf16_in_and_out(ctx, engine, oracle):
    M, K, F = 48, 1024, 256
    x, gq, gs, uq, us = _pairs_case(11, M, K, F)
    from rusty_b200.backend import bf16_bits_to_f32, f32_to_bf16_bits
    xr = bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(M, K)
    ql = QLinear.from_gate_up(ctx, gq, gs, uq, us)
    xt = UnifiedTensor.from_bf16(ctx, x, [M, K])
    y = UnifiedTensor.empty_with_dtype(ctx, [M, F], DType.BF16)
    engine.qlinear(ctx, xt, ql, y)
    assert rel_err(y.to_vec(ctx).reshape(M, F), _reference(oracle, xr, gq, gs, uq, us)) <= TOL_BF16


@pytest.mark.parametrize("M,K,F,ydt", [(128, 1024, 256, DType.BF16), (200, 4096, 192, DType.BF16), (512, 2048, 1000, DType.FP32),
                                       (65, 512, 64, DType.BF16), (2048, 1024, 7168, DType.BF16)])
def test_prefill_pairs_on_the_bf16_tensor_core_kernel(ctx, engine, oracle, M, K, F, ydt):
    """M >= 65 with bf16 activations: the bf16 MMA kernel applies silu(gate) * up in its epilogue (whole tiles and
    tiles cut along K alike)."""
    from canary import GuardedOutput
    from parity import rel_err_rows
    from rusty_b200.backend import bf16_bits_to_f32, f32_to_bf16_bits
    x, gq, gs, uq, us = _pairs_case(M + F, M, K, F)
    xr = bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(M, K)
    ql = QLinear.from_gate_up(ctx, gq, gs, uq, us)
    assert ql.plan(M, DType.BF16, ydt) == "tcgen05_f16"
    xt = UnifiedTensor.from_bf16(ctx, x, [M, K])
    g = GuardedOutput(ctx, [M, F], ydt)
    engine.qlinear(ctx, xt, ql, g.tensor)
    got = g.read()
    assert np.isfinite(got).all()
    # sampled rows at the large shape keep the oracle's share of the run short
    rows = np.arange(M) if M * F * K <= 2 ** 31 else np.unique(np.concatenate([np.arange(0, M, 37), [M - 1]]))
    want = _reference(oracle, xr[rows], gq, gs, uq, us)
    assert rel_err_rows(got[rows], want) <= (TOL_BF16 if ydt == DType.BF16 else 1e-4)


def test_shards_of_pairs_give_the_columns_of_the_whole(ctx, engine):
    M, K, F = 32, 1024, 512
    x, gq, gs, uq, us = _pairs_case(5, M, K, F)
    q, s = interleave_pairs(gq, uq), interleave_pairs(gs, us)
    xt = UnifiedTensor.new(ctx, x, [M, K])
    whole = UnifiedTensor.empty(ctx, [M, F])
    engine.qlinear(ctx, xt, QLinear.from_host(ctx, q, s).set_activation(capi.ACT_SWIGLU_PAIRS), whole)
    want = whole.to_vec(ctx).reshape(M, F)
    cols = []
    for r in range(4):
        rows = slice(r * 2 * F // 4, (r + 1) * 2 * F // 4)
        y = UnifiedTensor.empty(ctx, [M, F // 4])
        engine.qlinear(ctx, xt, QLinear.from_host(ctx, q[rows], s[rows]).set_activation(capi.ACT_SWIGLU_PAIRS), y)
        cols.append(y.to_vec(ctx).reshape(M, F // 4))
    assert np.array_equal(np.concatenate(cols, axis=1).view(np.uint32), want.view(np.uint32))


def test_pairs_are_refused_where_they_make_no_sense(ctx):
    rng = np.random.default_rng(1)
    odd = QLinear.from_host(ctx, rng.integers(-127, 128, size=(7, 64), dtype=np.int8), np.ones(7, np.float32))
    with pytest.raises(BackendError) as e:
        odd.set_activation(capi.ACT_SWIGLU_PAIRS)
    assert e.value.kind == "InvalidDimensions"
    kn = QLinear.from_host(ctx, rng.integers(-127, 128, size=(64, 32), dtype=np.int8), np.ones(32, np.float32), layout=capi.LAYOUT_KN)
    with pytest.raises(BackendError) as e:
        kn.set_activation(capi.ACT_SWIGLU_PAIRS)
    assert e.value.kind == "UnsupportedOperation"
