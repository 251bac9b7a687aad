"""The steps in front of a layer's Linears: Embedding gather (rusty-graph/src/lib.rs:121-135), RMSNorm with and
without the residual add (rusty-backend/src/kernels.wgsl:81-102, :570-597) and the Linear that applies the norm in its
own activation pre-pass, against the oracle's restatement of the shaders.

Tolerances.  The gather and the residual sum are exact (bit for bit).  The norm's sum of squares is a tree sum on
the device and a sequential sum in the shader/oracle: both are within sqrt(K) * 2^-24 of the exact mean, so the
outputs agree to 1e-5 of the row's largest value (TOL_FP32, the tolerance the benchmark specification states for f32)
and to 1e-6 with the formula evaluated in float64."""
import numpy as np
import pytest

from canary import GuardedOutput
from parity import TOL_BF16, TOL_FP32, assert_bits_equal, rel_err_rows
from rusty_b200 import BackendError, DType, QLinear, UnifiedTensor
from rusty_b200.backend import Graph, bf16_bits_to_f32

pytestmark = pytest.mark.gpu


def _norm_f64(v, w, eps=1e-5):
    v = v.astype(np.float64)
    return v / np.sqrt((v * v).mean(-1, keepdims=True) + eps) * w.astype(np.float64)


def _rows(seed, M, K, outlier=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if outlier:
        x[::2, K // 3] *= 300.0          # one huge activation in every other row
        x[1::3] *= 1e-3                  # and some very quiet rows
    r = (rng.standard_normal((M, K)) * 0.5).astype(np.float32)
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    return x, r, w


@pytest.mark.parametrize("M,K", [(1, 4096), (32, 4096), (7, 8192), (3, 28672), (64, 4), (5, 1000), (130, 256)])
@pytest.mark.parametrize("residual", [False, True])
def test_rms_norm_rows_match_the_shader(ctx, engine, oracle, M, K, residual):
    x, r, w = _rows(M * 31 + K, M, K, outlier=True)
    tx, tr, tw = UnifiedTensor.new(ctx, x, [M, K]), UnifiedTensor.new(ctx, r, [M, K]), UnifiedTensor.new(ctx, w, [K])
    out = UnifiedTensor.new(ctx, np.full(M * K, np.nan, np.float32), [M, K])
    if residual:
        sm = UnifiedTensor.new(ctx, np.full(M * K, np.nan, np.float32), [M, K])
        engine.rms_norm_residual(ctx, tx, tr, tw, out, sum_out=sm)
        want, want_sum = oracle.rms_norm(x, w, residual=r, return_sum=True)
        assert_bits_equal(sm.to_vec(ctx).reshape(M, K), want_sum)
        exact = _norm_f64(x + r, w)
        # the same call without a buffer for the sum
        out2 = UnifiedTensor.new(ctx, np.full(M * K, np.nan, np.float32), [M, K])
        engine.rms_norm_residual(ctx, tx, tr, tw, out2)
        assert_bits_equal(out2.to_vec(ctx), out.to_vec(ctx))
    else:
        engine.rms_norm(ctx, tx, tw, out)
        want = oracle.rms_norm(x, w)
        exact = _norm_f64(x, w)
    got = out.to_vec(ctx).reshape(M, K)
    assert np.isfinite(got).all()
    assert rel_err_rows(got, want) <= TOL_FP32
    assert rel_err_rows(got, exact) <= 1e-6


def test_rms_norm_argument_errors(ctx, engine):
    x = UnifiedTensor.zeros(ctx, [2, 8])
    w = UnifiedTensor.zeros(ctx, [8])
    small = UnifiedTensor.zeros(ctx, [8])
    with pytest.raises(BackendError) as e:
        engine.rms_norm(ctx, x, w, small)
    assert e.value.kind == "InvalidDimensions"
    with pytest.raises(BackendError) as e:
        engine.rms_norm(ctx, x, w, x)
    assert e.value.kind == "InvalidOperation"
    x6 = UnifiedTensor.zeros(ctx, [2, 6])
    with pytest.raises(BackendError) as e:
        engine.rms_norm(ctx, x6, UnifiedTensor.zeros(ctx, [6]), UnifiedTensor.zeros(ctx, [2, 6]))
    assert e.value.kind == "InvalidDimensions"


@pytest.mark.parametrize("vocab,dim,n", [(1000, 64, 1), (32000, 4096, 32), (128256, 4096, 7), (50, 8, 300)])
def test_embedding_gathers_rows_bit_for_bit(ctx, engine, oracle, vocab, dim, n):
    rng = np.random.default_rng(vocab + n)
    table = rng.standard_normal((vocab, dim)).astype(np.float32)
    ids = rng.integers(0, vocab, size=n).astype(np.uint32)
    ids[0], ids[-1] = vocab - 1, 0
    tt = UnifiedTensor.new(ctx, table, [vocab, dim])
    ti = UnifiedTensor.from_bytes_with_dtype(ctx, ids, [n * 4], DType.U8)
    g = GuardedOutput(ctx, [n, dim])
    engine.embedding(ctx, tt, ti, g.tensor)
    got = g.read()
    want, bad = oracle.embedding(table, ids)
    assert bad == 0
    assert_bits_equal(got, want)


def test_embedding_id_outside_the_table_is_reported_and_zeroed(ctx, engine, oracle):
    vocab, dim = 100, 16
    table = np.arange(vocab * dim, dtype=np.float32).reshape(vocab, dim) + 1.0
    ids = np.array([3, 100, 7, 4000000000], np.uint32)
    tt = UnifiedTensor.new(ctx, table, [vocab, dim])
    ti = UnifiedTensor.from_bytes_with_dtype(ctx, ids, [16], DType.U8)
    out = UnifiedTensor.new(ctx, np.full(4 * dim, np.nan, np.float32), [4, dim])
    engine.embedding(ctx, tt, ti, out)
    with pytest.raises(BackendError) as e:
        ctx.sync()
    assert e.value.kind == "InvalidOperation" and "outside the table" in str(e.value)
    ctx.sync()                                   # reported once; the context keeps working
    want, bad = oracle.embedding(table, ids)
    assert bad == 2
    assert_bits_equal(out.to_vec(ctx).reshape(4, dim), want)


def _linear_case(seed, M, K, N):
    rng = np.random.default_rng(seed)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    return q, s


# fused in the pre-pass: 3 <= M, the row fits the registers of its threads; the others run the norm kernel first
@pytest.mark.parametrize("M,K,N,fused", [(32, 4096, 1024, True), (64, 8192, 512, True), (8, 14336, 256, True),
                                         (5, 1024, 136, True), (100, 512, 192, True), (3, 16, 64, True),
                                         (1, 4096, 512, False), (2, 1024, 96, False), (64, 11008, 128, False),
                                         (16, 28672, 64, False)])
@pytest.mark.parametrize("residual", [False, True])
def test_normed_linear_matches_norm_then_linear(ctx, engine, oracle, M, K, N, fused, residual):
    x, r, w = _rows(M + K + N, M, K, outlier=True)
    q, s = _linear_case(N * 3 + K, M, K, N)
    ql = QLinear.from_host(ctx, q, s)
    assert (ql.plan(M) == "tcgen05") == (M >= 3)
    tx, tr, tw = UnifiedTensor.new(ctx, x, [M, K]), UnifiedTensor.new(ctx, r, [M, K]), UnifiedTensor.new(ctx, w, [K])
    normed = UnifiedTensor.new(ctx, np.full(M * K, np.nan, np.float32), [M, K])
    sm = UnifiedTensor.new(ctx, np.full(M * K, np.nan, np.float32), [M, K]) if residual else None
    g = GuardedOutput(ctx, [M, N])
    launches = ctx.launch_count()
    engine.qlinear_normed(ctx, tx, tw, ql, g.tensor, residual=tr if residual else None, normed_out=normed, sum_out=sm)
    launches = ctx.launch_count() - launches
    y = g.read()
    passes = (M + 63) // 64
    assert launches == (2 * passes if fused else (3 if M >= 3 else 2)), launches   # no norm kernel when fused
    if residual:
        want_n, want_sum = oracle.rms_norm(x, w, residual=r, return_sum=True)
        assert_bits_equal(sm.to_vec(ctx).reshape(M, K), want_sum)
    else:
        want_n = oracle.rms_norm(x, w)
    got_n = normed.to_vec(ctx).reshape(M, K)
    assert np.isfinite(y).all() and np.isfinite(got_n).all()
    assert rel_err_rows(got_n, want_n) <= TOL_FP32
    # the Linear itself is exact on the activations the kernel normalised ...
    assert rel_err_rows(y, oracle.qlinear_rowscale(got_n, q, s)) <= TOL_FP32
    # ... and the whole composition stays within the norm's own tolerance of the shader chain
    assert rel_err_rows(y, oracle.qlinear_rowscale(want_n, q, s)) <= 2 * TOL_FP32
    # without the optional outputs: the same y, bit for bit
    y2 = UnifiedTensor.new(ctx, np.full(M * N, np.nan, np.float32), [M, N])
    engine.qlinear_normed(ctx, tx, tw, ql, y2, residual=tr if residual else None)
    assert_bits_equal(y2.to_vec(ctx).reshape(M, N), y)


def test_normed_linear_into_pairs_and_bf16_and_a_graph(ctx, engine, oracle):
    """norm2 -> gate|up with the SwiGLU epilogue, a bf16 output, and the fused call inside a captured graph."""
    from rusty_b200.backend import interleave_pairs
    M, K, F = 32, 4096, 512
    x, r, w = _rows(5, M, K)
    rng = np.random.default_rng(6)
    gq, uq = (rng.integers(-127, 128, size=(F, K), dtype=np.int8) for _ in range(2))
    gs = rng.uniform(0.0005, 0.002, size=F).astype(np.float32)
    us = rng.uniform(0.001, 0.02, size=F).astype(np.float32)
    ql = QLinear.from_gate_up(ctx, gq, gs, uq, us)
    tx, tr, tw = UnifiedTensor.new(ctx, x, [M, K]), UnifiedTensor.new(ctx, r, [M, K]), UnifiedTensor.new(ctx, w, [K])
    y = UnifiedTensor.new(ctx, np.full(M * F, np.nan, np.float32), [M, F])
    g = Graph(ctx)
    with g:
        engine.qlinear_normed(ctx, tx, tw, ql, y, residual=tr)
    g.launch()
    g.launch()
    xn = oracle.rms_norm(x, w, residual=r)
    want = oracle.mul(oracle.silu(oracle.qlinear_rowscale(xn, gq, gs)), oracle.qlinear_rowscale(xn, uq, us))
    assert rel_err_rows(y.to_vec(ctx).reshape(M, F), want) <= 2 * TOL_FP32
    # bf16 output of a plain Linear
    q, s = _linear_case(9, M, K, 256)
    ql2 = QLinear.from_host(ctx, q, s)
    yb = UnifiedTensor.empty_with_dtype(ctx, [M, 256], DType.BF16)
    engine.qlinear_normed(ctx, tx, tw, ql2, yb)
    got = bf16_bits_to_f32(yb.to_bytes(ctx).view(np.uint16)).reshape(M, 256)
    assert rel_err_rows(got, oracle.qlinear_rowscale(oracle.rms_norm(x, w), q, s)) <= TOL_BF16


# ---- residual add in the Linear's epilogue (x = x + o_proj(...), x = x + down_proj(...)) ----
@pytest.mark.parametrize("M,K,N", [(1, 1024, 256), (2, 4096, 512), (4, 512, 200), (32, 4096, 4096), (64, 2048, 1000), (100, 512, 192)])
@pytest.mark.parametrize("in_place", [False, True])
def test_residual_epilogue_equals_linear_then_add_bit_for_bit(ctx, engine, oracle, M, K, N, in_place):
    rng = np.random.default_rng(M + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    q, s = _linear_case(K + N, M, K, N)
    res = (rng.standard_normal((M, N)) * 3).astype(np.float32)
    ql = QLinear.from_host(ctx, q, s)
    tx = UnifiedTensor.new(ctx, x, [M, K])
    lin = UnifiedTensor.empty(ctx, [M, N])
    engine.qlinear(ctx, tx, ql, lin)
    tr = UnifiedTensor.new(ctx, res, [M, N])
    want = UnifiedTensor.empty(ctx, [M, N])
    engine.add(ctx, lin, tr, want)
    if in_place:
        engine.qlinear_residual(ctx, tx, ql, tr, tr)
        got = tr.to_vec(ctx)
    else:
        g = GuardedOutput(ctx, [M, N])
        engine.qlinear_residual(ctx, tx, ql, tr, g.tensor)
        got = g.read()
        assert_bits_equal(tr.to_vec(ctx).reshape(M, N), res)       # the residual itself is untouched
    assert_bits_equal(np.asarray(got).reshape(M, N), want.to_vec(ctx).reshape(M, N))
    assert rel_err_rows(np.asarray(got).reshape(M, N), res + oracle.qlinear_rowscale(x, q, s)) <= TOL_FP32


def test_residual_epilogue_of_the_bf16_prefill_kernel(ctx, engine, oracle):
    from rusty_b200.backend import f32_to_bf16_bits
    M, K, N = 300, 1024, 640
    rng = np.random.default_rng(3)
    x = rng.standard_normal((M, K)).astype(np.float32)
    q, s = _linear_case(4, M, K, N)
    res = (rng.standard_normal((M, N)) * 3).astype(np.float32)
    xr = bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(M, K)
    rr = bf16_bits_to_f32(f32_to_bf16_bits(res)).reshape(M, N)
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    tx = UnifiedTensor.from_bf16(ctx, x, [M, K])
    tr = UnifiedTensor.from_bf16(ctx, res, [M, N])
    g = GuardedOutput(ctx, [M, N], DType.BF16)
    engine.qlinear_residual(ctx, tx, ql, tr, g.tensor)
    assert rel_err_rows(g.read(), rr + oracle.qlinear_rowscale(xr, q, s)) <= TOL_BF16
    with pytest.raises(BackendError) as e:                         # not together with the pair activation
        from rusty_b200 import capi
        engine.qlinear_residual(ctx, tx, QLinear.from_host(ctx, q, s).set_activation(capi.ACT_SWIGLU_PAIRS), tr, g.tensor)
    assert e.value.kind == "InvalidOperation"
