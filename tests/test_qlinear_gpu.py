"""GPU parity of the fused int8 linear against the reference's own
dequantise-then-matmul composition (the oracle), through the C ABI."""
import numpy as np
import pytest

from canary import GuardedOutput
from parity import TOL_BF16, TOL_FP32, assert_bits_equal, rel_err, rel_err_rows
from rusty_b200 import BackendError, ComputeEngine, DType, Linear, LoRAAdapter, QLinear, UnifiedTensor
from rusty_b200 import capi
from rusty_b200.backend import bf16_bits_to_f32, f32_to_bf16_bits
from rusty_b200.workloads import affine_g64_from_sym, sym_row_linear

pytestmark = pytest.mark.gpu


def _forward(ctx, engine, ql, x, x_dtype=DType.FP32, y_dtype=DType.FP32):
    M = x.shape[0]
    xt = UnifiedTensor.from_bf16(ctx, x, list(x.shape)) if x_dtype == DType.BF16 else UnifiedTensor.new(ctx, x, list(x.shape))
    y = GuardedOutput(ctx, [M, ql.N], y_dtype)   # NaN-prefilled payload + canary pad behind it
    engine.qlinear(ctx, xt, ql, y.tensor)
    return y.read()


def _oracle_band(oracle, x, wf, y_ref):
    """How far the reference arithmetic itself sits from the exact sums."""
    return rel_err(y_ref, oracle.matmul_bt_f64(x, wf))


def test_golden_small_all_modes(ctx, engine, kat):
    x, q, s = kat["ql_x"], kat["ql_q"], kat["ql_s"]
    got = _forward(ctx, engine, QLinear.from_host(ctx, q, s), x)
    assert rel_err(got, kat["ql_y_nk"]) <= TOL_FP32
    got = _forward(ctx, engine, QLinear.from_host(ctx, np.ascontiguousarray(q.T), s, layout=capi.LAYOUT_KN), x)
    assert rel_err(got, kat["ql_y_kn"]) <= TOL_FP32
    x2 = kat["qa_x"]
    got = _forward(ctx, engine, QLinear.from_host(ctx, kat["qa_u"], kat["qa_s"], kat["qa_b"]), x2)
    assert rel_err(got, kat["qa_y_nk"]) <= TOL_FP32
    got = _forward(ctx, engine, QLinear.from_host(ctx, kat["qa_ukn"], kat["qa_s"], kat["qa_b"], layout=capi.LAYOUT_KN), x2)
    assert rel_err(got, kat["qa_y_kn"]) <= TOL_FP32


def test_config1_gemv_sym_row(ctx, engine, oracle):
    """x f32 [1,4096] . int8 W[4096,4096], per-row scales, seed 0."""
    x, q, s = sym_row_linear(0, 1, 4096, 4096)
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(1) in ("gemv", "gemv_mma")
    got = _forward(ctx, engine, ql, x)
    wf = oracle.dequantize_rowscale(q, s)
    ref = oracle.matmul_bt(x, wf)
    assert rel_err(got, ref) <= TOL_FP32
    # no farther from the exact sums than the reference's own arithmetic is
    assert rel_err(got, oracle.matmul_bt_f64(x, wf)) <= max(_oracle_band(oracle, x, wf, ref), 1e-6) * 1.5


def test_config1_gemv_affine_native_layout(ctx, engine, oracle):
    x, q, _ = sym_row_linear(0, 1, 4096, 4096)
    u, s, b = affine_g64_from_sym(q, 0)
    got = _forward(ctx, engine, QLinear.from_host(ctx, u, s, b), x)
    ref = oracle.qlinear_affine(x, u, s, b, u.shape)
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("K,N", [(4096, 11008), (11008, 4096), (1024, 130), (80, 17), (14336, 512)])
def test_gemv_shapes_sym(ctx, engine, oracle, M, K, N):
    x, q, s = sym_row_linear(K + N + M, M, K, N)
    got = _forward(ctx, engine, QLinear.from_host(ctx, q, s), x)
    ref = oracle.matmul_bt(x, oracle.dequantize_rowscale(q, s), mt=True)
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("M,K,N", [(1, 4096, 1024), (3, 11008, 256), (4, 192, 19)])
def test_gemv_shapes_affine(ctx, engine, oracle, M, K, N):
    x, q, _ = sym_row_linear(K + N + M, M, K, N)
    u, s, b = affine_g64_from_sym(q, K)
    got = _forward(ctx, engine, QLinear.from_host(ctx, u, s, b), x)
    ref = oracle.matmul_bt(x, oracle.affine_dequantize(u, s, b, mt=True).reshape(N, K), mt=True)
    assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (2, 1000, 320), (3, 11008, 4096), (32, 4096, 1024), (7, 48, 40),
                                   (256, 1024, 520)])
def test_gemv_kn_layout(ctx, engine, oracle, M, K, N):
    """rusty's own Linear orientation: weight stored [in, out].  With one scale per output and K % 16 == 0 the weight is
    re-laid-out once at create and takes the same kernels as [out, in] storage (bit-identical results); otherwise the
    [in, out] CUDA-core kernel runs."""
    x, q, s = sym_row_linear(K * 3 + N, M, K, N)
    qkn = np.ascontiguousarray(q.T)
    ql_kn = QLinear.from_host(ctx, qkn, s, layout=capi.LAYOUT_KN)
    got = _forward(ctx, engine, ql_kn, x)
    if K % 16 == 0:
        ql_nk = QLinear.from_host(ctx, q, s)
        assert ql_kn.plan(M) == ql_nk.plan(M)
        assert_bits_equal(got, _forward(ctx, engine, ql_nk, x))
        if M >= 128:
            assert ql_kn.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    else:
        assert ql_kn.plan(M) == "gemv"
    ref = oracle.matmul_bt(x, oracle.dequantize_rowscale(q, s), mt=True)
    assert rel_err(got, ref) <= TOL_FP32
    if N % 64 == 0:
        rng = np.random.default_rng(K)
        ukn = (qkn.astype(np.int16) + 128).astype(np.uint8)
        sg = rng.uniform(0.001, 0.02, size=K * N // 64).astype(np.float32)
        bg = rng.uniform(-1, 1, size=K * N // 64).astype(np.float32)
        got = _forward(ctx, engine, QLinear.from_host(ctx, ukn, sg, bg, layout=capi.LAYOUT_KN), x)
        wkn = oracle.affine_dequantize(ukn, sg, bg, mt=True).reshape(K, N)
        ref = oracle.matmul_bt(x, np.ascontiguousarray(wkn.T), mt=True)
        assert rel_err(got, ref) <= TOL_FP32


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (2, 128, 64), (1, 1152, 192), (2, 11008, 4096), (5, 4096, 11008), (1, 8192, 64),
                                   (2, 6144, 128)])
def test_affine_g64_in_rustys_own_layout_takes_the_tensor_core_gemv(ctx, engine, oracle, M, K, N):
    """The reference's own quantised format ([in,out] bytes, one (scale, bias) per 64 consecutive output features of an
    input row, rusty-loader/src/lib.rs:155-218) with K % 128 == 0: re-laid-out once at create, then the int8 tensor-core
    GEMV with the group's scales folded into the activations.  Against the reference's arithmetic (dequantise, then the
    f32 matmul) and against the exact sums."""
    x, q, _ = sym_row_linear(K + 5 * N + M, M, K, N)
    x[0, ::97] *= 40.0   # a heavy tail inside every K slice
    rng = np.random.default_rng(K + N)
    ukn = (np.ascontiguousarray(q.T).astype(np.int16) + 128).astype(np.uint8)
    sg = rng.uniform(0.001, 0.02, size=K * N // 64).astype(np.float32)
    bg = (-128.0 * sg + rng.uniform(-0.05, 0.05, size=sg.size)).astype(np.float32)
    ql = QLinear.from_host(ctx, ukn, sg, bg, layout=capi.LAYOUT_KN)
    assert ql.plan(M) == "gemv_mma"
    got = _forward(ctx, engine, ql, x)
    wkn = oracle.affine_dequantize(ukn, sg, bg, mt=True).reshape(K, N)
    wf = np.ascontiguousarray(wkn.T)
    ref = oracle.matmul_bt(x, wf, mt=True)
    assert rel_err(got, ref) <= TOL_FP32
    assert rel_err(got, oracle.matmul_bt_f64(x, wf)) <= max(_oracle_band(oracle, x, wf, ref), 1e-6) * 1.5
    # bf16 activations are consumed exactly; a bf16 y is the f32 result rounded once
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    got_b = _forward(ctx, engine, ql, x, x_dtype=DType.BF16)
    assert rel_err(got_b, oracle.matmul_bt(xb, wf, mt=True)) <= TOL_FP32
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    assert np.array_equal(f32_to_bf16_bits(got16), f32_to_bf16_bits(got_b))
    # the same answer on every run, and rows of a batch do not depend on their neighbours
    assert_bits_equal(got, _forward(ctx, engine, ql, x))
    if M > 1:
        assert_bits_equal(got[M - 1:], _forward(ctx, engine, ql, x[M - 1:]))


def test_bf16_activations_and_outputs(ctx, engine, oracle):
    """bf16 x is consumed exactly (the oracle sees the rounded values); a bf16 y
    is the f32 result rounded once."""
    x, q, s = sym_row_linear(21, 2, 4096, 1024)
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    ql = QLinear.from_host(ctx, q, s)
    ref = oracle.matmul_bt(xb, oracle.dequantize_rowscale(q, s), mt=True)
    got = _forward(ctx, engine, ql, x, x_dtype=DType.BF16)
    assert rel_err(got, ref) <= TOL_FP32
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    assert rel_err(got16, ref) <= TOL_BF16
    assert np.array_equal(f32_to_bf16_bits(got16), f32_to_bf16_bits(got))  # exactly one rounding of the f32 result


def test_weight_values_cover_all_256_bytes(ctx, engine, oracle):
    """Every int8 value (including -128) and every u8 value dequantises exactly:
    with x = one-hot rows the output IS the dequantised weight."""
    K, N = 256, 64
    q = np.tile(np.arange(-128, 128, dtype=np.int8), (N, 1))
    q = np.roll(q, 3, axis=1)
    s = np.ones(N, np.float32)
    for k0 in (0, 3, 131, 255):
        x = np.zeros((1, K), np.float32)
        x[0, k0] = 1.0
        got = _forward(ctx, engine, QLinear.from_host(ctx, q, s), x)
        assert np.array_equal(got[0], q[:, k0].astype(np.float32))
    u = (q.astype(np.int16) + 128).astype(np.uint8)
    sg = np.ones(N * K // 64, np.float32)
    bg = np.zeros(N * K // 64, np.float32)
    x = np.zeros((1, K), np.float32)
    x[0, 7] = 1.0
    got = _forward(ctx, engine, QLinear.from_host(ctx, u, sg, bg), x)
    assert np.array_equal(got[0], u[:, 7].astype(np.float32))


def test_linearity_and_row_independence(ctx, engine):
    """Size-independent properties at a full-size shape: f(a+b) = f(a)+f(b) within
    rounding, and each activation row's result does not depend on its neighbours."""
    x, q, s = sym_row_linear(33, 4, 4096, 14336)
    ql = QLinear.from_host(ctx, q, s)
    y = _forward(ctx, engine, ql, x)
    y2 = _forward(ctx, engine, ql, x[:2])
    y0 = _forward(ctx, engine, ql, x[:1])
    assert_bits_equal(y2[:1], y0)                 # same kernel, one row more: identical bits for the shared row
    assert rel_err(y[:2], y2) <= TOL_FP32          # four rows run on another kernel: equal within tolerance
    ysum = _forward(ctx, engine, ql, (x[0:1] + x[1:2]))
    assert rel_err(ysum, y[0:1] + y[1:2]) <= TOL_FP32


def test_linear_api_quantized_and_lora(ctx, engine, oracle):
    """Linear.forward keeps the reference contract: x . W[in,out] (+ (x.A).B)."""
    rng = np.random.default_rng(5)
    K, N, M = 256, 192, 3
    w = rng.standard_normal((K, N)).astype(np.float32)
    x = rng.standard_normal((2, M, K)).astype(np.float32)            # leading dims are flattened
    lin = Linear.new(ctx, UnifiedTensor.new(ctx, w, [K, N]))
    xt = UnifiedTensor.new(ctx, x, list(x.shape))
    y = lin.forward(engine, xt)
    assert y.shape == [2, M, N]
    ref = oracle.matmul_tiled(x.reshape(-1, K), w)
    assert rel_err(y.to_vec(ctx).reshape(-1, N), ref) <= TOL_FP32
    # LoRA branch: A = 0.01, B = 0 at construction (no change), then a non-zero B
    lora = LoRAAdapter(ctx, K, N, rank=4, alpha=16.0)
    y2 = Linear.with_lora(ctx, lin.weight, lora).forward(engine, xt)
    assert_bits_equal(y2.to_vec(ctx), y.to_vec(ctx))
    bmat = rng.standard_normal((4, N)).astype(np.float32)
    lora.b.write_data(ctx, bmat)
    y3 = Linear.with_lora(ctx, lin.weight, lora).forward(engine, xt)
    a = np.full((K, 4), 0.01, np.float32)
    ref3 = ref + oracle.matmul_tiled(oracle.matmul_tiled(x.reshape(-1, K), a), bmat)
    assert rel_err(y3.to_vec(ctx).reshape(-1, N), ref3) <= TOL_FP32
    # the same Linear over a quantised weight
    _, q, s = sym_row_linear(9, 1, K, N)
    qlin = Linear.from_quantized(ctx, QLinear.from_host(ctx, q, s))
    yq = qlin.forward(engine, xt)
    refq = oracle.matmul_bt(x.reshape(-1, K), oracle.dequantize_rowscale(q, s))
    assert yq.shape == [2, M, N] and rel_err(yq.to_vec(ctx).reshape(-1, N), refq) <= TOL_FP32


def test_empty_and_invalid(ctx, engine):
    _, q, s = sym_row_linear(1, 1, 64, 16)
    ql = QLinear.from_host(ctx, q, s)
    x0 = UnifiedTensor.empty(ctx, [0, 64])
    y0 = UnifiedTensor.empty(ctx, [0, 16])
    engine.qlinear(ctx, x0, ql, y0)  # M = 0: nothing to do, no error
    x = UnifiedTensor.new(ctx, np.zeros((2, 64), np.float32), [2, 64])
    with pytest.raises(BackendError) as e:
        engine.qlinear(ctx, x, ql, UnifiedTensor.empty(ctx, [1, 16]))
    assert e.value.kind == "InvalidDimensions"
    with pytest.raises(BackendError) as e:
        QLinear.from_host(ctx, np.zeros((16, 72), np.uint8), np.zeros(18, np.float32), np.zeros(18, np.float32))
    assert e.value.kind == "InvalidDimensions"   # a 64-group would straddle rows
    with pytest.raises(BackendError) as e:
        xi = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(128, np.uint8), [2, 64], DType.I8)
        engine.qlinear(ctx, xi, ql, UnifiedTensor.empty(ctx, [2, 16]))
    assert e.value.kind == "InvalidDataType"
    ctx.sync()


# ---- tensor-core (tcgen05 / TMEM) path: batches of activation rows ----

@pytest.mark.parametrize("M,K,N", [(5, 256, 128), (8, 4096, 4096), (32, 4096, 1024), (32, 4096, 14336), (17, 1024, 130),
                                   (64, 8192, 1024), (32, 14336, 4096), (100, 512, 384), (6, 80, 24), (33, 4096, 128256)])
def test_tc_shapes_f32(ctx, engine, oracle, M, K, N):
    x, q, s = sym_row_linear(K + 3 * N + M, M, K, N)
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M) == "tcgen05"
    got = _forward(ctx, engine, ql, x)
    ctx.sync()  # also surfaces a device-side wait that gave up
    if N * K * M > 2e10:
        rows = [0, M // 2, M - 1]  # full-size LM head: a few activation rows against the scalar oracle
        ref = oracle.matmul_bt(x[rows], oracle.dequantize_rowscale(q, s), mt=True)
        assert rel_err(got[rows], ref) <= TOL_FP32
        assert np.isfinite(got).all()
    else:
        ref = oracle.matmul_bt(x, oracle.dequantize_rowscale(q, s), mt=True)
        assert rel_err(got, ref) <= TOL_FP32
        assert rel_err_rows(got, ref) <= TOL_FP32


@pytest.mark.parametrize("K,N", [(4096, 768), (4096, 512), (14336, 512), (4096, 3584), (4096, 16032), (4096, 1536), (4096, 7168),
                                 (14336, 1024), (4096, 1024), (4096, 32064)])
def test_tc_shard_shapes_of_the_decode_stack(ctx, engine, oracle, K, N):
    """What a rank runs when the Llama-3-8B-shaped stack is cut 4 or 8 ways (few row tiles, up to 28 pieces per tile)."""
    M = 32
    x, q, s = sym_row_linear(K + N, M, K, N)
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M) == "tcgen05"
    got = _forward(ctx, engine, ql, x)
    ctx.sync()
    assert rel_err(got, oracle.matmul_bt(x, oracle.dequantize_rowscale(q, s), mt=True)) <= TOL_FP32


@pytest.mark.parametrize("M", [8, 32, 64])
@pytest.mark.parametrize("xdt", ["f32", "bf16"])
def test_tc_heavy_tailed_activations(ctx, engine, oracle, M, xdt):
    """One element per row 1000 times the row's spread: the digit planes hang below the row MAXIMUM, so every other
    element of such a row keeps ten bits less.  f32 activations carry four planes (28 bits below the maximum) and
    must hold the fp32 tolerance row by row; bf16 activations carry three (21 bits), which the bf16 budget covers."""
    K, N = 4096, 1024
    x, q, s = sym_row_linear(4000 + M, M, K, N)
    rng = np.random.default_rng(M)
    x[np.arange(M), rng.integers(0, K, size=M)] *= 1000.0
    bf = xdt == "bf16"
    xe = bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(M, K) if bf else x
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M, DType.BF16 if bf else DType.FP32, DType.FP32) == "tcgen05"
    got = _forward(ctx, engine, ql, x, x_dtype=DType.BF16 if bf else DType.FP32)
    ref = oracle.matmul_bt(xe, oracle.dequantize_rowscale(q, s), mt=True)
    if bf:
        assert rel_err_rows(got, ref) <= 1e-4      # measured ~5e-5 at worst; the stated budget for bf16 inputs is 1e-2
    else:
        assert rel_err_rows(got, ref) <= TOL_FP32
        assert rel_err_rows(got, oracle.matmul_bt_f64(xe, oracle.dequantize_rowscale(q, s))) <= 2e-6


def _sampled_weight_rows(N, rng, n_random=384):
    """First and last 160 output features (tile edges) plus a random sample: enough to pin a full-size Linear
    against the scalar oracle in seconds."""
    edge = np.concatenate([np.arange(0, min(160, N)), np.arange(max(0, N - 160), N)])
    return np.unique(np.concatenate([edge, rng.integers(0, N, size=n_random)]))


@pytest.mark.parametrize("M,K,N,pairs", [
    (64, 8192, 10240, False),    # Llama-2-70B-shaped q|k|v, batch-64 decode
    (64, 8192, 57344, True),     # gate|up as (gate, up) pairs, silu(gate)*up in the epilogue
    (64, 28672, 8192, False),    # down
    (1, 11008, 4096, False),     # Llama-7B-shaped down, batch-1 decode
    (1, 4096, 32000, False),     # Llama-7B-shaped LM head
])
def test_full_size_shapes_of_the_70b_and_7b_stacks(ctx, engine, oracle, M, K, N, pairs):
    rng = np.random.default_rng(K + N)
    x = rng.standard_normal((M, K), dtype=np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    if pairs:
        s[0::2] = rng.uniform(0.0002, 0.001, size=N // 2).astype(np.float32)   # gates land in the curved part of silu
    ql = QLinear.from_host(ctx, q, s)
    if pairs:
        ql.set_activation(capi.ACT_SWIGLU_PAIRS)
    xt = UnifiedTensor.new(ctx, x, [M, K])
    y = GuardedOutput(ctx, [M, ql.out_features])
    engine.qlinear(ctx, xt, ql, y.tensor)
    got = y.read()
    ctx.sync()
    assert np.isfinite(got).all()
    rows = sorted({0, M // 2, M - 1})
    if pairs:
        cols = _sampled_weight_rows(N // 2, rng)
        g = oracle.qlinear_rowscale(x[rows], q[2 * cols], s[2 * cols])
        u = oracle.qlinear_rowscale(x[rows], q[2 * cols + 1], s[2 * cols + 1])
        ref = oracle.mul(oracle.silu(g), u)
    else:
        cols = _sampled_weight_rows(N, rng)
        ref = oracle.qlinear_rowscale(x[rows], q[cols], s[cols])
    assert rel_err_rows(got[np.ix_(rows, cols)], ref) <= TOL_FP32


@pytest.mark.parametrize("M,K,N", [(2048, 4096, 6144), (2048, 14336, 4096), (8192, 8192, 1024)])
def test_prefill_f16_full_size_rows(ctx, engine, oracle, M, K, N):
    """2048-token (Llama-3-8B shapes) and 4 x 2048-token (Llama-2-70B width) prefill calls, sampled outputs."""
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K), dtype=np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(M, K)
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    got = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    ctx.sync()
    assert np.isfinite(got).all()
    rows = np.unique(np.concatenate([np.arange(0, 3), np.arange(M - 3, M), rng.integers(0, M, size=26)]))
    cols = _sampled_weight_rows(N, rng, 192)
    ref = oracle.qlinear_rowscale(xb[rows], q[cols], s[cols])
    assert rel_err_rows(got[np.ix_(rows, cols)], ref) <= TOL_BF16


def test_tc_is_closer_to_exact_than_the_reference_arithmetic(ctx, engine, oracle):
    """Integer tensor-core sums are exact; the result sits nearer the float64
    dot products than the reference's own sequential f32 accumulation does."""
    x, q, s = sym_row_linear(77, 16, 4096, 2048)
    wf = oracle.dequantize_rowscale(q, s)
    got = _forward(ctx, engine, QLinear.from_host(ctx, q, s), x)
    exact = oracle.matmul_bt_f64(x, wf)
    ref = oracle.matmul_bt(x, wf, mt=True)
    assert rel_err(got, exact) <= 2e-7
    assert rel_err(got, exact) <= rel_err(ref, exact)


def test_tc_bf16_in_out(ctx, engine, oracle):
    x, q, s = sym_row_linear(78, 32, 4096, 4096)
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    ql = QLinear.from_host(ctx, q, s)
    ref = oracle.matmul_bt(xb, oracle.dequantize_rowscale(q, s), mt=True)
    got = _forward(ctx, engine, ql, x, x_dtype=DType.BF16)
    assert rel_err(got, ref) <= TOL_FP32
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    assert rel_err(got16, ref) <= TOL_BF16


def test_tc_split_k_is_deterministic_and_leaves_scratch_clean(ctx, engine):
    """K split over CTAs sums integers, so repeated calls give identical bits,
    and the shared scratch is zero again for the next call of another shape."""
    x, q, s = sym_row_linear(79, 32, 4096, 1024)   # 8 row tiles -> every tile is cut over several CTAs
    ql = QLinear.from_host(ctx, q, s)
    a = _forward(ctx, engine, ql, x)
    for _ in range(3):
        assert_bits_equal(_forward(ctx, engine, ql, x), a)
    x2, q2, s2 = sym_row_linear(80, 8, 2048, 512)
    ql2 = QLinear.from_host(ctx, q2, s2)
    b = _forward(ctx, engine, ql2, x2)
    assert_bits_equal(_forward(ctx, engine, ql, x), a)
    assert_bits_equal(_forward(ctx, engine, ql2, x2), b)


def test_tc_rows_do_not_interact(ctx, engine):
    x, q, s = sym_row_linear(81, 32, 4096, 4096)
    x[3] *= 1000.0      # rows have their own digit scale
    x[7] = 0.0          # an all-zero row
    ql = QLinear.from_host(ctx, q, s)
    y = _forward(ctx, engine, ql, x)
    assert np.all(y[7] == 0.0)
    y24 = _forward(ctx, engine, ql, x[:24])      # same digit count as the 32-row call: identical bits
    assert_bits_equal(y[:24], y24)
    y8 = _forward(ctx, engine, ql, x[:8])        # narrower batch keeps one more digit: equal within tolerance
    assert rel_err(y8, y[:8]) <= TOL_FP32


def test_tc_nonfinite_activation_poisons_its_row_only(ctx, engine):
    x, q, s = sym_row_linear(82, 8, 1024, 256)
    x[2, 5] = np.nan
    y = _forward(ctx, engine, QLinear.from_host(ctx, q, s), x)
    assert np.isnan(y[2]).all() and np.isfinite(np.delete(y, 2, axis=0)).all()


# ---- prefill path: fp16 weights in tensor memory x bf16 activations ----

@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (300, 4096, 1000), (96, 192, 24), (2048, 4096, 512), (65, 64, 8)])
def test_prefill_affine_g64_on_the_bf16_kernel(ctx, engine, oracle, M, K, N):
    """The reference's own layout (u8, scale and bias per 64 elements) with bf16 activations at M >= 65: the converter
    warps of the tensor-core kernel apply scale and bias while converting, the product rounded to bf16 (tolerance
    1e-2, as for every path that rounds to bf16; the f32 paths keep 1e-5 on the CUDA-core kernel)."""
    x, q, _ = sym_row_linear(3 * K + N + M, M, K, N)
    rng = np.random.default_rng(K + N)
    u = (q.astype(np.int16) + 128).astype(np.uint8)
    sg = rng.uniform(0.001, 0.02, size=N * K // 64).astype(np.float32)
    bg = (np.float32(-128.0) * sg * rng.uniform(0.9, 1.1, size=N * K // 64)).astype(np.float32)   # zero point near 128, not on it
    ql = QLinear.from_host(ctx, u, sg, bg)
    assert ql.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    got32 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.FP32)
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    wf = oracle.affine_dequantize(u, sg, bg, mt=True).reshape(N, K)
    rows = slice(None) if M * N * K < 3e9 else [0, 1, M // 2, M - 1]
    ref = oracle.matmul_bt(xb[rows], wf, mt=True)
    assert np.isfinite(got32).all()
    assert rel_err_rows(got32[rows], ref) <= TOL_BF16
    assert rel_err_rows(got16[rows], ref) <= TOL_BF16
    # the weights really are rounded to bf16 and nothing else: against that model the f32 output is tight
    wb = bf16_bits_to_f32(f32_to_bf16_bits(wf)).reshape(N, K)
    assert rel_err(got32[rows], xb[rows].astype(np.float64) @ wb.astype(np.float64).T) <= 5e-4   # (fused multiply-add on the device, separate multiply and add in the oracle: a few bf16 roundings differ)
    # f32 activations keep the exact CUDA-core kernel
    assert ql.plan(M, DType.FP32, DType.FP32) == "gemv"

@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (300, 4096, 1024), (96, 128, 64), (2048, 4096, 512), (65, 1152, 192), (512, 4096, 11008)])
def test_prefill_native_affine_layout_on_the_bf16_kernel(ctx, engine, oracle, M, K, N):
    """rusty's own [in,out] storage in the reference's affine format (groups of 64 along the OUTPUT dimension), bf16
    activations, M >= 65: after the one-time re-layout the converter warps apply one (scale, bias) per element while
    converting (a warp's 32 rows lie in one group, so the 64 scales of a stage are the same addresses for every lane)."""
    x, q, _ = sym_row_linear(7 * K + N + M, M, K, N)
    rng = np.random.default_rng(K + 3 * N)
    ukn = (np.ascontiguousarray(q.T).astype(np.int16) + 128).astype(np.uint8)
    sg = rng.uniform(0.001, 0.02, size=K * N // 64).astype(np.float32)
    bg = (np.float32(-128.0) * sg * rng.uniform(0.9, 1.1, size=sg.size)).astype(np.float32)
    ql = QLinear.from_host(ctx, ukn, sg, bg, layout=capi.LAYOUT_KN)
    assert ql.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    assert ql.plan(M, DType.FP32, DType.FP32) == "gemv_mma"      # f32 activations keep the exact path
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    got32 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.FP32)
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    wf = np.ascontiguousarray(oracle.affine_dequantize(ukn, sg, bg, mt=True).reshape(K, N).T)
    rows = slice(None) if M * N * K < 3e9 else [0, 1, M // 2, M - 1]
    ref = oracle.matmul_bt(xb[rows], wf, mt=True)
    assert np.isfinite(got32).all()
    assert rel_err_rows(got32[rows], ref) <= TOL_BF16
    assert rel_err_rows(got16[rows], ref) <= TOL_BF16
    wb = bf16_bits_to_f32(f32_to_bf16_bits(wf)).reshape(N, K)
    assert rel_err(got32[rows], xb[rows].astype(np.float64) @ wb.astype(np.float64).T) <= 5e-4


@pytest.mark.parametrize("M,K,N", [(128, 512, 256), (512, 4096, 1024), (200, 1024, 130), (96, 4096, 4096), (300, 80, 24),
                                   (512, 4096, 11008)])
def test_prefill_f16_shapes(ctx, engine, oracle, M, K, N):
    x, q, s = sym_row_linear(5 * K + N + M, M, K, N)
    xb = bf16_bits_to_f32(f32_to_bf16_bits(x))
    ql = QLinear.from_host(ctx, q, s)
    assert ql.plan(M, DType.BF16, DType.BF16) == "tcgen05_f16"
    got32 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.FP32)
    got16 = _forward(ctx, engine, ql, x, x_dtype=DType.BF16, y_dtype=DType.BF16)
    ctx.sync()
    wf = oracle.dequantize_rowscale(q, s)
    rows = slice(None) if M * N * K < 3e9 else [0, 1, M // 2, M - 1]
    ref = oracle.matmul_bt(xb[rows], wf, mt=True)
    assert rel_err(got32[rows], ref) <= TOL_FP32         # products are exact, accumulation is fp32
    assert rel_err(got16[rows], ref) <= TOL_BF16
    exact = xb.astype(np.float64) @ wf.astype(np.float64).T
    assert rel_err(got32, exact) <= TOL_FP32
    # a bf16 y is the f32 result rounded once; tiles cut along K add their f32 pieces in arrival order, so two
    # runs may differ in the last f32 bit and, rarely, in the bf16 rounding that follows
    assert rel_err(got16, got32) <= 2.0 ** -8      # half a bf16 ulp of the largest value, plus the f32 wobble
    assert np.mean(f32_to_bf16_bits(got16) != f32_to_bf16_bits(got32)) < 1e-3
