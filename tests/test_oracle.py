"""CPU tests of the oracle itself: hand-derived literals, the committed golden
vectors, the numpy mirror, and the documented divergence from the reference's
dispatch.  No GPU."""
import hashlib

import numpy as np

from parity import assert_bits_equal, rel_err
from rusty_b200.workloads import affine_g64_from_sym, sym_row_linear


def test_ops_test_identity_product(oracle, kat):
    # rusty-backend/examples/ops_test.rs:9-17 — the only matmul anchor in the reference
    a = np.array([[1, 2], [3, 4]], np.float32)
    out = oracle.matmul_tiled(a, np.eye(2, dtype=np.float32))
    assert out.ravel().tolist() == [1.0, 2.0, 3.0, 4.0]
    assert_bits_equal(out, kat["ops_out"])


def test_dequantize_lane_order_is_lsb_first(oracle):
    word = np.array([0x04030201], "<u4")
    assert oracle.dequantize(word.view(np.uint8)).tolist() == [1.0, 2.0, 3.0, 4.0]


def test_dequantize_is_unsigned_without_scale(oracle):
    raw = np.array([0, 127, 128, 255], np.uint8)
    assert oracle.dequantize(raw).tolist() == [0.0, 127.0, 128.0, 255.0]


def test_dequantize_ragged_lengths(oracle, kat):
    raw = kat["deq_in"]
    assert_bits_equal(oracle.dequantize(raw), kat["deq_out"])
    # 7 logical bytes, 7 outputs: the 8th store is guarded away
    o7 = oracle.dequantize(raw[:8], n_in=7, n_out=7)
    assert o7.tolist() == [1, 2, 3, 4, 0, 127, 128]
    # input buffer shorter than the dispatch: outputs past the last word are untouched
    o = oracle.dequantize(raw[:8], n_in=12, n_out=12, out_init=np.full(12, -1.0, np.float32))
    assert o[:8].tolist() == [1, 2, 3, 4, 0, 127, 128, 255] and o[8:].tolist() == [-1, -1, -1, -1]


def test_dequantize_matches_numpy_mirror(oracle, kat):
    big = kat["deq_big_in"]
    assert_bits_equal(oracle.dequantize(big), oracle.np_dequantize(big))
    assert_bits_equal(oracle.dequantize(big), kat["deq_big_out"])


def test_affine_group_boundary(oracle):
    u = np.arange(128, dtype=np.uint8)
    s = np.array([0.5, 2.0], np.float32)
    b = np.array([1.0, -3.0], np.float32)
    out = oracle.affine_dequantize(u, s, b)
    assert out[63] == 63 * 0.5 + 1.0 and out[64] == 64 * 2.0 - 3.0
    assert out[0] == 1.0 and out[127] == 127 * 2.0 - 3.0


def test_affine_matches_golden_and_mirror(oracle, kat):
    out = oracle.affine_dequantize(kat["aff_u"], kat["aff_s"], kat["aff_b"])
    assert_bits_equal(out, kat["aff_out"])
    assert_bits_equal(out, oracle.np_affine_dequantize(kat["aff_u"], kat["aff_s"], kat["aff_b"]))
    assert_bits_equal(oracle.affine_dequantize(kat["aff_u"], kat["aff_s"], kat["aff_b"], fma=True), kat["aff_out_fma"])


def test_affine_as_dispatched_truncates_at_4194240(oracle):
    """Documents the reference defect: a 2-D dispatch indexed by x alone never
    writes element 65535*64 and beyond (lib.rs:4976-4987, kernels.wgsl:387)."""
    n = 65535 * 64 + 128
    u = np.full(n, 3, np.uint8)
    s = np.full(n // 64 + 1, 2.0, np.float32)
    b = np.full(n // 64 + 1, 1.0, np.float32)
    init = np.full(n, -9.0, np.float32)
    got = oracle.affine_dequantize(u, s, b, as_dispatched=True, out_init=init)
    assert got[65535 * 64 - 1] == 7.0 and np.all(got[65535 * 64:] == -9.0)
    full = oracle.affine_dequantize(u, s, b)
    assert np.all(full == 7.0)


def test_matmul_tails_match_golden_and_mirror(oracle, kat):
    for i in range(int(kat["mm_count"])):
        a, b = kat[f"mm{i}_a"], kat[f"mm{i}_b"]
        out = oracle.matmul_tiled(a, b)
        assert_bits_equal(out, kat[f"mm{i}_out"])
        assert_bits_equal(out, oracle.np_matmul_seq(a, b))
        assert_bits_equal(oracle.matmul_bt(a, np.ascontiguousarray(b.T)), out)  # same sum, other storage order
        assert_bits_equal(oracle.matmul_tiled(a, b, fma=True), kat[f"mm{i}_out_fma"])


def test_threaded_variants_are_bit_identical(oracle):
    x, q, s = sym_row_linear(3, 2, 256, 96)
    wf = oracle.dequantize_rowscale(q, s)
    assert_bits_equal(oracle.matmul_bt(x, wf, mt=True), oracle.matmul_bt(x, wf))
    assert_bits_equal(oracle.qlinear_rowscale_fused_mt(x, q, s), oracle.matmul_bt(x, wf))
    assert rel_err(oracle.qlinear_rowscale_fused_mt(x, q, s, simd=True), oracle.matmul_bt(x, wf)) < 1e-5


def test_sym_row_equals_affine_restatement(oracle):
    """u8 = q+128, bias = -128*scale, scale repeated per 64-group expresses the
    symmetric mode in the reference's native layout (cross-check, not bit-exact)."""
    x, q, s = sym_row_linear(5, 2, 256, 64)
    y_sym = oracle.qlinear_rowscale(x, q, s)
    u = (q.astype(np.int16) + 128).astype(np.uint8)
    sg = np.repeat(s, 256 // 64).astype(np.float32)
    bg = (np.float32(-128.0) * sg).astype(np.float32)
    y_aff = oracle.qlinear_affine(x, u, sg, bg, u.shape)
    assert rel_err(y_aff, y_sym) < 1e-5


def test_fused_goldens(oracle, kat):
    assert_bits_equal(oracle.qlinear_rowscale(kat["ql_x"], kat["ql_q"], kat["ql_s"]), kat["ql_y_nk"])
    assert_bits_equal(oracle.qlinear_rowscale(kat["ql_x"], np.ascontiguousarray(kat["ql_q"].T), kat["ql_s"], layout_nk=False),
                      kat["ql_y_kn"])
    assert_bits_equal(kat["ql_y_nk"], kat["ql_y_kn"])  # same sums in the same k order
    assert_bits_equal(oracle.qlinear_affine(kat["qa_x"], kat["qa_u"], kat["qa_s"], kat["qa_b"], kat["qa_u"].shape), kat["qa_y_nk"])
    assert_bits_equal(oracle.qlinear_affine(kat["qa_x"], kat["qa_ukn"], kat["qa_s"], kat["qa_b"], kat["qa_ukn"].shape,
                                            layout_nk=False), kat["qa_y_kn"])


def test_config1_digest(oracle, kat):
    x, q, s = sym_row_linear(0, 1, 4096, 4096)
    y = oracle.qlinear_rowscale(x, q, s)
    assert hashlib.sha256(y.tobytes()).digest() == kat["cfg1_y_sha256"].tobytes()
    assert_bits_equal(y[0, :16], kat["cfg1_y_head"])
    # the reference's own ambiguity band (FMA contraction or not) and distance from the exact sums
    wf = oracle.dequantize_rowscale(q, s)
    y64 = oracle.matmul_bt_f64(x, wf)
    assert rel_err(oracle.matmul_bt(x, wf, fma=True), y) < 2e-6
    assert rel_err(y, y64) < 5e-6
    u, sg, bg = affine_g64_from_sym(q, 0)
    ya = oracle.qlinear_affine(x, u, sg, bg, u.shape)
    assert hashlib.sha256(ya.tobytes()).digest() == kat["cfg1_affine_y_sha256"].tobytes()


# ---- glue after the linears: SiLU, mul, pair-interleaved SwiGLU, greedy sampling, top_k ----

def test_silu_mul_hand_values(oracle):
    x = np.array([0.0, 1.0, -1.0, 10.0, -10.0], np.float32)
    got = oracle.silu(x)
    want = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))     # kernels.wgsl:104-113 in exact arithmetic
    assert got[0] == 0.0 and np.allclose(got, want, rtol=3e-7, atol=0)
    assert abs(float(got[1]) - 0.7310585786300049) < 1e-7 and abs(float(got[2]) + 0.2689414213699951) < 1e-7
    a = np.array([1.5, -2.0, 3.0], np.float32)
    b = np.array([2.0, 0.5, -1.0], np.float32)
    assert oracle.mul(a, b).tolist() == [3.0, -1.0, -3.0]                     # kernels.wgsl:146-151


def test_swiglu_pairs_is_silu_of_the_gate_times_up(oracle):
    """MLP::forward (rusty-graph/src/lib.rs:317-323) applies SiLU to the GATE projection; columns (2j, 2j+1) hold
    (gate_j, up_j)."""
    rng = np.random.default_rng(0)
    g = rng.standard_normal((3, 5)).astype(np.float32) * 3
    u = rng.standard_normal((3, 5)).astype(np.float32)
    s = np.empty((3, 10), np.float32)
    s[:, 0::2], s[:, 1::2] = g, u
    got = oracle.swiglu_pairs(s)
    assert np.array_equal(got.view(np.uint32), oracle.mul(oracle.silu(g), u).view(np.uint32))
    assert not np.array_equal(got, oracle.mul(oracle.silu(u), g))              # the unused fused shader's order differs


def test_greedy_sample_and_top_k_tie_rules(oracle):
    x = np.array([1.0, 5.0, 3.0, 5.0, 2.0], np.float32)
    assert oracle.greedy_sample(x) == 3             # Iterator::max_by keeps the last maximum (tokenizer.rs:151-158)
    assert oracle.top_k(x, 3).tolist() == [1, 3, 2]  # strict '>' keeps the first (kernels.wgsl:168-188)
    assert oracle.greedy_sample(np.array([], np.float32)) == 0
    assert oracle.greedy_sample(np.array([np.nan, -1.0, np.nan], np.float32)) == 1
    assert oracle.top_k(np.array([-2e9, -3e9], np.float32), 1).tolist() == [0]   # nothing beats the -1e9 start: index 0


# ---- the steps in front of a layer's Linears (kernels.wgsl:81-102, :570-597; rusty-graph/src/lib.rs:121-135) ----
def test_rms_norm_follows_the_shader_formula(oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    x[2] *= 1e-4
    x[3, 17] = 500.0
    r = rng.standard_normal((5, 256)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 256).astype(np.float32)
    got = oracle.rms_norm(x, w)
    exact = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * w
    assert np.max(np.abs(got - exact) / np.max(np.abs(exact), axis=1, keepdims=True)) < 1e-6
    # the shader's own sequence of f32 operations, restated with numpy scalars for one row
    ss = np.float32(0)
    for v in x[1]:
        ss = np.float32(ss + np.float32(v * v))
    inv = np.float32(1.0) / np.sqrt(np.float32(np.float32(ss / np.float32(256)) + np.float32(1e-5)))
    assert np.array_equal(got[1], (x[1] * inv) * w)
    got_r, s = oracle.rms_norm(x, w, residual=r, return_sum=True)
    assert np.array_equal(s, x + r)
    assert np.array_equal(got_r, oracle.rms_norm(x + r, w))
    # a row of zeros stays zero (eps keeps the root away from 0)
    assert np.array_equal(oracle.rms_norm(np.zeros((1, 8), np.float32), np.ones(8, np.float32)), np.zeros((1, 8), np.float32))


def test_embedding_picks_rows(oracle):
    table = np.arange(40, dtype=np.float32).reshape(10, 4)
    out, bad = oracle.embedding(table, [9, 0, 3, 3])
    assert bad == 0 and np.array_equal(out, table[[9, 0, 3, 3]])
    out, bad = oracle.embedding(table, [10, 2])
    assert bad == 1 and np.array_equal(out[0], np.zeros(4, np.float32)) and np.array_equal(out[1], table[2])
    out, bad = oracle.embedding(table, [])
    assert out.shape == (0, 4) and bad == 0
