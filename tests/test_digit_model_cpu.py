"""The arithmetic of the int8 tensor-core GEMV (rusty_b200/csrc/gemv_mma.cu) restated in numpy, checked on CPU: why feeding
the tensor core integers loses nothing against the reference's f32 dequantise-then-matmul.

Per activation row and K slice (8 slices: k-bytes [128 w, 128 w + 128) of every 1024): a power-of-two scale brings the
slice's largest |a| into [64, 128); T = round(a * scale * 2^21) is split EXACTLY into four balanced base-128 digits; the
integer dot products per digit plane are recombined in 64-bit integers and leave the slice as a double; the slices are
added in a fixed order and rounded to f32 once.  For weights with one scale per output row that scale multiplies the sum;
for the reference's own format (u8 [in,out], one scale and bias per 64 consecutive outputs of an input row) the group's
scales ride on the activations, a = fl32(x * s_g), and the bias term sum_k x * b_g is added per slice in double."""
import numpy as np
import pytest

from parity import TOL_FP32, rel_err


def _digits(a32: np.ndarray):
    """a32: one K slice of one activation row (f32).  Returns (digit planes int64 [4, n], most significant first; e2)."""
    v = float(np.max(np.abs(a32))) if a32.size else 0.0
    if v == 0.0:
        return np.zeros((4, a32.size), np.int64), 0
    e = int(np.floor(np.log2(v))) + 1          # v = f * 2^e, f in [0.5, 1)
    e2 = 7 - e                                 # v * 2^e2 in [64, 128)
    if v * 2.0 ** e2 > 127.0:
        e2 -= 1
    t = np.rint(a32.astype(np.float64) * 2.0 ** (e2 + 21)).astype(np.int64)   # the device does this in f32: exact, |t| < 2^28
    assert np.all(np.abs(t) <= 127 * 2 ** 21)
    planes, rest = [], t.copy()
    for _ in range(3):                         # least significant first: balanced digits in [-64, 63]
        d = ((rest + 64) % 128) - 64
        planes.append(d)
        rest = (rest - d) // 128
    planes.append(rest)                        # top digit
    assert np.all(np.abs(rest) <= 127) and all(np.all((p >= -64) & (p <= 63)) for p in planes[:3])
    d3, d2, d1, d0 = planes                    # d0 = most significant
    assert np.array_equal(((d0 * 128 + d1) * 128 + d2) * 128 + d3, t)         # the split is exact
    return np.stack([d0, d1, d2, d3]), e2


def _slices(K: int):
    for w in range(8):
        idx = np.concatenate([np.arange(c + 128 * w, min(c + 128 * w + 128, K)) for c in range(0, K, 1024)
                              if c + 128 * w < K]) if K > 128 * w else np.zeros(0, np.int64)
        yield idx.astype(np.int64)


def _model_row(a32: np.ndarray, wq: np.ndarray, extra=None) -> np.ndarray:
    """One activation row a32 [K] against integer weights wq [N, K]; `extra(idx)` adds a per-slice double [N]."""
    N, K = wq.shape
    acc = np.zeros(N, np.float64)
    for idx in _slices(K):
        if idx.size == 0:
            continue
        d, e2 = _digits(a32[idx])
        w = wq[:, idx].astype(np.int64)
        hi = (w @ d[0]) * 128 + (w @ d[1])     # as the kernel folds its accumulator columns
        lo = (w @ d[2]) * 128 + (w @ d[3])
        part = (hi * 16384 + lo).astype(np.float64) * 2.0 ** (-e2 - 21)       # exact: an integer times a power of two
        if extra is not None:
            part = part + extra(idx)
        acc += part                            # slices in a fixed order
    return acc.astype(np.float32)              # one rounding


@pytest.mark.parametrize("K,N", [(1024, 48), (4096, 64), (1152, 33)])
def test_symmetric_weights_model_matches_the_oracle(oracle, K, N):
    from rusty_b200.workloads import sym_row_linear
    x, q, s = sym_row_linear(K + N, 2, K, N)
    x[0, ::97] *= 40.0
    got = np.stack([_model_row(x[m], q) * s for m in range(2)])
    wf = oracle.dequantize_rowscale(q, s)
    ref = oracle.matmul_bt(x, wf)
    assert rel_err(got, ref) <= TOL_FP32
    # and closer to the exact sums than the reference's own f32 accumulation is
    exact = oracle.matmul_bt_f64(x, wf)
    assert rel_err(got, exact) <= max(rel_err(ref, exact), 1e-7) * 1.5


@pytest.mark.parametrize("K,N", [(1024, 64), (4096, 128), (1152, 192)])
def test_reference_format_model_matches_the_oracle(oracle, K, N):
    from rusty_b200.workloads import sym_row_linear
    x, q, _ = sym_row_linear(3 * K + N, 2, K, N)
    x[1, ::61] *= 25.0
    rng = np.random.default_rng(K + N)
    ukn = (np.ascontiguousarray(q.T).astype(np.int16) + 128).astype(np.uint8)          # [K, N]
    sg = rng.uniform(0.001, 0.02, size=(K, N // 64)).astype(np.float32)
    bg = (-128.0 * sg + rng.uniform(-0.05, 0.05, size=sg.shape)).astype(np.float32)
    got = np.empty((2, N), np.float32)
    for g in range(N // 64):
        u = np.ascontiguousarray(ukn[:, 64 * g:64 * g + 64].T)                           # the group's rows, [64, K]
        for m in range(2):
            a = (x[m] * sg[:, g]).astype(np.float32)                                     # one f32 rounding per element
            bias = lambda idx, m=m, g=g: float(np.dot(x[m, idx].astype(np.float64), bg[idx, g].astype(np.float64)))
            got[m, 64 * g:64 * g + 64] = _model_row(a, u, extra=bias)
    ref = oracle.qlinear_affine(x, ukn, sg.ravel(), bg.ravel(), ukn.shape, layout_nk=False)
    assert rel_err(got, ref) <= TOL_FP32
    wf = np.ascontiguousarray(oracle.affine_dequantize(ukn, sg.ravel(), bg.ravel()).reshape(K, N).T)
    exact = oracle.matmul_bt_f64(x, wf)
    assert rel_err(got, exact) <= max(rel_err(ref, exact), 1e-6) * 1.5
