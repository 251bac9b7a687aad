"""ctypes front end of the CPU oracle (``oracle/rusty_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke``
and by the CPU-baseline legs of ``bench.py``; never by the product package.

PARITY UNPINNED: the reference holds no golden vector for this path and its
Rust + WGSL sources cannot run here, so the oracle is pinned only by the shader
text each C function cites.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u32p = C.POINTER(C.c_uint32)
_i8p = C.POINTER(C.c_int8)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "rusty_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _words(b: np.ndarray):
    """View a byte array as little-endian u32 words, zero-padded to a multiple of 4."""
    b = np.ascontiguousarray(b).view(np.uint8).ravel()
    pad = (-b.size) % 4
    if pad:
        b = np.concatenate([b, np.zeros(pad, np.uint8)])
    w = b.view("<u4").copy()
    return w, w.ctypes.data_as(_u32p)


def num_threads() -> int:
    return lib().oracle_num_threads()


def set_num_threads(n: int) -> int:
    """Use `n` host threads in the threaded (timing) variants, whatever OMP_NUM_THREADS says; returns the count in force."""
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def matmul_tiled(a, b, fma: bool = False) -> np.ndarray:
    a, pa = _f32(a)
    b, pb = _f32(b)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    out = np.empty((M, N), np.float32)
    fn = lib().oracle_matmul_tiled_fma if fma else lib().oracle_matmul_tiled
    fn(pa, pb, out.ctypes.data_as(_f32p), C.c_uint32(M), C.c_uint32(K), C.c_uint32(N))
    return out


def matmul_bt(a, b, fma: bool = False, mt: bool = False) -> np.ndarray:
    a, pa = _f32(a)
    b, pb = _f32(b)
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2
    out = np.empty((M, N), np.float32)
    if mt:
        fn = lib().oracle_matmul_bt_mt
    else:
        fn = lib().oracle_matmul_bt_fma if fma else lib().oracle_matmul_bt
    fn(pa, pb, out.ctypes.data_as(_f32p), C.c_uint32(M), C.c_uint32(K), C.c_uint32(N))
    return out


def matmul_bt_f64(a, b) -> np.ndarray:
    a, pa = _f32(a)
    b, pb = _f32(b)
    M, K = a.shape
    N, _ = b.shape
    out = np.empty((M, N), np.float64)
    lib().oracle_matmul_bt_f64(pa, pb, out.ctypes.data_as(_f64p), C.c_uint32(M), C.c_uint32(K), C.c_uint32(N))
    return out


def dequantize(in_bytes, n_in: int | None = None, n_out: int | None = None, out_init=None) -> np.ndarray:
    """`dequantize` shader: n_in = product of the input tensor's shape (defaults
    to the byte count), n_out = length of the f32 output (defaults to n_in)."""
    raw = np.ascontiguousarray(in_bytes).view(np.uint8).ravel()
    w, pw = _words(raw)
    n_in = raw.size if n_in is None else n_in
    n_out = n_in if n_out is None else n_out
    out = np.full(n_out, np.nan, np.float32) if out_init is None else np.array(out_init, np.float32)
    lib().oracle_dequantize(pw, C.c_size_t(w.size), C.c_size_t(n_in), out.ctypes.data_as(_f32p), C.c_size_t(n_out))
    return out


def affine_dequantize(w_u8, scales, biases, n: int | None = None, fma=False, as_dispatched=False,
                      out_init=None, mt=False) -> np.ndarray:
    raw = np.ascontiguousarray(w_u8).view(np.uint8).ravel()
    n = raw.size if n is None else n
    w, pw = _words(raw)
    s, ps = _f32(np.ravel(scales))
    b, pb = _f32(np.ravel(biases))
    assert s.size * 64 >= n and b.size * 64 >= n
    out = np.full(n, np.nan, np.float32) if out_init is None else np.array(out_init, np.float32)
    if as_dispatched:
        fn = lib().oracle_affine_dequantize_as_dispatched
    elif mt:
        fn = lib().oracle_affine_dequantize_mt
    else:
        fn = lib().oracle_affine_dequantize_fma if fma else lib().oracle_affine_dequantize
    fn(pw, ps, pb, out.ctypes.data_as(_f32p), C.c_size_t(n))
    return out


def dequantize_rowscale(q, scale, layout_nk: bool = True) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    if layout_nk:
        N, K = q.shape
    else:
        K, N = q.shape
    s, ps = _f32(scale)
    assert s.size == N
    wf = np.empty(q.shape, np.float32)
    lib().oracle_dequantize_rowscale(q.ctypes.data_as(_i8p), ps, wf.ctypes.data_as(_f32p),
                                     C.c_uint32(K), C.c_uint32(N), C.c_int(1 if layout_nk else 0))
    return wf


def qlinear_rowscale(x, q, scale, layout_nk: bool = True) -> np.ndarray:
    """Mode B composite: sign-extended unpack * per-row scale, then matmul_bt
    ([N,K] layout) or matmul_tiled ([K,N] layout)."""
    wf = dequantize_rowscale(q, scale, layout_nk)
    return matmul_bt(x, wf) if layout_nk else matmul_tiled(x, wf)


def qlinear_affine(x, w_u8, scales, biases, shape, layout_nk: bool = True) -> np.ndarray:
    """Mode A composite: affine_dequantize over the flat index, then the matmul
    that matches the weight's storage order."""
    wf = affine_dequantize(w_u8, scales, biases).reshape(shape)
    return matmul_bt(x, wf) if layout_nk else matmul_tiled(x, wf)


def time_matmul_bt_mt(a, wf, simd: bool) -> None:
    """One threaded f32 matmul_bt call (timing leg only; result discarded)."""
    a, pa = _f32(a)
    wf, pw = _f32(wf)
    M, K = a.shape
    N, _ = wf.shape
    out = np.empty((M, N), np.float32)
    fn = lib().oracle_matmul_bt_mt_simd if simd else lib().oracle_matmul_bt_mt
    fn(pa, pw, out.ctypes.data_as(_f32p), C.c_uint32(M), C.c_uint32(K), C.c_uint32(N))
    return out


def qlinear_rowscale_fused_mt(x, q, scale, simd: bool = False) -> np.ndarray:
    x, px = _f32(x)
    q = np.ascontiguousarray(q, dtype=np.int8)
    s, ps = _f32(scale)
    M, K = x.shape
    N, _ = q.shape
    y = np.empty((M, N), np.float32)
    fn = lib().oracle_qlinear_rowscale_fused_mt_simd if simd else lib().oracle_qlinear_rowscale_fused_mt
    fn(px, q.ctypes.data_as(_i8p), ps, y.ctypes.data_as(_f32p), C.c_uint32(M), C.c_uint32(K), C.c_uint32(N))
    return y


# --- numpy mirrors (independent restatement used to cross-check the C code) ---

def np_dequantize(in_bytes) -> np.ndarray:
    """kernels.wgsl:156-166 for an input whose length is a multiple of 4."""
    w = np.ascontiguousarray(in_bytes).view(np.uint8).ravel().view("<u4")
    lanes = np.stack([(w >> (8 * j)) & 0xFF for j in range(4)], axis=1)
    return lanes.astype(np.float32).ravel()


def np_affine_dequantize(w_u8, scales, biases) -> np.ndarray:
    """kernels.wgsl:385-400 (intended semantics, every element)."""
    u = np.ascontiguousarray(w_u8).view(np.uint8).ravel()
    g = np.arange(u.size) // 64
    s = np.asarray(scales, np.float32).ravel()[g]
    b = np.asarray(biases, np.float32).ravel()[g]
    return (u.astype(np.float32) * s).astype(np.float32) + b


def np_matmul_seq(a, b_kn) -> np.ndarray:
    """k-ascending f32 accumulation, vectorised over outputs (kernels.wgsl:24-49)."""
    a = np.asarray(a, np.float32)
    b_kn = np.asarray(b_kn, np.float32)
    acc = np.zeros((a.shape[0], b_kn.shape[1]), np.float32)
    for k in range(a.shape[1]):
        acc = acc + (a[:, k:k + 1] * b_kn[k:k + 1, :]).astype(np.float32)
    return acc


def silu(x) -> np.ndarray:
    """`silu` shader: x * (1 / (1 + exp(-x)))."""
    a, pa = _f32(np.ravel(x))
    out = np.empty(a.size, np.float32)
    lib().oracle_silu(pa, out.ctypes.data_as(_f32p), C.c_size_t(a.size))
    return out.reshape(np.shape(x))


def mul(a, b) -> np.ndarray:
    """`mul` shader: elementwise product."""
    x, px = _f32(np.ravel(a))
    y, py = _f32(np.ravel(b))
    assert x.size == y.size
    out = np.empty(x.size, np.float32)
    lib().oracle_mul(px, py, out.ctypes.data_as(_f32p), C.c_size_t(x.size))
    return out.reshape(np.shape(a))


def swiglu_pairs(s) -> np.ndarray:
    """[M, 2F] with (gate_j, up_j) in columns (2j, 2j+1) -> [M, F] = silu(gate) * up (MLP::forward order)."""
    s2 = np.ascontiguousarray(s, np.float32)
    M, F2 = s2.shape
    out = np.empty((M, F2 // 2), np.float32)
    lib().oracle_swiglu_pairs(s2.ctypes.data_as(_f32p), out.ctypes.data_as(_f32p), C.c_uint32(M), C.c_uint32(F2 // 2))
    return out


def rms_norm(x, weight, residual=None, eps: float = 1e-5, return_sum: bool = False):
    """`rms_norm` / `rms_norm_residual` shaders applied to every row of x[M, K] (sequential f32 sums)."""
    a = np.ascontiguousarray(x, np.float32)
    M, K = a.reshape(-1, a.shape[-1]).shape
    w, pw = _f32(np.ravel(weight))
    assert w.size == K
    r = None if residual is None else np.ascontiguousarray(residual, np.float32)
    out = np.empty((M, K), np.float32)
    sm = np.empty((M, K), np.float32) if (return_sum and r is not None) else None
    lib().oracle_rms_norm_rows(a.ctypes.data_as(_f32p), r.ctypes.data_as(_f32p) if r is not None else None, pw,
                               out.ctypes.data_as(_f32p), sm.ctypes.data_as(_f32p) if sm is not None else None,
                               C.c_uint32(M), C.c_uint32(K), C.c_float(eps))
    out = out.reshape(a.shape)
    return (out, sm.reshape(a.shape)) if sm is not None else out


def embedding(table, ids):
    """Embedding::forward: rows of table[vocab, dim] picked by ids; returns (out[n, dim], ids outside the table)."""
    t = np.ascontiguousarray(table, np.float32)
    i = np.ascontiguousarray(ids, np.uint32)
    out = np.empty((i.size, t.shape[1]), np.float32)
    lib().oracle_embedding.restype = C.c_uint32
    bad = lib().oracle_embedding(t.ctypes.data_as(_f32p), i.ctypes.data_as(C.POINTER(C.c_uint32)), out.ctypes.data_as(_f32p),
                                 C.c_size_t(i.size), C.c_uint32(t.shape[0]), C.c_uint32(t.shape[1]))
    return out, int(bad)


def greedy_sample(logits) -> int:
    """Sampler::sample with temperature <= 0: index of the maximum, the last one among equals."""
    a, pa = _f32(np.ravel(logits))
    lib().oracle_greedy_sample.restype = C.c_uint32
    return int(lib().oracle_greedy_sample(pa, C.c_size_t(a.size)))


def top_k(values, k: int) -> np.ndarray:
    """`top_k` shader: k indices, largest first, first index among equals."""
    a, pa = _f32(np.ravel(values))
    out = np.zeros(k, np.uint32)
    lib().oracle_top_k(pa, C.c_size_t(a.size), C.c_uint32(k), out.ctypes.data_as(C.POINTER(C.c_uint32)))
    return out
