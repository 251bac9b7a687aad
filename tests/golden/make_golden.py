"""Writes tests/golden/kat.npz: small known-answer vectors for the path.

    python tests/golden/make_golden.py

The reference (Rust + WGSL via wgpu) cannot run in this environment and holds
no golden vectors of its own for matmul / dequantize, so these vectors are
produced by the C oracle (oracle/rusty_oracle.c), whose functions restate the
shader text line by line.  Hand-derivable cases (byte-lane order, the 2x2
identity product of rusty-backend/examples/ops_test.rs:9-17) are additionally
asserted against literals in tests/test_oracle.py, which is what pins the
oracle; the rest pins the CUDA kernels and guards the oracle against drift.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from rusty_b200.workloads import affine_g64_from_sym, sym_row_linear  # noqa: E402


def main() -> None:
    out = {}
    rng = np.random.default_rng(1234)

    # 1. ops_test.rs: [[1,2],[3,4]] x identity
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.eye(2, dtype=np.float32)
    out["ops_a"], out["ops_b"], out["ops_out"] = a, b, O.matmul_tiled(a, b)

    # 2. dequantize: lane order, extremes, ragged lengths
    raw = np.array([1, 2, 3, 4, 0, 127, 128, 255, 9, 8, 7, 6], np.uint8)
    out["deq_in"] = raw
    out["deq_out"] = O.dequantize(raw)                       # 12 in, 12 out
    out["deq_out_n7"] = O.dequantize(raw[:8], n_in=7, n_out=7)   # out shorter than 2 words
    out["deq_out_short_in"] = O.dequantize(raw[:8], n_in=12, n_out=12,
                                           out_init=np.full(12, -1.0, np.float32))  # input has 2 words only
    big = rng.integers(0, 256, size=1000, dtype=np.uint8)
    out["deq_big_in"], out["deq_big_out"] = big, O.dequantize(big)

    # 3. affine_dequantize: group boundary 63/64, n not a multiple of 64 or 16
    n = 203
    u = rng.integers(0, 256, size=n, dtype=np.uint8)
    s = rng.uniform(0.001, 0.02, size=4).astype(np.float32)
    bb = rng.uniform(-2, 2, size=4).astype(np.float32)
    out["aff_u"], out["aff_s"], out["aff_b"] = u, s, bb
    out["aff_out"] = O.affine_dequantize(u, s, bb)
    out["aff_out_fma"] = O.affine_dequantize(u, s, bb, fma=True)

    # 4. matmul tails around the 16-wide tile
    dims = [1, 15, 16, 17, 33]
    k = 0
    for M in dims:
        for K in (1, 17, 33):
            for N in (1, 16, 33):
                a = rng.standard_normal((M, K)).astype(np.float32)
                b = rng.standard_normal((K, N)).astype(np.float32)
                out[f"mm{k}_a"], out[f"mm{k}_b"] = a, b
                out[f"mm{k}_out"] = O.matmul_tiled(a, b)
                out[f"mm{k}_out_fma"] = O.matmul_tiled(a, b, fma=True)
                out[f"mm{k}_bt_out_fma"] = O.matmul_bt(a, np.ascontiguousarray(b.T), fma=True)
                k += 1
    out["mm_count"] = np.array(k)

    # 5. fused linear, both modes and layouts, small
    x, q, sc = sym_row_linear(7, 3, 128, 48)
    out["ql_x"], out["ql_q"], out["ql_s"] = x, q, sc
    out["ql_y_nk"] = O.qlinear_rowscale(x, q, sc, layout_nk=True)
    qkn = np.ascontiguousarray(q.T)
    out["ql_y_kn"] = O.qlinear_rowscale(x, qkn, sc, layout_nk=False)
    x2, q2, _ = sym_row_linear(8, 2, 128, 64)
    u2, s2, b2 = affine_g64_from_sym(q2, 8)
    out["qa_x"], out["qa_u"], out["qa_s"], out["qa_b"] = x2, u2, s2, b2
    out["qa_y_nk"] = O.qlinear_affine(x2, u2, s2, b2, u2.shape, layout_nk=True)
    u2kn = np.ascontiguousarray(u2.T)  # a [K,N] = [128,64] stored matrix with its own flat groups
    out["qa_ukn"] = u2kn
    out["qa_y_kn"] = O.qlinear_affine(x2, u2kn, s2, b2, u2kn.shape, layout_nk=False)

    # 6. digests of the oracle on the first benchmark configuration (seed 0)
    x, q, sc = sym_row_linear(0, 1, 4096, 4096)
    y = O.qlinear_rowscale(x, q, sc, layout_nk=True)
    out["cfg1_y_sha256"] = np.frombuffer(hashlib.sha256(y.tobytes()).digest(), np.uint8)
    out["cfg1_y_head"] = y[0, :16].copy()
    u, s, b = affine_g64_from_sym(q, 0)
    ya = O.qlinear_affine(x, u, s, b, u.shape, layout_nk=True)
    out["cfg1_affine_y_sha256"] = np.frombuffer(hashlib.sha256(ya.tobytes()).digest(), np.uint8)
    out["cfg1_affine_y_head"] = ya[0, :16].copy()

    path = os.path.join(HERE, "kat.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
