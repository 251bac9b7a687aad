"""Error measures shared by the parity tests.

fp32 dot products of N(0,1) x uniform-int8 terms cross zero, so an elementwise
relative error is unbounded even between two correct evaluations (the
reference's own sequential f32 sum sits up to ~7e-3 elementwise from the exact
value on a K=4096 row).  Parity is therefore measured in the max norm:

    rel_err(y, ref) = max |y - ref| / max |ref|

and, stricter, row by row (``rel_err_rows``: each activation row against its own largest output),
with the tolerances the benchmark specification states: 1e-5 for fp32 paths,
1e-2 for paths that round activations or outputs to bf16.  Integer unpacking is
compared bit for bit.
"""
import numpy as np

TOL_FP32 = 1e-5
TOL_BF16 = 1e-2


def rel_err(y, ref) -> float:
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    assert y.shape == ref.shape, (y.shape, ref.shape)
    denom = float(np.max(np.abs(ref))) if ref.size else 1.0
    if denom == 0.0:
        denom = 1.0
    return float(np.max(np.abs(y - ref))) / denom if ref.size else 0.0


def rel_err_rows(y, ref) -> float:
    """The stricter, row-wise measure: every activation row is normalised by ITS OWN largest reference output,
    max_m ( max_n |y - ref| / max_n |ref[m, :]| ).  Rows of different magnitude (or one row with an outlier
    activation) cannot hide behind the largest row of the batch."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    assert y.shape == ref.shape and y.ndim == 2, (y.shape, ref.shape)
    if not ref.size:
        return 0.0
    denom = np.max(np.abs(ref), axis=1)
    denom[denom == 0.0] = 1.0
    return float(np.max(np.max(np.abs(y - ref), axis=1) / denom))


def assert_bits_equal(a, b):
    a = np.ascontiguousarray(a, np.float32).view(np.uint32)
    b = np.ascontiguousarray(b, np.float32).view(np.uint32)
    assert a.shape == b.shape
    bad = np.flatnonzero(a.ravel() != b.ravel())
    assert bad.size == 0, f"{bad.size} of {a.size} values differ in their bits, first at flat index {bad[:5]}"
