"""The allocation-free entry point, checked against the regular one.

`rusty_cuda_qlinear_i8_forward_static` exists for hosts that may not call
cudaMalloc once they are running (a serving loop with pre-carved memory, a
process whose allocator owns the device).  It takes raw device pointers and
keeps its scratch in an array built into the library.  Here it is called
twice in a row through the C ABI and must agree with
`rusty_cuda_qlinear_forward` on the same inputs; shapes beyond the built-in
scratch must be refused.  This file sorts last so that a run stopping at the
first failure has already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from parity import TOL_FP32, rel_err
from rusty_b200 import QLinear, UnifiedTensor, capi
from rusty_b200.workloads import sym_row_linear

pytestmark = pytest.mark.gpu


def _static_forward(ctx, ql, x, y, M, N, K):
    w, sc, _ = ql._keep
    return capi.lib().rusty_cuda_qlinear_i8_forward_static(
        C.c_void_p(w.device_ptr()), C.c_void_p(sc.device_ptr()), C.c_void_p(x.device_ptr()), C.c_void_p(y.device_ptr()),
        M, N, K, C.c_void_p(ctx.stream()))


# the last shape has more row tiles than SMs with a remainder: whole tiles AND cut tiles in one launch, N % 128 != 0
@pytest.mark.parametrize("M,K,N", [(8, 4096, 4096), (5, 1024, 1000), (1, 8192, 384), (8, 4096, 128 * 200 + 40)])
def test_static_scratch_entry_matches_regular_entry_twice(ctx, engine, oracle, M, K, N):
    xh, qh, sh = sym_row_linear(900 + M + N, M, K, N)
    ql = QLinear.from_host(ctx, qh, sh)
    x = UnifiedTensor.new(ctx, xh, [M, K])
    y_ref = UnifiedTensor.empty(ctx, [M, N])
    engine.qlinear(ctx, x, ql, y_ref)
    want = y_ref.to_vec(ctx).reshape(M, N)
    for call in range(2):   # the array keeps the previous call's contents: a second call must still be right
        y = UnifiedTensor.new(ctx, np.full(M * N, np.nan, np.float32), [M, N])
        rc = _static_forward(ctx, ql, x, y, M, N, K)
        assert rc == capi.OK, capi.lib().rusty_cuda_last_error(None)
        assert capi.lib().rusty_cuda_qlinear_i8_static_status(C.c_void_p(ctx.stream())) == capi.OK   # no wait gave up
        got = y.to_vec(ctx).reshape(M, N)
        assert rel_err(got, want) <= TOL_FP32, f"call {call}"
    ref = oracle.matmul_bt(xh, oracle.dequantize_rowscale(qh, sh), mt=True)
    assert rel_err(got, ref) <= TOL_FP32


def test_static_scratch_entry_refuses_what_does_not_fit(ctx):
    xh, qh, sh = sym_row_linear(7, 1, 64, 16)
    ql = QLinear.from_host(ctx, qh, sh)
    x = UnifiedTensor.new(ctx, np.zeros(9 * 16384, np.float32), [9, 16384])
    y = UnifiedTensor.empty(ctx, [9, 16])
    lib = capi.lib()
    w, sc, _ = ql._keep
    args = (C.c_void_p(w.device_ptr()), C.c_void_p(sc.device_ptr()), C.c_void_p(x.device_ptr()), C.c_void_p(y.device_ptr()))
    assert lib.rusty_cuda_qlinear_i8_forward_static(*args, 9, 16, 64, C.c_void_p(ctx.stream())) == capi.ERR_INVALID_DIMENSIONS
    assert b"fixed scratch" in lib.rusty_cuda_last_error(None)
    assert lib.rusty_cuda_qlinear_i8_forward_static(*args, 1, 16, 16384, C.c_void_p(ctx.stream())) == capi.ERR_INVALID_DIMENSIONS
    assert lib.rusty_cuda_qlinear_i8_forward_static(*args, 1, 16, 72, C.c_void_p(ctx.stream())) == capi.ERR_INVALID_DIMENSIONS
    assert lib.rusty_cuda_qlinear_i8_forward_static(None, *args[1:], 1, 16, 64, C.c_void_p(ctx.stream())) == capi.ERR_INVALID_OPERATION
    # more output features than the built-in arrival counters cover (one per 128-row tile): refused on the host,
    # nothing is launched and none of the (too small) buffers is touched
    assert lib.rusty_cuda_qlinear_i8_forward_static(*args, 1, 262144 + 1, 64, C.c_void_p(ctx.stream())) == capi.ERR_INVALID_DIMENSIONS
    assert b"N <= 262144" in lib.rusty_cuda_last_error(None)
    ctx.sync()
