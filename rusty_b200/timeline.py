"""Where the time of one decode Linear goes: `python -m rusty_b200.timeline M K N [count]`.

Records `count` fused linears of one shape (separate weight copies, so every launch streams HBM) into a CUDA graph
with the library's timeline hook attached (rusty_cuda_debug_set_timeline), replays the graph a few times and prints,
per Linear, the %globaltimer stamps of the digit pre-pass and of the int8 tensor-core kernel in microseconds relative
to the first pre-pass.  A development aid for the M >= 5 path; the numbers quoted in profiles/ come from it.
"""
from __future__ import annotations

import ctypes as C
import sys

import numpy as np

from . import ComputeEngine, CudaContext, DType, QLinear, UnifiedTensor
from .backend import Graph
from .capi import check, lib
from .workloads import sym_row_linear

REGION = 152 * 16


def main(argv) -> int:
    if len(argv) < 3:
        print(__doc__)
        return 2
    M, K, N = (int(a) for a in argv[:3])
    count = int(argv[3]) if len(argv) > 3 else 8
    ctx = CudaContext(0)
    eng = ComputeEngine(ctx)
    x, q, s = sym_row_linear(0, M, K, N)
    qls = [QLinear.from_host(ctx, q, s) for _ in range(count)]
    if qls[0].plan(M) != "tcgen05":
        print(f"M={M}: the timeline covers the int8 tensor-core kernel pair (plan is {qls[0].plan(M)})")
        return 2
    xt = UnifiedTensor.new(ctx, x, [M, K])
    y = UnifiedTensor.empty(ctx, [M, N])
    dbg = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(count * REGION, np.int64), [count * REGION * 8], DType.U8)
    for ql in qls:
        eng.qlinear(ctx, xt, ql, y)
    ctx.sync()
    check(lib().rusty_cuda_debug_set_timeline(ctx.handle, dbg.buffer()), ctx.handle)
    g = Graph(ctx)
    with g:
        for ql in qls:
            eng.qlinear(ctx, xt, ql, y)
    check(lib().rusty_cuda_debug_set_timeline(ctx.handle, None), ctx.handle)
    for _ in range(3):
        g.launch()
    ctx.sync()
    t = dbg.to_bytes(ctx).view(np.int64).reshape(count, 152, 16)
    t0 = t[0, 150, 0]

    def us(v) -> str:
        return "%7.2f" % ((v - t0) / 1000.0) if v else "    -  "

    print(f"{M}x{K}x{N}: microseconds from the first pre-pass; one line per Linear (the first ones include start-up)")
    for i in range(count):
        d, ct = t[i, 150], t[i, :148]
        act = ct[:, 0] > 0
        c0 = ct[0]
        print(f"L{i}: pre-pass waited={us(d[1])} end={us(d[2])} | GEMM ctas={int(act.sum())} first_mma={us(c0[4])} last_mma={us(c0[5])} "
              f"staged={us(c0[7])} reduce_issued={us(c0[8])} pieces_in={us(c0[10])} converted={us(c0[11])} "
              f"exit[min,max]={us(ct[act, 15].min())},{us(ct[act, 15].max())}")
    if count >= 4:
        period = (t[count - 1, 150, 1] - t[2, 150, 1]) / 1000.0 / (count - 3)
        print(f"period per Linear (steady state): {period:.2f} us")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
