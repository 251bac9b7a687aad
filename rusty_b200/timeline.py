"""Timeline of the decode kernel pair (digit pre-pass + int8 tensor-core GEMM) inside a CUDA-graph replay.

A development tool, not part of the product path.  It needs the development build of the library, whose kernels can
write ``%globaltimer`` stamps into a buffer (the regular build compiles the stamps out and does not export the hook):

    RUSTY_TIMELINE=1 python -m rusty_b200.build          # rebuilds everything with -DRUSTY_TIMELINE
    python -m rusty_b200.timeline 32 4096 4096           # M K N, one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29701 \
        -m rusty_b200.timeline 32 4096 4096              # two ranks: every Linear is a row shard pushed to the peer
    python -m rusty_b200.build                           # back to the regular build

Twelve Linears with separate weight copies are captured in one graph and replayed; the steady-state Linears are
printed with the times (µs from the first pre-pass of the graph, this GPU's clock) at which the phases were reached:
minimum and maximum over the CTAs of the GEMM.  Development-build environment switches: RUSTY_PEER_EXP=1 drops the
meeting of the ranks, =2 the stores into the other ranks' memory, =3 both; RUSTY_TC_SMS=n plans the GEMM for n SMs.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

NL = 12
REGION = 152 * 16   # 148 CTAs x 16 stamps, then the pre-pass's stamps in region 150


def main() -> None:
    M, K, N = (int(a) for a in sys.argv[1:4])
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo")   # host channel for the IPC handles and for printing in rank order
    import rusty_b200
    from rusty_b200 import DType, QLinear, UnifiedTensor, capi
    from rusty_b200.backend import Graph
    from rusty_b200.shard import Arena, arena_layout, forward_pushed, shard_rows
    from rusty_b200.workloads import sym_row_linear

    l = C.CDLL(capi.LIB_PATH)
    if not hasattr(l, "rusty_cuda_debug_set_timeline"):
        raise SystemExit("this is the regular build: rebuild with RUSTY_TIMELINE=1 python -m rusty_b200.build")
    l.rusty_cuda_debug_set_timeline.argtypes = [C.c_void_p, C.c_void_p]

    ctx = rusty_b200.CudaContext(int(os.environ.get("LOCAL_RANK", "0")))
    eng = rusty_b200.ComputeEngine(ctx)
    x, q, s = sym_row_linear(0, M, K, N)
    rows = shard_rows(N, world, rank)
    qls = [QLinear.from_host(ctx, q[rows], s[rows]) for _ in range(NL)]
    xt = UnifiedTensor.new(ctx, x, [M, K])
    arena = None
    if world > 1:
        offsets, total = arena_layout([(0, M * N * 4), (1, M * N * 4)])
        arena = Arena(ctx, total, world, rank)
        arena.connect(dist)
        ys = [arena.tensor(offsets[i], [M, N], DType.FP32) for i in range(2)]

        def chain():
            for i, ql in enumerate(qls):
                forward_pushed(ctx, arena, ql, xt, M, ys[i % 2])
    else:
        y = UnifiedTensor.empty(ctx, [M, N])

        def chain():
            for ql in qls:
                eng.qlinear(ctx, xt, ql, y)
    dbg = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(NL * REGION, np.int64), [NL * REGION * 8], DType.U8)
    chain()
    ctx.sync()
    if dist:
        dist.barrier()
    l.rusty_cuda_debug_set_timeline(ctx.handle, dbg.buffer())
    g = Graph(ctx)
    with g:
        chain()
    l.rusty_cuda_debug_set_timeline(ctx.handle, None)
    if dist:
        dist.barrier()
    for _ in range(500):
        g.launch()
    ctx.sync()
    if dist:
        dist.barrier()
    t = dbg.to_bytes(ctx).view(np.int64).reshape(NL, 152, 16)
    t0 = t[0, 150, 0]

    def us(v):
        return "%7.2f" % ((v - t0) / 1000.0) if v else "    -  "

    out = [f"rank {rank} of {world}: {M}x{K}x{N} plan {qls[0].plan(M)}"]
    for i in range(6, 10):
        d, ct = t[i, 150], t[i, :148]
        act = ct[:, 0] > 0

        def mm(sl):
            v = ct[act, sl]
            v = v[v > 0]
            return (us(v.min()) + "," + us(v.max())) if v.size else "-"
        sync = f" arrived={us(d[4])} told_peers={us(d[5])} polls={int(d[6])} met={us(d[3])}" if world > 1 else ""
        out.append(f"L{i}: pre-pass launched={us(d[0])} released={us(d[1])}{sync} end={us(d[2])} | GEMM ctas={int(act.sum())} "
                   f"start[{mm(0)}] released[{mm(1)}] first_mma[{mm(4)}] last_mma[{mm(5)}] folded[{mm(7)}] pieces_done[{mm(11)}] exit[{mm(15)}]")
    out.append("period per Linear: %.2f us" % ((t[9, 150, 1] - t[5, 150, 1]) / 4000.0))
    for r in range(world):
        if r == rank:
            print("\n".join(out), flush=True)
        if dist:
            dist.barrier()
    ctx.sync()
    if arena is not None:
        dist.barrier()
        arena.destroy()
    ctx.destroy()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
