"""Output-feature sharding of the quantised Linears over the GPUs of one node.

Rank r of G keeps rows [r*N/G, (r+1)*N/G) of every W[out,in] (and their scales);
activations are replicated; each Linear's output is all-gathered so every rank
continues with the whole y[M,N].  The reference has no multi-device code; the
partitioning rule and the reassembly order live here so that CPU ranks (gloo)
and GPU ranks (NCCL through the C ABI) share them.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import numpy as np

from . import capi
from .backend import CudaContext, DType, Graph, UnifiedTensor
from .capi import check, lib


def shard_rows(n: int, world: int, rank: int) -> slice:
    """Rows of W[out,in] (and entries of scale[out]) owned by `rank`."""
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by {world} ranks")
    nl = n // world
    return slice(rank * nl, (rank + 1) * nl)


def assemble(gathered: Sequence[np.ndarray]) -> np.ndarray:
    """Rank-major pieces [G][M, N/G] -> y[M, N] (what the interleave kernel does on the device)."""
    return np.concatenate(list(gathered), axis=1)


class Comm:
    """NCCL communicator owned by the C library (one per context)."""

    def __init__(self, ctx: CudaContext, world: int, rank: int, unique_id: bytes):
        assert len(unique_id) == 128
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        check(lib().rusty_cuda_comm_create(ctx.handle, world, rank, buf, C.byref(h)), ctx.handle)
        self._h, self.ctx, self.world, self.rank = h, ctx, world, rank

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib().rusty_cuda_comm_unique_id(buf))
        return buf.raw

    def check(self) -> None:
        check(lib().rusty_cuda_comm_check(self._h), self.ctx.handle)

    def destroy(self) -> None:
        if self._h is not None:
            lib().rusty_cuda_comm_destroy(self._h)
            self._h = None


def forward_sharded(ctx: CudaContext, comm: Comm, ql_shard, x: UnifiedTensor, M: int, gather_ws: UnifiedTensor,
                    y_full: UnifiedTensor) -> None:
    check(lib().rusty_cuda_qlinear_forward_sharded(ctx.handle, comm._h, ql_shard._h, x.buffer(), int(x.dtype), M,
                                                   gather_ws.buffer(), y_full.buffer(), int(y_full.dtype)), ctx.handle)


class ShardedStack:
    """Runs a LinearStack built with (rank, world): every Linear is this rank's
    shard followed by the all-gather of its output."""

    def __init__(self, stack, dist):
        self.stack = stack
        self.ctx = stack.ctx
        ctx = self.ctx
        world, rank = stack.world, stack.rank
        ids: List = [Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        self.comm = Comm(ctx, world, rank, ids[0])
        M, ydt = stack.M, stack.y_dtype
        self.full_outputs = {}
        for n_full, name in zip(stack.full_n, stack.names):
            key = -1 if name == "lm_head" else n_full
            if key not in self.full_outputs:
                self.full_outputs[key] = UnifiedTensor.empty_with_dtype(ctx, [M, n_full], ydt)
        self._ys = [self.full_outputs[-1 if nm == "lm_head" else n] for n, nm in zip(stack.full_n, stack.names)]
        biggest = max(stack.full_n)
        self.gather_ws = UnifiedTensor.empty_with_dtype(ctx, [M, biggest], ydt)
        self.graph = None

    def full_logits(self) -> UnifiedTensor:
        return self.full_outputs[-1]

    def step(self) -> None:
        s = self.stack
        n = len(s.qls)
        arr = C.c_void_p * n
        check(lib().rusty_cuda_qlinear_forward_sharded_batch(
            self.ctx.handle, self.comm._h, n, arr(*[q._h for q in s.qls]), arr(*[x.buffer() for x in s._xs]),
            int(s.x_dtype), s.M, self.gather_ws.buffer(), arr(*[y.buffer() for y in self._ys]), int(s.y_dtype)),
            self.ctx.handle)

    def capture(self) -> Graph:
        self.step()          # NCCL sets up its channels on the first collective: do that outside the capture
        self.ctx.sync()
        g = Graph(self.ctx)
        with g:
            self.step()
        self.graph = g
        return g

    def replay(self) -> None:
        self.graph.launch()

    def plans(self):
        return self.stack.plans()
