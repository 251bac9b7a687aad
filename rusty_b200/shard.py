"""Output-feature sharding of the quantised Linears over the GPUs of one node.

Rank r of G keeps rows [r*N/G, (r+1)*N/G) of every W[out,in] (and their scales);
activations are replicated; each Linear's output is all-gathered so every rank
continues with the whole y[M,N].  The reference has no multi-device code; the
partitioning rule and the reassembly order live here so that CPU ranks (gloo)
and GPU ranks (NCCL through the C ABI) share them.

Two exchanges are offered: the NCCL all-gather (`Comm`, `ShardedStack`) and
stores into the other ranks' memory from the kernel's epilogue (`Arena`,
`PushedStack`), which needs one process per GPU on one node.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence, Tuple

import numpy as np

from . import capi
from .backend import CudaContext, DType, Graph, UnifiedTensor, _Storage
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


# ---------------------------------------------------------------------------------------------------------------
# Exchange by peer stores
# ---------------------------------------------------------------------------------------------------------------
IPC_HANDLE_BYTES = 64
ARENA_ALIGN = 256


def arena_layout(sizes: Sequence[Tuple[object, int]]) -> Tuple[Dict[object, int], int]:
    """Offsets of named buffers inside an arena's data region, identical on every rank: first come, first placed,
    each start rounded up to 256 bytes.  Returns ({key: offset}, total bytes).  A key given twice keeps its first slot
    and must ask for the same size."""
    offsets: Dict[object, int] = {}
    seen: Dict[object, int] = {}
    total = 0
    for key, nbytes in sizes:
        if nbytes < 0:
            raise ValueError(f"{key!r}: negative size")
        if key in offsets:
            if seen[key] != nbytes:
                raise ValueError(f"{key!r}: sizes {seen[key]} and {nbytes} disagree")
            continue
        offsets[key] = total
        seen[key] = nbytes
        total += (nbytes + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN
    return offsets, total


class _ArenaStorage(_Storage):
    """A window of an arena wearing the interface of a device buffer."""

    def __init__(self, arena: "Arena", offset: int, nbytes: int):
        h = C.c_void_p()
        check(lib().rusty_cuda_arena_buf(arena._h, offset, nbytes, C.byref(h)), arena.ctx.handle)
        self.h, self.ctx, self.nbytes, self._arena = h, arena.ctx, nbytes, arena


class Arena:
    """One device allocation with the same layout on every rank; rank r's kernels store into all of them."""

    def __init__(self, ctx: CudaContext, nbytes: int, world: int, rank: int):
        h = C.c_void_p()
        check(lib().rusty_cuda_arena_create(ctx.handle, nbytes, world, rank, C.byref(h)), ctx.handle)
        self._h, self.ctx, self.world, self.rank, self.nbytes = h, ctx, world, rank, nbytes

    def export(self) -> bytes:
        buf = C.create_string_buffer(IPC_HANDLE_BYTES)
        check(lib().rusty_cuda_arena_export(self._h, buf), self.ctx.handle)
        return buf.raw

    def attach(self, handles: Sequence[bytes]) -> None:
        assert len(handles) == self.world and all(len(h) == IPC_HANDLE_BYTES for h in handles)
        blob = C.create_string_buffer(b"".join(handles), IPC_HANDLE_BYTES * self.world)
        check(lib().rusty_cuda_arena_attach(self._h, blob), self.ctx.handle)

    def connect(self, dist) -> None:
        """Swap handles over a torch.distributed process group (any backend) and map the peers."""
        if self.world == 1:
            return
        handles: List = [None] * self.world
        dist.all_gather_object(handles, self.export())
        self.attach(handles)
        dist.barrier()  # nobody pushes before everybody has attached

    def tensor(self, offset: int, shape: Sequence[int], dtype: DType) -> UnifiedTensor:
        n = int(np.prod(shape, dtype=np.int64)) * dtype.size_bytes()
        return UnifiedTensor(_ArenaStorage(self, offset, n), shape, dtype)

    def wait(self) -> None:
        check(lib().rusty_cuda_arena_wait(self.ctx.handle, self._h), self.ctx.handle)

    def destroy(self) -> None:
        if self._h is not None:
            lib().rusty_cuda_arena_destroy(self._h)
            self._h = None


def forward_pushed(ctx: CudaContext, arena: Arena, ql_shard, x: UnifiedTensor, M: int, y_full: UnifiedTensor) -> None:
    check(lib().rusty_cuda_qlinear_forward_pushed(ctx.handle, arena._h, ql_shard._h, x.buffer(), int(x.dtype), M,
                                                  y_full.buffer(), int(y_full.dtype)), ctx.handle)


def argmax_rows_sharded(ctx: CudaContext, arena: Arena, logits_shard: UnifiedTensor, table: UnifiedTensor,
                        out_idx: UnifiedTensor, out_val=None) -> None:
    """Greedy token per row over column shards: only (value, index) candidates cross NVLink, never the logits.
    `table` is an arena buffer of world * M * 8 bytes at the same offset on every rank; out_idx is u32[M]."""
    M, Nl = int(np.prod(logits_shard.shape[:-1], dtype=np.int64)), int(logits_shard.shape[-1])
    check(lib().rusty_cuda_argmax_rows_sharded(ctx.handle, arena._h, logits_shard.buffer(), M, Nl, table.buffer(),
                                               out_idx.buffer(), out_val.buffer() if out_val is not None else None),
          ctx.handle)


def top_k_rows_sharded(ctx: CudaContext, arena: Arena, logits_shard: UnifiedTensor, k: int, table: UnifiedTensor,
                       out_idx: UnifiedTensor, out_val=None) -> None:
    """The k largest logits per row over column shards: k (value, index) pairs per row and rank cross NVLink.
    `table` is an arena buffer of world * M * k * 8 bytes at the same offset on every rank; out_idx is u32[M, k]."""
    M, Nl = int(np.prod(logits_shard.shape[:-1], dtype=np.int64)), int(logits_shard.shape[-1])
    check(lib().rusty_cuda_top_k_rows_sharded(ctx.handle, arena._h, logits_shard.buffer(), M, Nl, k, table.buffer(),
                                              out_idx.buffer(), out_val.buffer() if out_val is not None else None),
          ctx.handle)


class PushedStack:
    """Runs a LinearStack built with (rank, world): every Linear computes this rank's output columns and stores them
    into every rank's copy of the full output (no collective call).  Outputs of equal width share one arena buffer;
    the stack never writes the same buffer in two consecutive Linears."""

    def __init__(self, stack, dist):
        self.stack = stack
        self.ctx = stack.ctx
        ctx = self.ctx
        M, ydt = stack.M, stack.y_dtype
        keys = [(-1 if nm == "lm_head" else n) for n, nm in zip(stack.full_n, stack.names)]
        for a, b in zip(keys, keys[1:]):
            assert a != b, "two consecutive Linears would share an output buffer"
        sizes = [(k, M * (n if k != -1 else n) * ydt.size_bytes()) for k, n in zip(keys, stack.full_n)]
        sizes.append(("candidates", stack.world * M * 8))   # greedy tail: per-rank (value, index) of every row
        offsets, total = arena_layout(sizes)
        self.arena = Arena(ctx, total, stack.world, stack.rank)
        self.arena.connect(dist)
        self.full_outputs = {k: self.arena.tensor(offsets[k], [M, n], ydt) for k, n in zip(keys, stack.full_n)}
        self._ys = [self.full_outputs[k] for k in keys]
        self._table = self.arena.tensor(offsets["candidates"], [stack.world * M * 8], DType.U8)
        self.tokens = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(M, np.uint32), [M * 4], DType.U8)
        self.graph = None
        self._dist = dist

    def full_logits(self) -> UnifiedTensor:
        return self.full_outputs[-1]

    def step(self) -> None:
        s = self.stack
        n = len(s.qls)
        arr = C.c_void_p * n
        check(lib().rusty_cuda_qlinear_forward_pushed_batch(
            self.ctx.handle, self.arena._h, n, arr(*[q._h for q in s.qls]), arr(*[x.buffer() for x in s._xs]),
            int(s.x_dtype), s.M, arr(*[y.buffer() for y in self._ys]), int(s.y_dtype)), self.ctx.handle)
        self.arena.wait()   # the logits (and everything before them) are complete on this rank after the step

    def capture(self) -> Graph:
        g = Graph(self.ctx)
        with g:
            self.step()
        self.graph = g
        return g

    def step_greedy(self) -> None:
        """Every Linear but the LM head pushed; the LM head stays local ([M, vocab / world] on this rank) and only the
        per-rank arg-max candidates are exchanged: every rank ends with the M greedy tokens."""
        s = self.stack
        n = len(s.qls) - 1
        arr = C.c_void_p * n
        check(lib().rusty_cuda_qlinear_forward_pushed_batch(
            self.ctx.handle, self.arena._h, n, arr(*[q._h for q in s.qls[:n]]), arr(*[x.buffer() for x in s._xs[:n]]),
            int(s.x_dtype), s.M, arr(*[y.buffer() for y in self._ys[:n]]), int(s.y_dtype)), self.ctx.handle)
        check(lib().rusty_cuda_qlinear_forward(self.ctx.handle, s.qls[n]._h, s._xs[n].buffer(), int(s.x_dtype), s.M,
                                               s.logits.buffer(), int(s.y_dtype)), self.ctx.handle)
        argmax_rows_sharded(self.ctx, self.arena, s.logits, self._table, self.tokens)

    def capture_greedy(self) -> Graph:
        g = Graph(self.ctx)
        with g:
            self.step_greedy()
        self.greedy_graph = g
        return g

    def replay(self) -> None:
        self.graph.launch()

    def plans(self):
        return self.stack.plans()

    def close(self) -> None:
        self.ctx.sync()
        if self.stack.world > 1:
            self._dist.barrier()  # every rank has stopped pushing before any arena goes away
        self.full_outputs.clear()
        self._ys = []
        self.arena.destroy()
