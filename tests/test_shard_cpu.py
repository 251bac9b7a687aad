"""world_size-2 test of the sharding rule on CPU ranks (gloo): each rank applies
the oracle to its row shard, the pieces are all-gathered and reassembled, and
the result must equal the unsharded oracle bit for bit."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from rusty_b200.shard import assemble, shard_rows
        from rusty_b200.workloads import sym_row_linear
        M, K, N = 3, 256, 96
        x, w, s = sym_row_linear(42, M, K, N)
        rows = shard_rows(N, world, rank)
        y_local = O.qlinear_rowscale(x, w[rows], s[rows])
        pieces = [torch.empty(M, N // world, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(pieces, torch.from_numpy(y_local))
        y = assemble([p.numpy() for p in pieces])
        y_ref = O.qlinear_rowscale(x, w, s)
        ok = y.shape == y_ref.shape and np.array_equal(y.view(np.uint32), y_ref.view(np.uint32))
        # the timing protocol of the bench: max over ranks
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        q.put((rank, bool(ok), float(t.item())))
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reassemble_bit_exactly():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] for r in results)
    assert all(r[2] == 2.0 for r in results)


def test_shard_rows_rule():
    from rusty_b200.shard import shard_rows
    assert shard_rows(1024, 8, 0) == slice(0, 128) and shard_rows(1024, 8, 7) == slice(896, 1024)
    import pytest
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
