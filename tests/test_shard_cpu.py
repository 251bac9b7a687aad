"""world_size-2 test of the sharding rule on CPU ranks (gloo): each rank applies
the oracle to its shard of output features (rows of [out,in] weights; columns of the reference's own [in,out] affine
format, taken through the loader), the pieces are all-gathered and reassembled, and the result must equal the unsharded
oracle bit for bit."""
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
        # a pair-interleaved gate|up weight: a rank's rows are whole (gate, up) pairs, so silu(gate) * up of its shard
        # is a block of columns of the whole [M, N/2] result
        from rusty_b200.backend import interleave_pairs
        F = N // 2
        wp, sp = interleave_pairs(w[:F], w[F:]), interleave_pairs(s[:F], s[F:])
        act_local = O.swiglu_pairs(O.qlinear_rowscale(x, wp[rows], sp[rows]))
        pieces = [torch.empty(M, F // world, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(pieces, torch.from_numpy(act_local))
        act = assemble([p.numpy() for p in pieces])
        act_ref = O.mul(O.silu(O.qlinear_rowscale(x, w[:F], s[:F])), O.qlinear_rowscale(x, w[F:], s[F:]))
        ok = ok and act.shape == act_ref.shape and np.array_equal(act.view(np.uint32), act_ref.view(np.uint32))
        # the reference's own format through the loader: u8 [in,out] with a (scale, bias) per 64 consecutive outputs of an
        # input row; a rank's shard is a column block of whole groups and yields a block of columns of y
        import tempfile
        from rusty_b200 import capi
        from rusty_b200.loader import WeightsContext, save_file
        Kn, Nn = 128, 256
        rng = np.random.default_rng(7)
        ukn = rng.integers(0, 256, size=(Kn, Nn), dtype=np.uint8)
        sg = rng.uniform(0.001, 0.02, size=Kn * Nn // 64).astype(np.float32)
        bg = (-128.0 * sg + rng.uniform(-0.05, 0.05, size=sg.size)).astype(np.float32)
        xn = rng.standard_normal((M, Kn), dtype=np.float32)
        path = os.path.join(tempfile.gettempdir(), "rusty_shard_cpu_%d_%d.safetensors" % (port, rank))
        save_file(path, {"w.weight": ukn, "w.scales": sg, "w.biases": bg})
        wc = WeightsContext()
        wc.load_file(path)
        q2, s2, b2 = wc.quantized_shard("w", capi.LAYOUT_KN, rank, world)
        os.unlink(path)
        yn_local = O.qlinear_affine(xn, q2, s2, b2, q2.shape, layout_nk=False)
        pieces = [torch.empty(M, Nn // world, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(pieces, torch.from_numpy(np.ascontiguousarray(yn_local)))
        yn = assemble([p.numpy() for p in pieces])
        yn_ref = O.qlinear_affine(xn, ukn, sg, bg, ukn.shape, layout_nk=False)
        ok = ok and yn.shape == yn_ref.shape and np.array_equal(yn.view(np.uint32), yn_ref.view(np.uint32))
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


def test_arena_layout_is_the_same_on_every_rank():
    from rusty_b200.shard import ARENA_ALIGN, arena_layout
    sizes = [(6144, 32 * 6144 * 4), (4096, 32 * 4096 * 4), (14336, 32 * 14336 * 4), (4096, 32 * 4096 * 4), (-1, 100)]
    offsets, total = arena_layout(sizes)
    assert offsets == {6144: 0, 4096: 786432, 14336: 786432 + 524288, -1: 786432 + 524288 + 1835008}
    assert all(o % ARENA_ALIGN == 0 for o in offsets.values()) and total == offsets[-1] + 256
    import pytest
    with pytest.raises(ValueError):
        arena_layout([(1, 10), (1, 20)])


def test_interleave_pairs():
    from rusty_b200.backend import interleave_pairs
    a, b = np.arange(6).reshape(3, 2), 10 + np.arange(6).reshape(3, 2)
    assert interleave_pairs(a, b).tolist() == [[0, 1], [10, 11], [2, 3], [12, 13], [4, 5], [14, 15]]


def test_shard_rows_rule():
    from rusty_b200.shard import shard_rows
    assert shard_rows(1024, 8, 0) == slice(0, 128) and shard_rows(1024, 8, 7) == slice(896, 1024)
    import pytest
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
