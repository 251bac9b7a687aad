"""GPU tests of the output-feature sharded forward (NCCL all-gather through the C ABI).  With one GPU the
communicator has a single rank; with two or more the same check runs on two ranks in child processes and the
sharded result must equal the single-GPU result bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_RANK_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
sys.path.insert(0, os.path.join({root!r}, "tests"))
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")                       # plumbing for the unique id only; the data path is NCCL in the library
import rusty_b200
from rusty_b200 import DType, QLinear, UnifiedTensor
from rusty_b200.shard import Comm, forward_sharded, shard_rows
from rusty_b200.workloads import sym_row_linear
from parity import rel_err
ctx = rusty_b200.CudaContext(rank)
eng = rusty_b200.ComputeEngine(ctx)
ids = [Comm.unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
comm = Comm(ctx, world, rank, ids[0])
ok = True
for (M, K, N) in [(1, 1024, 512), (32, 4096, 2048), (256, 512, 1024)]:
    x, q, s = sym_row_linear(M + N, M, K, N)
    rows = shard_rows(N, world, rank)
    shard = QLinear.from_host(ctx, q[rows], s[rows])
    full = QLinear.from_host(ctx, q, s)
    xt = UnifiedTensor.new(ctx, x, [M, K])
    ws = UnifiedTensor.empty(ctx, [M, N])
    y = UnifiedTensor.new(ctx, np.full(M * N, np.nan, np.float32), [M, N])
    forward_sharded(ctx, comm, shard, xt, M, ws, y)
    y1 = UnifiedTensor.empty(ctx, [M, N])
    eng.qlinear(ctx, xt, full, y1)
    a, b = y.to_vec(ctx), y1.to_vec(ctx)
    comm.check()
    same_kernel = shard.plan(M) == full.plan(M)
    ok = ok and (np.array_equal(a.view(np.uint32), b.view(np.uint32)) if same_kernel else rel_err(a, b) <= 1e-5)
sys.stdout.write("rank %d %s\n" % (rank, "ok" if ok else "MISMATCH")); sys.stdout.flush()
comm.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


# The same check for the exchange by peer stores: every rank's kernel writes its columns into every rank's y.
# The cases cover the kernel with the fused exchange (5 <= M, several 64-row passes included), the kernels followed
# by the copy kernel (M = 1, bf16 prefill) and outputs narrower than a 16-byte vector; each arena buffer is reused
# on alternate operations, as a layer stack does.
_PUSH_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
sys.path.insert(0, os.path.join({root!r}, "tests"))
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")                       # host channel for the IPC handles only
import rusty_b200
from rusty_b200 import DType, QLinear, UnifiedTensor, capi
from rusty_b200.shard import Arena, arena_layout, forward_pushed, shard_rows
from rusty_b200.workloads import sym_row_linear
from rusty_b200.backend import bf16_bits_to_f32
from parity import rel_err
ctx = rusty_b200.CudaContext(rank)
eng = rusty_b200.ComputeEngine(ctx)
cases = [(32, 4096, 2048, DType.FP32), (1, 1024, 512, DType.FP32), (256, 512, 1024, DType.FP32),
         (128, 1024, 768, DType.BF16), (3, 256, 6 * world, DType.FP32), (32, 4096, 2048, DType.FP32),
         (2, 1024, 512, "native"), (5, 2048, 1024, "native")]   # native: the reference's affine [in,out] format
sizes = [(i % 2, max(M * N * 4 for j, (M, K, N, dt) in enumerate(cases) if j % 2 == i % 2)) for i in range(len(cases))]
offsets, total = arena_layout(sizes)
arena = Arena(ctx, total, world, rank)
arena.connect(dist)
ok = True
pending = []
for i, (M, K, N, dt) in enumerate(cases):
    x, q, s = sym_row_linear(M + N + i, M, K, N)
    rows = shard_rows(N, world, rank)
    if dt == "native":
        # u8 [K, N], one (scale, bias) per 64 consecutive outputs of an input row; a rank's shard is whole groups
        dt = DType.FP32
        rng = np.random.default_rng(i)
        ukn = (np.ascontiguousarray(q.T).astype(np.int16) + 128).astype(np.uint8)
        sg = rng.uniform(0.001, 0.02, size=(K, N // 64)).astype(np.float32)
        bg = (-128.0 * sg + rng.uniform(-0.05, 0.05, size=sg.shape)).astype(np.float32)
        g = slice(rows.start // 64, rows.stop // 64)
        shard = QLinear.from_host(ctx, np.ascontiguousarray(ukn[:, rows]), np.ascontiguousarray(sg[:, g]), np.ascontiguousarray(bg[:, g]), layout=capi.LAYOUT_KN)
        full = QLinear.from_host(ctx, ukn, sg, bg, layout=capi.LAYOUT_KN)
        assert shard.plan(M) == "gemv_mma"
    else:
        shard = QLinear.from_host(ctx, q[rows], s[rows])
        full = QLinear.from_host(ctx, q, s)
    xt = UnifiedTensor.from_bf16(ctx, x, [M, K]) if dt == DType.BF16 else UnifiedTensor.new(ctx, x, [M, K])
    y = arena.tensor(offsets[i % 2], [M, N], dt)
    forward_pushed(ctx, arena, shard, xt, M, y)
    y1 = UnifiedTensor.empty_with_dtype(ctx, [M, N], dt)
    eng.qlinear(ctx, xt, full, y1)
    pending.append((y, y1, shard.plan(M, dt, dt) == full.plan(M, dt, dt), dt, (shard, full, xt)))
    if i % 2 == 1 or i == len(cases) - 1:
        # results of the last two operations live in the two buffers: wait for the peers' columns, then compare
        arena.wait()
        for (ya, yb, same_kernel, d, _keep) in pending:
            a, b = ya.to_bytes(ctx), yb.to_bytes(ctx)
            if d == DType.BF16:
                fa, fb = bf16_bits_to_f32(a.view(np.uint16)), bf16_bits_to_f32(b.view(np.uint16))
                ok = ok and rel_err(fa, fb) <= 1e-2
            elif same_kernel:
                ok = ok and np.array_equal(a, b)
            else:
                ok = ok and rel_err(a.view(np.float32), b.view(np.float32)) <= 1e-5
        pending = []
        ctx.sync()
        dist.barrier()   # the comparison read both buffers: nobody overwrites them before everybody is done
sys.stdout.write("rank %d %s\n" % (rank, "ok" if ok else "MISMATCH")); sys.stdout.flush()
ctx.sync(); dist.barrier()
arena.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''

# A rank that never pushes: the others' bounded wait runs out, the next sync reports Timeout and the context
# keeps working.  The absent rank is idle (no kernel in flight); nothing faults.
_TIMEOUT_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
import rusty_b200
from rusty_b200 import DType, QLinear, UnifiedTensor
from rusty_b200.capi import BackendError
from rusty_b200.shard import Arena, forward_pushed, shard_rows
from rusty_b200.workloads import sym_row_linear
ctx = rusty_b200.CudaContext(rank)
eng = rusty_b200.ComputeEngine(ctx)
M, K, N = 32, 1024, 512
arena = Arena(ctx, M * N * 4, world, rank)
arena.connect(dist)
x, q, s = sym_row_linear(3, M, K, N)
rows = shard_rows(N, world, rank)
shard = QLinear.from_host(ctx, q[rows], s[rows])
xt = UnifiedTensor.new(ctx, x, [M, K])
y = arena.tensor(0, [M, N], DType.FP32)
ok = True
if rank == 0:
    forward_pushed(ctx, arena, shard, xt, M, y)   # rank 1 never answers
    arena.wait()
    try:
        ctx.sync()
        ok = False
    except BackendError as e:
        ok = e.kind == "Timeout"
    # the context still works
    full = QLinear.from_host(ctx, q, s)
    y1 = UnifiedTensor.empty(ctx, [M, N])
    eng.qlinear(ctx, xt, full, y1)
    ctx.sync()
    ok = ok and bool(np.isfinite(y1.to_vec(ctx)).all())
dist.barrier()
sys.stdout.write("rank %d %s\n" % (rank, "ok" if ok else "FAILED")); sys.stdout.flush()
ctx.sync(); dist.barrier()
arena.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


# Greedy token over column shards of the logits: only candidates travel.
_ARGMAX_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
import rusty_b200
from rusty_b200 import DType, UnifiedTensor
from rusty_b200.shard import Arena, argmax_rows_sharded
ctx = rusty_b200.CudaContext(rank)
M, N = 32, 4096 * world
Nl = N // world
arena = Arena(ctx, world * M * 8, world, rank)
arena.connect(dist)
table = arena.tensor(0, [world * M * 8], DType.U8)
ok = True
for step in range(3):
    logits = np.random.default_rng(100 + step).standard_normal((M, N)).astype(np.float32)
    logits[0, [5, N - 3]] = 50.0        # equal maxima in the first and the last shard: the last wins
    logits[1, :] = np.nan               # no candidate anywhere
    logits[2, 17] = 60.0                # the winner lives in rank 0's columns
    shard = UnifiedTensor.new(ctx, np.ascontiguousarray(logits[:, rank * Nl:(rank + 1) * Nl]), [M, Nl])
    idx = UnifiedTensor.from_bytes_with_dtype(ctx, np.full(M, 0xFFFFFFFF, np.uint32), [M * 4], DType.U8)
    argmax_rows_sharded(ctx, arena, shard, table, idx)
    got = idx.to_bytes(ctx).view(np.uint32)
    want = np.array([0 if np.isnan(r).all() else (N - 1 - int(np.nanargmax(r[::-1]))) for r in logits], np.uint32)
    ok = ok and np.array_equal(got, want) and got[0] == N - 3 and got[1] == 0 and got[2] == 17
sys.stdout.write("rank %d %s\n" % (rank, "ok" if ok else "MISMATCH")); sys.stdout.flush()
ctx.sync(); dist.barrier()
arena.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


# The k largest logits over column shards: k (value, index) pairs per row and rank travel; every rank ends with the
# winners of the whole row, which must equal the single-device kernel's answer on the whole logits.
_TOPK_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
import rusty_b200
from rusty_b200 import DType, UnifiedTensor
from rusty_b200.shard import Arena, top_k_rows_sharded
ctx = rusty_b200.CudaContext(rank)
eng = rusty_b200.ComputeEngine(ctx)
M, N, k = 40, 4096 * world, 50
Nl = N // world
arena = Arena(ctx, world * M * k * 8, world, rank)
arena.connect(dist)
table = arena.tensor(0, [world * M * k * 8], DType.U8)
ok = True
for step in range(3):
    logits = np.random.default_rng(200 + step).standard_normal((M, N)).astype(np.float32)
    logits[0] = np.round(logits[0] * 3)      # ties across the shards: ascending index among equals
    logits[1, :] = np.nan                    # no candidate anywhere
    logits[2, Nl:] = -2e9                    # every winner lives in rank 0's columns
    shard = UnifiedTensor.new(ctx, np.ascontiguousarray(logits[:, rank * Nl:(rank + 1) * Nl]), [M, Nl])
    idx = UnifiedTensor.from_bytes_with_dtype(ctx, np.full(M * k, 0xFFFFFFFF, np.uint32), [M * k * 4], DType.U8)
    val = UnifiedTensor.new(ctx, np.full(M * k, np.nan, np.float32), [M, k])
    top_k_rows_sharded(ctx, arena, shard, k, table, idx, val)
    whole = UnifiedTensor.new(ctx, logits, [M, N])
    idx1 = UnifiedTensor.from_bytes_with_dtype(ctx, np.full(M * k, 0xFFFFFFFF, np.uint32), [M * k * 4], DType.U8)
    val1 = UnifiedTensor.new(ctx, np.full(M * k, np.nan, np.float32), [M, k])
    eng.top_k(ctx, whole, idx1, k, out_val=val1)
    a, b = idx.to_bytes(ctx).view(np.uint32), idx1.to_bytes(ctx).view(np.uint32)
    ok = ok and np.array_equal(a, b) and np.array_equal(val.to_vec(ctx).view(np.uint32), val1.to_vec(ctx).view(np.uint32))
    ok = ok and bool(np.all(a.reshape(M, k)[1] == 0)) and bool(np.all(a.reshape(M, k)[2] < Nl))
sys.stdout.write("rank %d %s\n" % (rank, "ok" if ok else "MISMATCH")); sys.stdout.flush()
ctx.sync(); dist.barrier()
arena.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


def _run(world: int, tmp_path, script_text: str = None, extra_env=None):
    script = tmp_path / "rank.py"
    script.write_text((script_text or _RANK_SCRIPT).format(root=ROOT))
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == world, r.stdout   # lines of two ranks may interleave


def test_single_rank_communicator(tmp_path):
    _run(1, tmp_path)


def test_two_ranks_match_single_gpu_bit_for_bit(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path)


def test_pushed_single_rank(tmp_path):
    _run(1, tmp_path, _PUSH_SCRIPT)


def test_pushed_two_ranks_match_single_gpu_bit_for_bit(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path, _PUSH_SCRIPT)


def test_pushed_unfused_copy_kernel_two_ranks(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path, _PUSH_SCRIPT, {"RUSTY_PUSH_UNFUSED": "1"})


def test_absent_rank_is_reported_as_timeout(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path, _TIMEOUT_SCRIPT, {"RUSTY_PEER_WAIT_MS": "300"})


def test_sharded_argmax_single_rank(tmp_path):
    _run(1, tmp_path, _ARGMAX_SCRIPT)


def test_sharded_argmax_two_ranks(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path, _ARGMAX_SCRIPT)


def test_sharded_top_k_single_rank(tmp_path):
    _run(1, tmp_path, _TOPK_SCRIPT)


def test_sharded_top_k_two_ranks(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path, _TOPK_SCRIPT)
