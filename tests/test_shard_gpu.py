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
print("rank", rank, "ok" if ok else "MISMATCH", flush=True)
comm.destroy(); ctx.destroy(); dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


def _run(world: int, tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT.format(root=ROOT))
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok") == world, r.stdout


def test_single_rank_communicator(tmp_path):
    _run(1, tmp_path)


def test_two_ranks_match_single_gpu_bit_for_bit(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2, tmp_path)
