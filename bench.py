#!/usr/bin/env python3
"""Benchmark of the quantised-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one pass of the Llama-shaped stack of int8 Linears (every q/k/v/o,
gate/up/down and the LM head once) over one batch of synthetic activations.
Prints ONE JSON line (rank 0).  Metric: decode tokens/s; the same line carries
the dominant kernel's HBM roofline, the single-Linear GEMV GB/s and prefill GEMM
TFLOP/s figures, an end-to-end number with host<->device copies in the timed
region, the sampled clocks and a CPU baseline.

Under torchrun (N > 1) every Linear is sharded by output features across the
ranks and its output all-gathered; total work is fixed ("strong" scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (stack, activation rows M, description[, activation dtype: "f32" (default) or "bf16"])
    "llama3-8b-decode32": ("llama3-8b", 32, "Llama-3-8B-shaped GQA linear stack, random int8 weights, batch-32 decode"),
    "llama7b-decode1": ("llama7b", 1, "Llama-7B-shaped linear stack, random int8 weights, batch-1 decode"),
    "llama2-70b-decode64": ("llama2-70b", 64, "Llama-2-70B-shaped linear stack, random int8 weights, batch-64 decode"),
    # the same batch-1 decode with every weight in the reference's own quantised format (fifth field: "native")
    "llama7b-decode1-native": ("llama7b", 1, "Llama-7B-shaped linear stack, random u8 weights in the reference's own format "
                               "([in,out], f32 scale and bias per 64 consecutive outputs of an input row), batch-1 decode", "f32", "native"),
    # prefill: every Linear at M = all prompt tokens, bf16 activations in and out, fp32 accumulate (tensor-core bound)
    "llama3-8b-prefill2048": ("llama3-8b", 2048, "Llama-3-8B-shaped GQA linear stack, random int8 weights, 2048-token prefill", "bf16"),
    "llama2-70b-prefill8192": ("llama2-70b", 8192, "Llama-2-70B-shaped linear stack, random int8 weights, batch 4 x 2048-token prefill", "bf16"),
}


def workload(name):
    """(stack, M, description, activation dtype) of a workload."""
    w = WORKLOADS[name]
    return w[0], w[1], w[2], (w[3] if len(w) > 3 else "f32")
def workload_is_native(name):
    """Whether the workload's weights are in the reference's own affine [in,out] format."""
    w = WORKLOADS[name]
    return len(w) > 4 and w[4] == "native"
DEFAULT_WORKLOAD = "llama3-8b-decode32"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle reasons sampled DURING the timed region.  Reads only (no setting is changed): NVML from a
    thread every 5 ms (the timed region is tens of milliseconds, too short for nvidia-smi's own loop, whose first
    sample arrives after ~100 ms; a 2 ms period measurably slowed a 2-GPU step whose ranks wait on one another); nvidia-smi is the fall-back when the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = None
        self.p = None
        self.thread = None
        self.stop_flag = False
        self.sm, self.reasons, self.mx = [], set(), None
        self.period_s = float(os.environ.get("RUSTY_BENCH_SAMPLE_MS", "5")) * 1e-3

    def _nvml_loop(self, nv, h):
        bits = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                r = int(get_reasons(h))
                for name, bit in bits.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period_s)

    def prepare(self):
        """Everything slow (loading and initialising NVML), done ahead of the timed region."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.idx)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._nv = (nv, h)
        except Exception:
            self._nv = None

    def start(self):
        if getattr(self, "_nv", "unset") == "unset":
            self.prepare()
        if self._nv is not None:
            import threading
            self.thread = threading.Thread(target=self._nvml_loop, args=self._nv, daemon=True)
            self.thread.start()
            return
        try:
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            if self.sm:
                out.update(sm_mhz=statistics.median(self.sm), sm_max_mhz=self.mx, reasons=sorted(self.reasons),
                           samples=len(self.sm), source="nvml")
            return out
        if self.p is None:
            return out
        try:
            self.p.terminate()
            self.p.wait(timeout=5)
        except Exception:
            pass
        try:
            self.f.flush()
            rows = [r.strip().split(", ") for r in open(self.f.name) if r.strip()]
            os.unlink(self.f.name)
        except Exception:
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for nm, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(nm)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       source="nvidia-smi")
        return out


# ----------------------------------------------------------------------------
# CPU arm: the oracle's threaded restatement of the reference arithmetic.
# ----------------------------------------------------------------------------
class CpuSample:
    """ONE layer (q,k,v,o,gate,up,down at batch M) of the stack on the host cores.
    two_step = the reference's own per-forward work: an f32 matmul over weights
    dequantised beforehand (untimed, as at its load time); fused = int8 read +
    dequant inside the dot product."""

    MAX_ROWS = 128   # a prefill workload is sampled on this many of its rows (time is linear in rows)

    def __init__(self, stack_name: str, M: int):
        from oracle import oracle as O
        from rusty_b200.workloads import STACKS
        self.O = O
        self.M_full = M
        M = min(M, self.MAX_ROWS)
        self.M = M
        shape = STACKS[stack_name]
        rng = np.random.default_rng(0)
        self.per_layer = shape.per_layer()
        self.ws = {}
        for _p, n, k in self.per_layer:
            if (n, k) not in self.ws:
                q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
                s = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
                self.ws[(n, k)] = (q, s, O.dequantize_rowscale(q, s))
        self.xs = {k: rng.standard_normal((M, k), dtype=np.float32) for _p, _n, k in self.per_layer}
        self.sample_weights = sum(n * k for _p, n, k in self.per_layer)
        self.total_weights = shape.weight_bytes()
        # every core this process may run on, whatever OMP_NUM_THREADS says (torchrun exports 1)
        try:
            cores = len(os.sched_getaffinity(0))
        except AttributeError:
            cores = os.cpu_count() or 1
        self.threads = O.set_num_threads(cores)

    def two_step(self) -> float:
        t0 = time.perf_counter()
        for _p, n, k in self.per_layer:
            self.O.time_matmul_bt_mt(self.xs[k], self.ws[(n, k)][2], simd=True)
        return time.perf_counter() - t0

    def fused(self) -> float:
        t0 = time.perf_counter()
        for _p, n, k in self.per_layer:
            self.O.qlinear_rowscale_fused_mt(self.xs[k], self.ws[(n, k)][0], self.ws[(n, k)][1], simd=True)
        return time.perf_counter() - t0

    def tokens_per_s(self, seconds_per_sample: float) -> float:
        return self.M / (seconds_per_sample * self.total_weights / self.sample_weights)

    def describe(self) -> str:
        rows = "" if self.M == self.M_full else " (%d of the workload's %d rows; time is linear in rows)" % (self.M, self.M_full)
        return ("one layer (q,k,v,o,gate,up,down) at batch %d%s per step, scaled to the whole stack by weight bytes "
                "(%d / %d); f32 matmul over pre-dequantised weights = the reference's per-forward work"
                % (self.M, rows, self.total_weights, self.sample_weights))


def workload_config(args, M: int, desc: str) -> dict:
    """The `config` object both arms print: what is computed, not how."""
    stack_name, _m, _d, act = workload(args.workload)
    from rusty_b200.workloads import STACKS
    shape = STACKS[stack_name]
    layers = shape.layers if args.layers is None else args.layers
    return {"workload": args.workload, "desc": desc, "batch_rows": M, "layers": layers,
            "linears_per_step": 4 * layers + 1,
            "weights": ("u8 [in,out], f32 scale and bias per 64 consecutive outputs of an input row (the reference's own format); "
                        "q|k|v and gate|up run as one Linear each") if workload_is_native(args.workload)
                       else "int8 [out,in], f32 scale per output row; q|k|v and gate|up run as one Linear each",
            "activations": "%s in, %s out, fp32 accumulate" % (act, act),
            "l2": "inputs larger than L2: every step streams all %.2f GB of weights, each layer from its own buffer"
                  % (sum(n * k for _p, n, k in shape.per_layer()) * layers / 1e9 + shape.vocab * shape.d / 1e9)}


def metric_name(M: int) -> str:
    return "decode_tokens_per_s" if M <= 64 else "prefill_tokens_per_s"


def run_reference(args, rank: int):
    """--impl reference: the reference's own arithmetic for the path on the host
    cores (the oracle port; the Rust + WGSL original cannot be built or run on a
    box without a Rust toolchain and a graphics stack).  One step = ONE layer of
    the stack (a bounded sample); the per-step time of the whole stack is that
    sample scaled by weight bytes, and both are printed."""
    if rank != 0:
        return
    stack_name, M, desc, act = workload(args.workload)
    cs = CpuSample(stack_name, M)
    for _ in range(args.warmup):
        cs.two_step()
    times = [cs.two_step() for _ in range(args.steps)]
    t_sample = sum(times) / len(times)
    val = cs.tokens_per_s(t_sample)
    step_s = M / val
    line = {
        "impl": "reference", "metric": metric_name(M), "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, M, desc),
        "sample_ms_measured": t_sample * 1e3,
        "ms_per_step_is": "extrapolated: measured sample (one layer) x total weight bytes / sample weight bytes",
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cs.threads, "kind": "port", "sample": cs.describe()},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# single-Linear figures (rank 0, N = 1): GEMV GB/s and GEMM TFLOP/s
# ----------------------------------------------------------------------------
def bench_single_linear(ctx, eng, M, K, N, x_dtype, y_dtype, iters, warm, l2_bytes=126 * 2**20, native=False):
    """Average device time per launch over `iters` launches that rotate through
    enough distinct weight copies to exceed L2 (so every launch streams HBM).  `native`: the weight in the reference's own
    quantised format (u8 [in,out], one f32 scale and bias per 64 consecutive output features of an input row,
    rusty-loader/src/lib.rs:155-218) instead of int8 [out,in] with one scale per output row."""
    from rusty_b200 import QLinear, UnifiedTensor, capi
    from rusty_b200.backend import Event
    from rusty_b200.workloads import affine_g64_from_sym, sym_row_linear
    x, q, s = sym_row_linear(0, M, K, N)
    copies = max(2, int(np.ceil(1.5 * l2_bytes / (N * K))) + 1)
    if native:
        u, sg, bg = affine_g64_from_sym(np.ascontiguousarray(q.T), 0)
        qls = [QLinear.from_host(ctx, u, sg, bg, layout=capi.LAYOUT_KN) for _ in range(copies)]
    else:
        qls = [QLinear.from_host(ctx, q, s) for _ in range(copies)]
    from rusty_b200 import DType
    xt = UnifiedTensor.from_bf16(ctx, x, [M, K]) if x_dtype == DType.BF16 else UnifiedTensor.new(ctx, x, [M, K])
    y = UnifiedTensor.empty_with_dtype(ctx, [M, N], y_dtype)
    from rusty_b200.backend import Graph
    for i in range(warm):
        eng.qlinear(ctx, xt, qls[i % copies], y)
    ctx.sync()
    g = Graph(ctx)          # the launches are replayed from a graph so host call overhead is not what is timed
    with g:
        for i in range(iters):
            eng.qlinear(ctx, xt, qls[i % copies], y)
    g.launch()
    ctx.sync()
    e0, e1 = Event(ctx), Event(ctx)
    e0.record()
    g.launch()
    e1.record()
    ms = e0.elapsed_ms(e1) / iters
    plan = qls[0].plan(M, x_dtype, y_dtype)
    alg_bytes = N * K + (N * K // 64 * 8 if native else N * 4) + M * K * x_dtype.size_bytes() + M * N * y_dtype.size_bytes()
    del qls
    return {"M": M, "K": K, "N": N, "kernel": plan, "us_per_launch": ms * 1e3, "algorithmic_bytes": alg_bytes,
            "gbs": alg_bytes / (ms * 1e-3) / 1e9, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "weight_copies": copies}


def run_stack(ctx, dist, args, stack_name, M, rank, world, local_rank, steps, warmup, clocks=False, e2e_logits=True,
              norms=False, act="f32", native=False):
    """One workload on this process group: the device-timed step (inputs resident in HBM), the end-to-end step (host
    activations in, rank 0 reads the logits back) and the greedy step (the token chosen on the device).  Returns the
    max-over-ranks figures; builds and frees its own weights."""
    from rusty_b200 import DType
    from rusty_b200.backend import Event, PinnedArray, bf16_bits_to_f32, download_async, f32_to_bf16_bits, upload_async
    from rusty_b200.stack import LinearStack
    from rusty_b200.workloads import STACKS
    shape = STACKS[stack_name]
    dt = DType.BF16 if act == "bf16" else DType.FP32
    npdt = np.uint16 if act == "bf16" else np.float32
    stack = LinearStack(ctx, shape, M, dt, dt, seed=0, rank=rank, world=world, layers=args.layers,
                        swiglu=not args.no_swiglu, norms=norms, native=native)
    if world > 1 and args.exchange != "none":
        from rusty_b200.shard import PushedStack, ShardedStack
        runner = PushedStack(stack, dist) if args.exchange == "push" else ShardedStack(stack, dist)
    else:
        runner = stack    # "none": every rank runs its shard and nothing is exchanged (a lower bound, not a result)
    runner.capture()

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-timed region: inputs resident in HBM ----
    sampler = ClockSampler(local_rank) if (clocks and rank == 0) else None
    if sampler:
        sampler.prepare()   # NVML start-up takes tens of milliseconds: before the barrier, or the other ranks' clocks
                            # would count the wait for rank 0 in their first step
    for _ in range(warmup - 1):
        runner.replay()
    barrier()
    runner.replay()         # the last warm-up step runs after the barrier: its exchanges line the GPUs up
    if sampler:
        sampler.start()
    l0 = ctx.launch_count()
    e0, e1 = Event(ctx), Event(ctx)
    e0.record()
    for _ in range(steps):
        runner.replay()
    e1.record()
    ms_total = e0.elapsed_ms(e1)
    barrier()
    launches = ctx.launch_count() - l0
    ms_step = max_over_ranks(ms_total / steps)
    # A box whose NVML calls are slow yields only a sample or two in a 60 ms region: every rank then repeats the same
    # steps, untimed, with the sampler still running, so that the clock figure always rests on a handful of samples
    # of the device under this load; `samples_in_timed_region` says how many fell into the timed steps themselves.
    in_region = len(sampler.sm) if sampler else 0
    few = max_over_ranks(1.0 if (sampler and in_region < 5) else 0.0) > 0.0
    if few:
        for _ in range(3 * steps):   # the same count on every rank: the ranks meet in every Linear
            runner.replay()
        ctx.sync()
        barrier()
    clk = sampler.stop() if sampler else None
    if clk is not None:
        clk["samples_in_timed_region"] = in_region

    # ---- end-to-end: host activations in on every rank, host logits out on rank 0, every step ----
    d_in = shape.d
    x_host = PinnedArray((M, d_in), npdt)
    x_host.array[...] = f32_to_bf16_bits(stack.host_inputs[d_in]) if act == "bf16" else stack.host_inputs[d_in]
    e2e = None
    if e2e_logits:
        logits_t = runner.full_logits() if hasattr(runner, "full_logits") else stack.logits
        # decode reads every row's logits back; prefill only the last token's (the one that is sampled from)
        rows_back = M if M <= 64 else 1
        y_host = PinnedArray((rows_back, logits_t.shape[1]), npdt)
        y_off = (M - rows_back) * int(logits_t.shape[1]) * dt.size_bytes()

        def one():
            upload_async(ctx, stack.inputs[d_in], x_host)
            runner.replay()
            if rank == 0:
                download_async(ctx, logits_t, y_host, y_off)
            ctx.sync()
        for _ in range(2):
            one()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            one()
        e2e_s = max_over_ranks((time.perf_counter() - t0) / steps)
        barrier()
        yh = bf16_bits_to_f32(y_host.array) if act == "bf16" else y_host.array
        finite = bool(np.isfinite(yh).all()) if rank == 0 else True
        e2e = {"value": M / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": x_host.nbytes,
               "d2h_bytes_per_step": y_host.nbytes, "ms_per_step": e2e_s * 1e3, "logits_finite": finite,
               "readback": "rank 0 reads the [%d, vocab] %s logits%s; every rank uploads the [M, d] activations"
                           % (rows_back, act, "" if rows_back == M else " of the last token")}
        y_host.free()

    # ---- the same step ending in one greedy token per row chosen on the device (what a greedy decoder reads back):
    # N > 1 keeps the LM head's logits local and exchanges arg-max candidates instead ----
    greedy = None
    if hasattr(runner, "capture_greedy") and act == "f32":
        runner.capture_greedy()
        tok_host = PinnedArray((M,), np.uint32)
        for _ in range(warmup - 1):
            runner.greedy_graph.launch()
        barrier()
        runner.greedy_graph.launch()
        g0, g1 = Event(ctx), Event(ctx)
        g0.record()
        for _ in range(steps):
            runner.greedy_graph.launch()
        g1.record()
        g_ms = max_over_ranks(g0.elapsed_ms(g1) / steps)
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            upload_async(ctx, stack.inputs[d_in], x_host)
            runner.greedy_graph.launch()
            if rank == 0:
                download_async(ctx, runner.tokens, tok_host)
            ctx.sync()
        g_e2e = max_over_ranks((time.perf_counter() - t0) / steps)
        barrier()
        greedy = {"value": M / (g_ms * 1e-3), "unit": "tokens/s", "ms_per_step": g_ms,
                  "e2e": {"value": M / g_e2e, "unit": "tokens/s", "ms_per_step": g_e2e * 1e3,
                          "h2d_bytes_per_step": x_host.nbytes, "d2h_bytes_per_step": tok_host.nbytes,
                          "readback": "rank 0 reads the M tokens"},
                  "tokens_in_range": bool((tok_host.array < shape.vocab).all())}
        tok_host.free()
    x_host.free()
    out = {"ms_step": ms_step, "launches": int(launches), "clocks": clk, "e2e": e2e, "greedy": greedy,
           "alg_bytes": stack.algorithmic_bytes(), "weight_gb": stack.weight_bytes() / 1e9, "plans": runner.plans(),
           "flops": stack.flops(),
           "swiglu": bool(stack.swiglu)}
    if hasattr(runner, "close"):
        runner.close()
    del runner, stack
    import gc
    gc.collect()
    ctx.pool_clear()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers (for profiling captures only)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-Linear, 70B and CPU legs")
    ap.add_argument("--no-70b", action="store_true", help="skip the llama2-70b-decode64 extra key")
    ap.add_argument("--exchange", default="push", choices=["push", "nccl", "none"],
                    help="N > 1: how a rank's output columns reach the other ranks: stores from the kernel's epilogue "
                         "into every rank's memory (push) or an NCCL all-gather after each Linear (nccl); none = no "
                         "exchange at all, a diagnostic lower bound whose line is not a benchmark result")
    ap.add_argument("--no-swiglu", action="store_true",
                    help="write gate|up as [M, 2*ffn] instead of applying silu(gate)*up in the kernel's epilogue")
    ap.add_argument("--single", default=None, metavar="MxKxN:f32|bf16[-native]",
                    help="run ONE fused linear of this shape --steps times on rotating weight copies and print its "
                         "timing (small case for profiler captures; not the benchmark line)")
    args = ap.parse_args()
    if args.warmup < 3 and args.layers is None:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.single:
        import rusty_b200
        from rusty_b200 import DType
        shape, _, dt = args.single.partition(":")
        M, K, N = (int(v) for v in shape.lower().split("x"))
        native = dt.endswith("-native")   # e.g. 1x4096x4096:f32-native = the reference's own affine [in,out] format
        d = DType.BF16 if dt.startswith("bf16") else DType.FP32
        ctx = rusty_b200.CudaContext(local_rank)
        r = bench_single_linear(ctx, rusty_b200.ComputeEngine(ctx), M, K, N, d, d, max(1, args.steps), max(1, args.warmup), native=native)
        print(json.dumps({"single": args.single, **r}), flush=True)
        return

    stack_name, M, desc, act = workload(args.workload)
    peaks = load_peaks()
    prefill = M > 64
    if prefill and args.steps > 5 and "--steps" not in sys.argv:
        args.steps = 5   # a prefill step is hundreds of milliseconds

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import rusty_b200
    from rusty_b200 import DType
    from rusty_b200.backend import Event, PinnedArray, download_async, upload_async
    from rusty_b200.stack import LinearStack
    from rusty_b200.workloads import STACKS

    ctx = rusty_b200.CudaContext(local_rank)
    eng = rusty_b200.ComputeEngine(ctx)
    shape = STACKS[stack_name]
    native = workload_is_native(args.workload)
    r = run_stack(ctx, dist, args, stack_name, M, rank, world, local_rank, args.steps, args.warmup, clocks=True, act=act, native=native)
    ms_step, launches, clocks, e2e, greedy = r["ms_step"], r["launches"], r["clocks"], r["e2e"], r["greedy"]
    alg_bytes, weight_gb, plans, swiglu = r["alg_bytes"], r["weight_gb"], r["plans"], r["swiglu"]

    value = M / (ms_step * 1e-3)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    if prefill:
        # tensor-core bound: 2*M*N*K flops per Linear over the whole step's device time, against the cuBLAS bf16
        # throughput measured in a seconds-long loop (the step is hundreds of milliseconds of back-to-back GEMMs)
        tfl = r["flops"] / (ms_step * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": tfl, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                    "frac": tfl / peaks["bf16_tflops_sustained"], "traffic": None, "peak_source": peaks["source"] + " (sustained)",
                    "frac_of_burst_peak": tfl / peaks["bf16_tflops"], "flops_per_step_per_gpu": r["flops"],
                    "note": "whole step (all launches of the bf16 tensor-core linear) / device time, per GPU"}
    else:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"],
                    # DRAM bytes per step: dram__bytes_read+write of the fused linear captured with ncu on one Linear of
                    # this stack (32 x 4096 x 14336: 59.44 MB for 61.14 MB algorithmic), scaled to the step by
                    # algorithmic bytes (traffic grows with the weight bytes streamed)
                    "traffic": alg_bytes * (59.44 / 61.14) if M > 4 else None, "peak_source": peaks["source"],
                    "algorithmic_bytes_per_step_per_gpu": alg_bytes,
                    "note": "whole step (all launches of the fused linear kernel) / device time, per GPU"}
    line = {
        "metric": metric_name(M), "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": act, "data": "synthetic",
        "config": workload_config(args, M, desc),
        "impl_detail": {"swiglu_epilogue": swiglu,
                        "parallelism": ("1 GPU" if world == 1 else f"output-feature shards x{world}, " + (
                            "outputs stored into every rank's memory by the kernel epilogue (NVLink peer stores)"
                            if args.exchange == "push" else "NCCL all-gather after each Linear" if args.exchange == "nccl"
                            else "NOTHING EXCHANGED (diagnostic lower bound, not a result)")),
                        "weight_gb_per_gpu_per_step": weight_gb, "kernels": plans},
        "roofline": roofline,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": clocks,
        "greedy": greedy,
    }

    # The block's RMSNorms riding in the Linears that follow them (norm1 -> q|k|v, norm2 + residual -> gate|up, final
    # norm -> lm_head): the same step with 65 norms added, as an extra key.
    if world == 1 and not args.no_extras and args.layers is None and not prefill and not native:
        rn = run_stack(ctx, dist, args, stack_name, M, rank, world, local_rank, args.steps, args.warmup, e2e_logits=False, norms=True)
        line["with_rms_norms"] = {"value": M / (rn["ms_step"] * 1e-3), "unit": "tokens/s", "ms_per_step": rn["ms_step"],
                                  "gpu_launches": rn["launches"],
                                  "note": "RMSNorm applied by the pre-pass of q|k|v, gate|up (with residual add) and lm_head; "
                                          "no norm kernel is launched"}

    # The 70B stack's Linears are four times larger, so output-feature sharding pays there first: the same measurement
    # on llama2-70b-decode64 rides along as an extra key (never the headline).
    if args.workload == DEFAULT_WORKLOAD and not args.no_extras and not args.no_70b and args.layers is None:
        sn, m70, d70, _a = workload("llama2-70b-decode64")
        r70 = run_stack(ctx, dist, args, sn, m70, rank, world, local_rank, max(3, min(args.steps, 10)), 3)
        line["llama2_70b_decode64"] = {
            "workload": "llama2-70b-decode64", "desc": d70, "value": m70 / (r70["ms_step"] * 1e-3), "unit": "tokens/s",
            "ms_per_step": r70["ms_step"], "n_gpus": world,
            "frac_of_hbm_peak_per_gpu": r70["alg_bytes"] / (r70["ms_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "e2e": r70["e2e"], "greedy": r70["greedy"], "gpu_launches": r70["launches"],
            "weight_gb_per_gpu_per_step": r70["weight_gb"]}

    if rank == 0 and world == 1 and not args.no_extras and not prefill:
        # single-Linear figures of the metric: GEMV GB/s, prefill GEMM TFLOP/s
        g1 = bench_single_linear(ctx, eng, 1, 4096, 4096, DType.FP32, DType.FP32, 200, 20)
        g2 = bench_single_linear(ctx, eng, 1, 4096, 11008, DType.BF16, DType.BF16, 200, 20)
        g1["frac_of_hbm_peak"] = g1["gbs"] / peaks["hbm_gbs"]
        g2["frac_of_hbm_peak"] = g2["gbs"] / peaks["hbm_gbs"]
        mm = bench_single_linear(ctx, eng, 512, 4096, 11008, DType.BF16, DType.BF16, 30, 5)
        mm["frac_of_bf16_peak"] = mm["tflops"] / peaks["bf16_tflops"]
        g0 = bench_single_linear(ctx, eng, 1, 4096, 4096, DType.FP32, DType.FP32, 200, 20, native=True)
        g0["frac_of_hbm_peak"] = g0["gbs"] / peaks["hbm_gbs"]
        g0["weights"] = "the reference's own format: u8 [in,out], f32 scale and bias per 64 consecutive outputs of an input row"
        line["gemv"] = {"config0_f32_1x4096x4096": g1, "config1_bf16_1x4096x11008": g2, "config0_native_affine_f32_1x4096x4096": g0}
        line["gemm"] = {"config1_bf16_512x4096x11008": mm, "peak_tflops": peaks["bf16_tflops"]}
        cs = CpuSample(stack_name, M)
        cs.two_step()
        t2 = min(cs.two_step() for _ in range(3))
        tf = min(cs.fused() for _ in range(3))
        line["cpu_baseline"] = {"value": cs.tokens_per_s(t2), "unit": "tokens/s", "cores": cs.threads, "kind": "port",
                                "fused_int8_value": cs.tokens_per_s(tf), "sample": cs.describe()}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
