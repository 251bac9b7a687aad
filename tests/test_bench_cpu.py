"""Host-side logic of bench.py that needs no GPU: the workload table, the config both arms print, the CPU sample."""
import importlib.util
import os
import types

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_workload_table_is_consistent():
    b = _bench()
    from rusty_b200.workloads import STACKS
    assert b.DEFAULT_WORKLOAD in b.WORKLOADS
    for name in b.WORKLOADS:
        stack, M, desc, act = b.workload(name)
        assert stack in STACKS and M >= 1 and desc and act in ("f32", "bf16")
        assert b.metric_name(M) == ("decode_tokens_per_s" if "decode" in name else "prefill_tokens_per_s")
    # the headline is the batch-32 decode of the Llama-3-8B shapes, f32 in and out
    assert b.workload(b.DEFAULT_WORKLOAD)[:2] == ("llama3-8b", 32) and b.workload(b.DEFAULT_WORKLOAD)[3] == "f32"


def test_native_format_workload_is_flagged_and_described():
    b = _bench()
    assert b.workload_is_native("llama7b-decode1-native") and not b.workload_is_native("llama7b-decode1")
    assert [n for n in b.WORKLOADS if b.workload_is_native(n)] == ["llama7b-decode1-native"]
    args = types.SimpleNamespace(workload="llama7b-decode1-native", layers=None)
    stack, M, desc, act = b.workload(args.workload)
    cfg = b.workload_config(args, M, desc)
    assert (stack, M, act) == ("llama7b", 1, "f32") and "[in,out]" in cfg["weights"] and "64 consecutive outputs" in cfg["weights"]
    plain = b.workload_config(types.SimpleNamespace(workload="llama7b-decode1", layers=None), 1, "d")
    assert "[out,in]" in plain["weights"] and cfg["linears_per_step"] == plain["linears_per_step"] == 129


def test_both_arms_print_the_same_config():
    b = _bench()
    args = types.SimpleNamespace(workload=b.DEFAULT_WORKLOAD, layers=None)
    stack, M, desc, act = b.workload(args.workload)
    c1, c2 = b.workload_config(args, M, desc), b.workload_config(args, M, desc)
    assert c1 == c2 and c1["workload"] == args.workload and c1["batch_rows"] == 32 and c1["linears_per_step"] == 129
    assert "model" not in c1


def test_cpu_sample_scales_by_weight_bytes_and_rows(oracle):
    b = _bench()
    cs = b.CpuSample("llama7b", 1)
    assert cs.M == 1 and cs.threads >= 1
    # one layer of 32: a sample that took t seconds stands for t * total / sample seconds of the whole stack
    t = 0.5
    assert np.isclose(cs.tokens_per_s(t), 1.0 / (t * cs.total_weights / cs.sample_weights))
    big = b.CpuSample.MAX_ROWS
    assert big == 128   # prefill workloads are sampled on 128 rows
