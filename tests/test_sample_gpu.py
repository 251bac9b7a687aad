"""The step after the LM head: greedy token choice on the device against Sampler::sample with temperature <= 0
(rusty-loader/src/tokenizer.rs:151-158: the last of equal maxima, 0 for an empty row)."""
import numpy as np
import pytest

from rusty_b200 import DType, UnifiedTensor

pytestmark = pytest.mark.gpu


def _run(ctx, engine, logits):
    M, N = logits.shape
    t = UnifiedTensor.new(ctx, logits, [M, N])
    idx = UnifiedTensor.from_bytes_with_dtype(ctx, np.full(M, 0xFFFFFFFF, np.uint32), [M * 4], DType.U8)
    val = UnifiedTensor.new(ctx, np.full(M, np.nan, np.float32), [M])
    engine.argmax_rows(ctx, t, idx, val)
    return idx.to_bytes(ctx).view(np.uint32), val.to_vec(ctx)


@pytest.mark.parametrize("M,N", [(1, 1), (1, 10), (3, 1000), (5, 1025), (32, 128256)])
def test_random_rows(ctx, engine, oracle, M, N):
    logits = np.random.default_rng(M * 31 + N).standard_normal((M, N)).astype(np.float32)
    idx, val = _run(ctx, engine, logits)
    want = np.array([oracle.greedy_sample(r) for r in logits], np.uint32)
    assert np.array_equal(idx, want)
    assert np.array_equal(val, logits[np.arange(M), want])


def test_ties_nan_and_infinities(ctx, engine, oracle):
    N = 5000
    rng = np.random.default_rng(0)
    rows = []
    r = rng.standard_normal(N).astype(np.float32)
    r[[7, 1500, 4999]] = 9.0                      # three equal maxima: the last wins
    rows.append(r)
    r = np.full(N, -np.inf, np.float32)            # all -inf: still "the last maximum"
    rows.append(r)
    r = rng.standard_normal(N).astype(np.float32)
    r[100] = np.nan
    r[200] = np.inf
    rows.append(r)
    rows.append(np.full(N, np.nan, np.float32))    # no candidate at all: 0
    r = np.zeros(N, np.float32)
    r[0] = 1.0                                      # maximum in the first column
    rows.append(r)
    logits = np.stack(rows)
    idx, val = _run(ctx, engine, logits)
    want = [oracle.greedy_sample(x) for x in logits]
    assert idx.tolist() == want == [4999, N - 1, 200, 0, 0]
    assert val[0] == 9.0 and val[1] == -np.inf and val[2] == np.inf and val[3] == -np.inf and val[4] == 1.0


def test_top_k_shader_differs_only_in_the_tie_rule(oracle):
    """k = 1 of the WGSL top_k takes the FIRST of equal maxima; the sampler takes the last (documented in the header)."""
    x = np.array([1.0, 5.0, 3.0, 5.0, 2.0], np.float32)
    assert oracle.top_k(x, 3).tolist() == [1, 3, 2] and oracle.greedy_sample(x) == 3


# ---- k > 1: WGSL `top_k` (rusty-backend/src/kernels.wgsl:168-188) for every row ----
def _topk(ctx, engine, logits, k):
    M, N = logits.shape
    t = UnifiedTensor.new(ctx, logits, [M, N])
    idx = UnifiedTensor.from_bytes_with_dtype(ctx, np.full(M * k, 0xFFFFFFFF, np.uint32), [M * k * 4], DType.U8)
    val = UnifiedTensor.new(ctx, np.full(M * k, np.nan, np.float32), [M, k])
    engine.top_k(ctx, t, idx, k, out_val=val)
    return idx.to_bytes(ctx).view(np.uint32).reshape(M, k), val.to_vec(ctx).reshape(M, k)


@pytest.mark.parametrize("M,N,k", [(1, 10, 3), (3, 1000, 50), (5, 1025, 1), (32, 128256, 50), (2, 2000, 1024), (4, 40, 64),
                                   (150, 333, 8)])
def test_top_k_random_rows_match_the_shader(ctx, engine, oracle, M, N, k):
    logits = np.random.default_rng(M * 31 + N + k).standard_normal((M, N)).astype(np.float32)
    idx, val = _topk(ctx, engine, logits, k)
    for m in range(M):
        want = oracle.top_k(logits[m], k)
        assert np.array_equal(idx[m], want), (m, idx[m][:8], want[:8])
        kk = min(k, N)
        assert np.array_equal(val[m, :kk], logits[m, want[:kk]])
        assert np.all(np.isneginf(val[m, kk:]))


def test_top_k_ties_nan_and_thresholds(ctx, engine, oracle):
    N, k = 6000, 40
    rng = np.random.default_rng(1)
    rows = []
    rows.append(np.round(rng.standard_normal(N) * 4).astype(np.float32))      # heavy ties: integers in about -16..16
    rows.append(np.full(N, 2.5, np.float32))                                  # all equal: the first k indices
    r = rng.standard_normal(N).astype(np.float32)
    r[::3] = np.nan
    r[5] = np.inf
    r[77] = -np.inf
    rows.append(r)
    r = np.full(N, -2e9, np.float32)                                          # nothing above the shader's -1e9 start value ...
    r[[10, 4000, 4001]] = [1.0, -5e8, 1.0]                                    # ... but three
    rows.append(r)
    r = rng.standard_normal(N).astype(np.float32)
    r[[3, 9]] = [0.0, -0.0]                                                   # the two zeros compare equal
    r[r > 0] = -r[r > 0]
    rows.append(r)
    rows.append(np.full(N, np.nan, np.float32))                               # no candidate at all
    logits = np.stack(rows)
    idx, val = _topk(ctx, engine, logits, k)
    for m in range(logits.shape[0]):
        assert np.array_equal(idx[m], oracle.top_k(logits[m], k)), m
    assert np.array_equal(idx[1], np.arange(k, dtype=np.uint32))
    assert np.array_equal(idx[3][:4], np.array([10, 4001, 4000, 0], np.uint32))
    assert np.all(idx[5] == 0) and np.all(np.isneginf(val[5]))


def test_top_k_argument_errors(ctx, engine):
    from rusty_b200 import BackendError
    t = UnifiedTensor.zeros(ctx, [2, 16])
    idx = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(8, np.uint32), [32], DType.U8)
    for k in (0, 1025):
        with pytest.raises(BackendError) as e:
            engine.top_k(ctx, t, idx, k)
        assert e.value.kind == "InvalidDimensions"
    with pytest.raises(BackendError) as e:
        engine.top_k(ctx, t, idx, 8)          # 2 x 8 indices do not fit 32 bytes
    assert e.value.kind == "InvalidDimensions"


# ---- temperature / top-p with the device's top-k and soft-max statistics ----
def test_softmax_stats_rows(ctx, engine):
    rng = np.random.default_rng(5)
    M, N = 6, 50000
    logits = (rng.standard_normal((M, N)) * 3).astype(np.float32)
    logits[1, ::7] = np.nan
    logits[2, 100] = 40.0
    t = UnifiedTensor.new(ctx, logits, [M, N])
    mx, sm = UnifiedTensor.empty(ctx, [M]), UnifiedTensor.empty(ctx, [M])
    for temp in (0.7, 1.0, 2.5):
        engine.softmax_stats(ctx, t, temp, mx, sm)
        got_mx, got_sm = mx.to_vec(ctx), sm.to_vec(ctx)
        want_mx = np.nanmax(logits, axis=1)
        want_sm = np.nansum(np.exp((logits.astype(np.float64) - want_mx[:, None]) / temp), axis=1)
        assert np.array_equal(got_mx, want_mx)
        assert np.max(np.abs(got_sm - want_sm) / want_sm) < 2e-6
    from rusty_b200 import BackendError
    with pytest.raises(BackendError) as e:
        engine.softmax_stats(ctx, t, 0.0, mx, sm)
    assert e.value.kind == "InvalidOperation"


def test_device_assisted_nucleus_sampling_matches_the_host_sampler(ctx, engine):
    """Same draws, same tokens: k pairs and two floats per row leave the device instead of the whole vocabulary; a row
    whose nucleus is longer than k takes the host path over its logits."""
    from rusty_b200.sampler import Sampler
    rng = np.random.default_rng(9)
    M, N = 8, 32000
    logits = (rng.standard_normal((M, N)) * 4).astype(np.float32)
    logits[3] *= 0.02                       # nearly flat row: the nucleus holds thousands of tokens -> host path
    t = UnifiedTensor.new(ctx, logits, [M, N])
    for temp, top_p in ((0.7, 0.9), (1.0, 0.5), (0.0, 0.9)):
        draws = [float(v) for v in rng.random(M)]
        it = iter(draws)
        got = Sampler(temp, top_p, rand=lambda: next(it)).sample_rows_from_device(ctx, engine, t, k=64)
        it2 = iter(draws)
        host = Sampler(temp, top_p, rand=lambda: next(it2))
        want = [host.sample(logits[m]) for m in range(M)]
        assert got == want, (temp, top_p, got, want)
