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
