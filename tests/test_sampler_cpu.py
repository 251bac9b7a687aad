"""Host mirror of rusty-loader's Sampler (tokenizer.rs:134-204): greedy tie rule, nucleus construction, the draw."""
import numpy as np

from rusty_b200.sampler import Sampler


def test_greedy_takes_the_last_maximum():
    s = Sampler(temperature=0.0)
    assert s.sample([1.0, 5.0, 3.0, 5.0, 2.0]) == 3
    assert s.sample([]) == 0
    assert Sampler(temperature=-1.0).sample([0.0, 0.0]) == 1


def test_greedy_agrees_with_the_oracle(oracle):
    rng = np.random.default_rng(0)
    s = Sampler(temperature=0.0)
    for _ in range(20):
        x = rng.integers(-3, 4, size=50).astype(np.float32)   # many ties
        assert s.sample(x) == oracle.greedy_sample(x)


def test_nucleus_and_draw():
    # probabilities 0.5, 0.3, 0.15, 0.05 at temperature 1
    p = np.array([0.05, 0.5, 0.15, 0.3], np.float32)
    logits = np.log(p)
    # top_p = 0.7: nucleus = {1 (0.5), 3 (0.3)}, renormalised 0.625 / 0.375
    for r, want in [(0.0, 1), (0.62, 1), (0.63, 3), (0.999, 3)]:
        assert Sampler(temperature=1.0, top_p=0.7, rand=lambda r=r: r).sample(logits) == want
    # top_p = 1.0 keeps everything, in descending order 1, 3, 2, 0
    for r, want in [(0.49, 1), (0.51, 3), (0.81, 2), (0.96, 0)]:
        assert Sampler(temperature=1.0, top_p=1.0, rand=lambda r=r: r).sample(logits) == want
    # a tiny top_p keeps only the most likely token
    assert Sampler(temperature=1.0, top_p=0.01, rand=lambda: 0.999).sample(logits) == 1


def test_temperature_sharpens():
    logits = np.array([0.0, 1.0, 2.0], np.float32)
    cold = Sampler(temperature=0.1, top_p=0.9, rand=lambda: 0.95)
    assert cold.sample(logits) == 2           # at T = 0.1 the top token alone exceeds 0.9
    hot = Sampler(temperature=10.0, top_p=1.0, rand=lambda: 0.95)
    assert hot.sample(logits) == 0            # nearly uniform: the last of the sorted order (2, 1, 0) is drawn


def test_defaults_are_the_reference_defaults():
    s = Sampler()
    assert abs(float(s.temperature) - 0.7) < 1e-7 and abs(float(s.top_p) - 0.9) < 1e-7


def test_nucleus_walk_over_candidates_equals_the_walk_over_the_whole_row():
    """The device hands the host the k largest logits (sorted as the shader sorts them) and the row's soft-max
    statistics; the walk over those candidates must choose what Sampler.sample chooses on the whole row."""
    import numpy as np
    from rusty_b200.sampler import Sampler
    rng = np.random.default_rng(7)
    for trial in range(40):
        n = int(rng.integers(50, 3000))
        logits = (rng.standard_normal(n) * rng.uniform(0.5, 6.0)).astype(np.float32)
        t, top_p = float(rng.uniform(0.3, 1.5)), float(rng.uniform(0.3, 0.98))
        r = float(rng.random())
        whole = Sampler(t, top_p, rand=lambda: r).sample(logits)
        order = np.lexsort((np.arange(n), -logits))            # value descending, index ascending among equals
        scaled_max = np.float32(logits.max())
        e = np.exp(((logits - scaled_max) / np.float32(t)).astype(np.float32)).astype(np.float32)
        exp_sum = np.float32(0.0)
        for v in e:
            exp_sum = np.float32(exp_sum + v)
        for k in (n, 256, 8):
            k = min(k, n)
            got = Sampler(t, top_p, rand=lambda: r).sample_from_candidates(order[:k], logits[order[:k]], scaled_max, exp_sum)
            if got is None:
                assert k < n          # only a truncated list may fail to reach top_p
            else:
                assert got == whole, (trial, k, got, whole)
