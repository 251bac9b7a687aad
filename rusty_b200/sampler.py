"""Host-side mirror of rusty-loader's Sampler (rusty-loader/src/tokenizer.rs:134-204).

Greedy choice (temperature <= 0) also exists on the device (`ComputeEngine.argmax_rows`, sharded form in
`rusty_b200.shard`); temperature / top-p sampling stays on the host, as in the reference, in f32 arithmetic and in the
reference's order of operations: scale by 1/temperature, soft-max with the maximum subtracted, sort by probability
(descending, stable), take the shortest prefix whose sum reaches top_p, renormalise, draw.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np


class Sampler:
    def __init__(self, temperature: float = 0.7, top_p: float = 0.9, rand: Optional[Callable[[], float]] = None):
        """Defaults of `impl Default for Sampler` (tokenizer.rs:140-147).  `rand` returns a uniform [0, 1) float; the
        reference calls rand::random::<f32>() (tokenizer.rs:193)."""
        self.temperature = np.float32(temperature)
        self.top_p = np.float32(top_p)
        self._rand = rand or (lambda: float(np.random.random()))

    def sample(self, logits) -> int:
        x = np.asarray(logits, np.float32).ravel()
        if self.temperature <= 0.0:
            # max_by(partial_cmp) keeps the LAST of equal maxima; an empty slice gives 0 (tokenizer.rs:151-158)
            if x.size == 0:
                return 0
            return int(x.size - 1 - np.argmax(x[::-1]))
        scaled = (x / self.temperature).astype(np.float32)
        max_val = np.float32(scaled.max()) if scaled.size else np.float32(-np.inf)
        e = np.exp((scaled - max_val).astype(np.float32)).astype(np.float32)
        exp_sum = np.float32(0.0)
        for v in e:                       # sequential f32 sum, as Iterator::sum does
            exp_sum = np.float32(exp_sum + v)
        probs = (e / exp_sum).astype(np.float32)
        order = np.argsort(-probs, kind="stable")          # sort_by(probs[b].partial_cmp(probs[a])) is stable
        cumsum = np.float32(0.0)
        nucleus = []
        for idx in order:
            cumsum = np.float32(cumsum + probs[idx])
            nucleus.append(int(idx))
            if cumsum >= self.top_p:
                break
        nucleus_sum = np.float32(0.0)
        for i in nucleus:
            nucleus_sum = np.float32(nucleus_sum + probs[i])
        r = np.float32(self._rand())
        cumsum = np.float32(0.0)
        for i in nucleus:
            cumsum = np.float32(cumsum + np.float32(probs[i] / nucleus_sum))
            if r < cumsum:
                return i
        return nucleus[0] if nucleus else 0
