"""Host-side mirror of rusty-loader's Sampler (rusty-loader/src/tokenizer.rs:134-204).

Greedy choice (temperature <= 0) also exists on the device (`ComputeEngine.argmax_rows`, sharded form in
`rusty_b200.shard`); temperature / top-p sampling stays on the host, as in the reference, in f32 arithmetic and in the
reference's order of operations: scale by 1/temperature, soft-max with the maximum subtracted, sort by probability
(descending, stable), take the shortest prefix whose sum reaches top_p, renormalise, draw.  `sample_rows_from_device`
does the same walk over the k largest logits of each row and the row's soft-max statistics, both computed on the
device, so that k pairs and two floats per row cross PCIe instead of the whole vocabulary; a row whose nucleus does not
fit into k falls back to reading its logits.
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

    def sample_from_candidates(self, idx, val, row_max: float, exp_sum: float):
        """The nucleus walk over candidates sorted by value (descending; equal values by ascending index), given the
        row's largest logit and sum exp((x - max) / T) over ALL logits.  Returns the token, or None when the
        candidates' probability mass does not reach top_p (the nucleus is longer than the list)."""
        t = self.temperature
        scaled = (np.asarray(val, np.float32) / t).astype(np.float32)            # the reference's order: scale, then subtract
        max_val = np.float32(np.float32(row_max) / t)
        probs = (np.exp((scaled - max_val).astype(np.float32)).astype(np.float32) / np.float32(exp_sum)).astype(np.float32)
        cumsum = np.float32(0.0)
        n = 0
        for p in probs:
            cumsum = np.float32(cumsum + p)
            n += 1
            if cumsum >= self.top_p:
                break
        else:
            return None
        nucleus_sum = np.float32(0.0)
        for p in probs[:n]:
            nucleus_sum = np.float32(nucleus_sum + p)
        r = np.float32(self._rand())
        cumsum = np.float32(0.0)
        for i in range(n):
            cumsum = np.float32(cumsum + np.float32(probs[i] / nucleus_sum))
            if r < cumsum:
                return int(idx[i])
        return int(idx[0])

    def sample_rows_from_device(self, ctx, engine, logits, k: int = 64):
        """One token per row of a device tensor logits[M, N] (f32).  temperature <= 0: the device arg-max.  Otherwise
        the device's top-k and soft-max statistics, then the reference's nucleus walk on the host."""
        from .backend import DType, UnifiedTensor
        M, N = int(np.prod(logits.shape[:-1], dtype=np.int64)), int(logits.shape[-1])
        if self.temperature <= 0.0:
            tok = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(M, np.uint32), [M * 4], DType.U8)
            engine.argmax_rows(ctx, logits, tok)
            return [int(t) for t in tok.to_bytes(ctx).view(np.uint32)]
        k = max(1, min(int(k), N, 1024))
        idx_t = UnifiedTensor.from_bytes_with_dtype(ctx, np.zeros(M * k, np.uint32), [M * k * 4], DType.U8)
        val_t = UnifiedTensor.empty(ctx, [M, k])
        mx_t, sm_t = UnifiedTensor.empty(ctx, [M]), UnifiedTensor.empty(ctx, [M])
        engine.top_k(ctx, logits, idx_t, k, out_val=val_t)
        engine.softmax_stats(ctx, logits, float(self.temperature), mx_t, sm_t)
        idx = idx_t.to_bytes(ctx).view(np.uint32).reshape(M, k)
        val = val_t.to_vec(ctx).reshape(M, k)
        mx, sm = mx_t.to_vec(ctx), sm_t.to_vec(ctx)
        out = []
        host_rows = None
        for m in range(M):
            tok = self.sample_from_candidates(idx[m], val[m], mx[m], sm[m])
            if tok is None:   # the nucleus is longer than k: the reference's own path over the whole row
                if host_rows is None:
                    host_rows = logits.to_vec(ctx).reshape(M, N)
                tok = self.sample(host_rows[m])
            out.append(tok)
        return out
