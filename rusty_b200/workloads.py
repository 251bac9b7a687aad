"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations.  There are no checkpoints or datasets involved: Llama
names below are SHAPES only, filled with random int8 weights.

Draw order is fixed (numpy ``default_rng(seed)``: x, then weights, then scales)
so every harness regenerates identical inputs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np


def sym_row_linear(seed: int, M: int, K: int, N: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """x f32 [M,K] ~ N(0,1); q int8 [N,K] uniform in [-127,127]; scale f32 [N] ~ U(0.001,0.02)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    q = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, size=N).astype(np.float32)
    return x, q, s


def affine_g64_from_sym(q: np.ndarray, seed: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """The same weights in the reference's native layout: u8 = q + 128, one scale
    ~ U(0.001,0.02) and bias = -128*scale per 64 consecutive flat elements."""
    rng = np.random.default_rng(seed + 1000)
    u = (q.astype(np.int16) + 128).astype(np.uint8)
    groups = q.size // 64
    s = rng.uniform(0.001, 0.02, size=groups).astype(np.float32)
    b = (np.float32(-128.0) * s).astype(np.float32)
    return u, s, b


@dataclass(frozen=True)
class StackShape:
    name: str
    d: int
    q: int
    kv: int
    ffn: int
    vocab: int
    layers: int

    def per_layer(self) -> List[Tuple[str, int, int]]:
        """(projection, out_features N, in_features K) in call order
        (rusty-graph/src/lib.rs:199-201, :270, :318-322)."""
        return [("q", self.q, self.d), ("k", self.kv, self.d), ("v", self.kv, self.d), ("o", self.d, self.q),
                ("gate", self.ffn, self.d), ("up", self.ffn, self.d), ("down", self.d, self.ffn)]

    def linears(self) -> List[Tuple[str, int, int]]:
        out = []
        for l in range(self.layers):
            out += [(f"l{l}.{p}", n, k) for p, n, k in self.per_layer()]
        out.append(("lm_head", self.vocab, self.d))
        return out

    def weight_bytes(self) -> int:
        return sum(n * k for _, n, k in self.linears())

    def scale_bytes(self) -> int:
        return sum(n * 4 for n, _k in [(n, k) for _, n, k in self.linears()])

    def flops_per_token(self) -> int:
        return 2 * self.weight_bytes()


STACKS: Dict[str, StackShape] = {
    "llama7b": StackShape("llama7b", 4096, 4096, 4096, 11008, 32000, 32),
    "llama3-8b": StackShape("llama3-8b", 4096, 4096, 1024, 14336, 128256, 32),
    "llama2-70b": StackShape("llama2-70b", 8192, 8192, 1024, 28672, 32000, 80),
}
