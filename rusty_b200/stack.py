"""The Llama-shaped stack of quantised Linears a decode / prefill step runs.

Mirrors the order in which rusty-graph calls Linear::forward during
LlamaModel::forward (rusty-graph/src/lib.rs:420-436): per layer q, k, v, o
(Attention::forward :199-201, :270) then gate, up, down (MLP::forward :318-322),
and lm_head after the last layer (:435).  Only the Linears are run: rope,
attention, SiLU, RMSNorm and the residual adds between them are other
components.  Every Linear therefore reads a fixed, normalised activation buffer
of its input width ([M, d], [M, q] or [M, ffn]) and writes its own output
buffer, so values stay finite over 32-80 layers of random weights; the bytes
moved and the kernels launched are those of the real chain.

Weights: random int8 in [-127,127] with per-output-row f32 scales in
U(0.001,0.02) (QMODE_SYM_ROW, [out,in] storage).  One host array per distinct
(N,K) shape is drawn and uploaded into a separate device buffer per layer, so a
step streams every layer's weights from HBM.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np

from . import capi
from .backend import (ComputeEngine, CudaContext, DType, Graph, QLinear, UnifiedTensor, qlinear_forward_batch)
from .workloads import StackShape


class LinearStack:
    def __init__(self, ctx: CudaContext, shape: StackShape, M: int, x_dtype: DType = DType.FP32,
                 y_dtype: DType = DType.FP32, seed: int = 0, rank: int = 0, world: int = 1,
                 layers: Optional[int] = None, fuse: bool = True, swiglu: bool = False, norms: bool = False,
                 native: bool = False, keep_host: bool = False):
        self.ctx, self.shape, self.M = ctx, shape, M
        self.x_dtype, self.y_dtype = x_dtype, y_dtype
        self.rank, self.world = rank, world
        self.layers = shape.layers if layers is None else layers
        rng = np.random.default_rng(seed)
        host_w: Dict[Tuple[int, int], Tuple[np.ndarray, np.ndarray]] = {}
        self.qls: List[QLinear] = []
        self.names: List[str] = []
        self.dims: List[Tuple[int, int]] = []   # (N_local, K): rows of this rank's weight
        self.out_n: List[int] = []               # output columns of this rank (N_local, or half of it for gate|up pairs)
        self.full_n: List[int] = []              # output columns over all ranks
        # gate|up stored pair-interleaved with silu(gate)*up applied in the kernel's epilogue (MLP::forward,
        # rusty-graph/src/lib.rs:317-323): its output is [M, ffn] and the [M, 2*ffn] intermediate never exists
        # native: every weight in the reference's own quantised format (u8 [in,out], one f32 scale and bias per 64
        # consecutive output features of an input row, rusty-loader/src/lib.rs:155-218) instead of int8 [out,in] with
        # one scale per output row; the pair epilogue needs the latter, so gate|up then writes [M, 2*ffn]
        self.native = native
        # keep_host (tests, small shapes only): the dequantised f32 weight [rows, K] of every Linear, as the reference holds it
        self.host_wf: List[Optional[np.ndarray]] = []
        self.swiglu = swiglu and fuse and not native

        def draw(n: int, k: int):
            if (n, k) not in host_w:
                q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
                s = rng.uniform(0.001, 0.02, size=n).astype(np.float32)
                host_w[(n, k)] = (q, s)
            return host_w[(n, k)]

        # Projections that read the same activation are stored back to back and run as ONE Linear
        # (q|k|v -> [M, q+2kv], gate|up -> [M, 2*ffn]); a shard keeps its slice of each member.
        self.fuse = fuse
        if fuse:
            groups = [("qkv", ["q", "k", "v"]), ("o", ["o"]), ("gate_up", ["gate", "up"]), ("down", ["down"])]
        else:
            groups = [(p, [p]) for p, _n, _k in shape.per_layer()]
        dims = {p: (n, k) for p, n, k in shape.per_layer()}
        linears = []
        for l in range(self.layers):
            linears += [(f"l{l}.{g}", [dims[m] for m in members]) for g, members in groups]
        linears.append(("lm_head", [(shape.vocab, shape.d)]))
        for name, members in linears:
            k = members[0][1]
            qs, ss = [], []
            for n, kk in members:
                assert kk == k and n % world == 0, f"{name}: N={n} not divisible by {world} ranks"
                nl = n // world
                q, s = draw(n, k)
                qs.append(q[rank * nl:(rank + 1) * nl])
                ss.append(s[rank * nl:(rank + 1) * nl])
            pairs = self.swiglu and name.endswith(".gate_up")
            if pairs:
                ql = QLinear.from_gate_up(ctx, qs[0], ss[0], qs[1], ss[1])
                n_rows = 2 * qs[0].shape[0]
            else:
                qcat = qs[0] if len(qs) == 1 else np.concatenate(qs, axis=0)
                scat = ss[0] if len(ss) == 1 else np.concatenate(ss)
                n_rows = qcat.shape[0]
                if native:
                    assert n_rows % 64 == 0, f"{name}: {n_rows} output features of this rank are not whole groups of 64"
                    ukn = (np.ascontiguousarray(qcat.T).astype(np.int16) + 128).astype(np.uint8)
                    sg = np.random.default_rng(seed + 131 * n_rows + k).uniform(0.001, 0.02, size=(k, n_rows // 64)).astype(np.float32)
                    bg = (np.float32(-128.0) * sg).astype(np.float32)
                    ql = QLinear.from_host(ctx, ukn, sg, bg, layout=capi.LAYOUT_KN)
                    if keep_host:   # w[k, n] = u * s[k, n / 64] + b[k, n / 64], rounded as the reference's dequantisation does
                        wkn = ukn.astype(np.float32) * np.repeat(sg, 64, axis=1) + np.repeat(bg, 64, axis=1)
                        self.host_wf.append(np.ascontiguousarray(wkn.T))
                else:
                    ql = QLinear.from_host(ctx, qcat, scat)
                    if keep_host:
                        self.host_wf.append(qcat.astype(np.float32) * scat[:, None])
            if len(self.host_wf) < len(self.qls) + 1:
                self.host_wf.append(None)
            self.qls.append(ql)
            self.names.append(name)
            self.dims.append((n_rows, k))
            self.out_n.append(ql.out_features)
            self.full_n.append(sum(n for n, _ in members) // (2 if pairs else 1))
        # activations: one fixed input per distinct K, N(0,1) like the benchmark's x
        self.inputs: Dict[int, UnifiedTensor] = {}
        self.host_inputs: Dict[int, np.ndarray] = {}
        for k in sorted({k for _, k in self.dims}):
            xh = rng.standard_normal((M, k), dtype=np.float32)
            self.host_inputs[k] = xh
            self.inputs[k] = (UnifiedTensor.from_bf16(ctx, xh, [M, k]) if x_dtype == DType.BF16
                              else UnifiedTensor.new(ctx, xh, [M, k]))
        # outputs: one buffer per distinct local N (reused across layers), logits separate
        self.outputs: Dict[int, UnifiedTensor] = {}
        for nl, name in zip(self.out_n, self.names):
            key = -1 if name == "lm_head" else nl
            if key not in self.outputs:
                self.outputs[key] = UnifiedTensor.empty_with_dtype(ctx, [M, nl], y_dtype)
        self.logits = self.outputs[-1]
        self._xs = [self.inputs[k] for _, k in self.dims]
        self._ys = [self.outputs[-1 if nm == "lm_head" else nl] for nl, nm in zip(self.out_n, self.names)]
        self.graph: Optional[Graph] = None
        # norms: the RMSNorms of a transformer block ride in the Linears that follow them (TransformerBlock::forward,
        # rusty-graph/src/lib.rs:365-377; LlamaModel::forward :433-435): norm1 -> q|k|v, norm2 of (x + attention
        # output) -> gate|up with the sum written back as the new residual stream, the final norm -> lm_head.
        # One weight vector per norm; the residual is a fixed buffer like the other inputs.
        self.norms = bool(norms) and fuse and world == 1 and x_dtype == DType.FP32
        self.norm_w: List[Optional[UnifiedTensor]] = [None] * len(self.qls)
        self.norm_res: List[Optional[UnifiedTensor]] = [None] * len(self.qls)
        self.norm_sum: Optional[UnifiedTensor] = None
        if self.norms:
            res = UnifiedTensor.new(ctx, (rng.standard_normal((M, shape.d)) * 0.5).astype(np.float32), [M, shape.d])
            self.norm_sum = UnifiedTensor.empty(ctx, [M, shape.d])
            for i, name in enumerate(self.names):
                if name.endswith(".qkv") or name.endswith(".gate_up") or name == "lm_head":
                    self.norm_w[i] = UnifiedTensor.new(ctx, rng.uniform(0.5, 1.5, size=shape.d).astype(np.float32), [shape.d])
                    if name.endswith(".gate_up"):
                        self.norm_res[i] = res

    # ---- accounting (algorithmic bytes / flops of ONE step on this rank) ----
    def weight_bytes(self) -> int:
        return sum(n * k for n, k in self.dims)

    def algorithmic_bytes(self) -> int:
        xs, ys = self.x_dtype.size_bytes(), self.y_dtype.size_bytes()
        per_w = (lambda n, k: n * k + n * k // 64 * 8) if self.native else (lambda n, k: n * k + n * 4)
        b = sum(per_w(n, k) + self.M * k * xs + self.M * no * ys for (n, k), no in zip(self.dims, self.out_n))
        for (n, k), w, r in zip(self.dims, self.norm_w, self.norm_res):
            if w is not None:   # norm weight, and for the residual form the residual read and the sum written
                b += k * 4 + (2 * self.M * k * 4 if r is not None else 0)
        return b

    def flops(self) -> int:
        return sum(2 * self.M * n * k for n, k in self.dims)

    def num_linears(self) -> int:
        return len(self.qls)

    # ---- execution ----
    def step(self) -> None:
        """Enqueue every Linear of the stack once (one host call; one call per Linear when norms ride along)."""
        if not self.norms:
            qlinear_forward_batch(self.ctx, self.qls, self._xs, self._ys, self.M, self.x_dtype, self.y_dtype)
            return
        eng = ComputeEngine(self.ctx)
        for ql, x, y, w, r in zip(self.qls, self._xs, self._ys, self.norm_w, self.norm_res):
            if w is None:
                eng.qlinear(self.ctx, x, ql, y)
            else:
                eng.qlinear_normed(self.ctx, x, w, ql, y, residual=r, sum_out=self.norm_sum if r is not None else None)

    def capture(self) -> Graph:
        g = Graph(self.ctx)
        with g:
            self.step()
        self.graph = g
        return g

    # ---- the step a greedy decoder needs: every Linear, then one token per row chosen on the device ----
    def step_greedy(self) -> None:
        from .backend import ComputeEngine
        if getattr(self, "tokens", None) is None:
            self.tokens = UnifiedTensor.from_bytes_with_dtype(self.ctx, np.zeros(self.M, np.uint32), [self.M * 4], DType.U8)
        self.step()
        ComputeEngine(self.ctx).argmax_rows(self.ctx, self.logits, self.tokens)

    def capture_greedy(self) -> Graph:
        self.step_greedy()   # allocates the token buffer outside the capture
        self.ctx.sync()
        g = Graph(self.ctx)
        with g:
            self.step_greedy()
        self.greedy_graph = g
        return g

    def replay(self) -> None:
        self.graph.launch()

    def plans(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for q in self.qls:
            p = q.plan(self.M, self.x_dtype, self.y_dtype)
            out[p] = out.get(p, 0) + 1
        return out
