"""Host mirror of rusty-graph's Linear and LoRAAdapter (rusty-graph/src/lib.rs:16-110).

``Linear.forward(engine, x)`` keeps the reference contract — ``x . W`` with the
weight stored ``[in, out]``, no bias, optional LoRA branch ``(x . A) . B`` added
without alpha/rank scaling (lib.rs:72-80) — and gains ``from_quantized`` so the
same call routes to the fused int8 kernels.  Leading dimensions of ``x`` are
flattened to rows (the reference reads shape[0] and shape[1] only, which breaks
on 3-D activations; rusty/src/nn/linear.rs:63 documents the flattening).
The autograd tape the reference records per matmul (rusty-autograd/src/lib.rs:468-477)
is training machinery and is not mirrored.
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .backend import ComputeEngine, CudaContext, DType, QLinear, UnifiedTensor


class LoRAAdapter:
    def __init__(self, ctx: CudaContext, in_dim: int, out_dim: int, rank: int, alpha: float):
        # lib.rs:38-43: A filled with 0.01, B with 0.0
        self.a = UnifiedTensor.new(ctx, np.full(in_dim * rank, 0.01, np.float32), [in_dim, rank])
        self.b = UnifiedTensor.new(ctx, np.zeros(rank * out_dim, np.float32), [rank, out_dim])
        self.alpha = alpha
        self.rank = rank

    def params(self):
        return [self.a, self.b]


class Linear:
    def __init__(self, ctx: CudaContext, weight: Optional[UnifiedTensor], lora: Optional[LoRAAdapter] = None,
                 qweight: Optional[QLinear] = None):
        self.ctx = ctx
        self.weight = weight      # f32 [in, out]
        self.qweight = qweight    # fused int8 weight
        self.lora = lora

    @staticmethod
    def new(ctx: CudaContext, weight: UnifiedTensor) -> "Linear":
        return Linear(ctx, weight)

    @staticmethod
    def with_lora(ctx: CudaContext, weight: UnifiedTensor, lora: LoRAAdapter) -> "Linear":
        return Linear(ctx, weight, lora)

    @staticmethod
    def from_quantized(ctx: CudaContext, qweight: QLinear, lora: Optional[LoRAAdapter] = None) -> "Linear":
        return Linear(ctx, None, lora, qweight)

    def out_features(self) -> int:
        return self.qweight.N if self.qweight is not None else self.weight.shape[1]

    def in_features(self) -> int:
        return self.qweight.K if self.qweight is not None else self.weight.shape[0]

    def forward(self, engine: ComputeEngine, x: UnifiedTensor, out_dtype: DType = DType.FP32) -> UnifiedTensor:
        ctx = self.ctx
        k = self.in_features()
        rows = int(np.prod(x.shape[:-1], dtype=np.int64))
        assert x.shape[-1] == k, f"Linear expects last dim {k}, got {x.shape}"
        x2 = x.reshaped([rows, k])
        n = self.out_features()
        if self.qweight is not None:
            out = UnifiedTensor.empty_with_dtype(ctx, [rows, n], out_dtype)
            engine.qlinear(ctx, x2, self.qweight, out)
        else:
            out = UnifiedTensor.empty(ctx, [rows, n])
            engine.matmul(ctx, x2, self.weight, out)
        if self.lora is not None:
            assert x2.dtype == DType.FP32 and out.dtype == DType.FP32, "the LoRA branch is f32"
            temp = UnifiedTensor.empty(ctx, [rows, self.lora.rank])
            engine.matmul(ctx, x2, self.lora.a, temp)
            lora_out = UnifiedTensor.empty(ctx, [rows, n])
            engine.matmul(ctx, temp, self.lora.b, lora_out)
            summed = UnifiedTensor.empty(ctx, [rows, n])
            engine.add(ctx, out, lora_out, summed)
            out = summed
        return out.reshaped(list(x.shape[:-1]) + [n])

    def params(self):
        p = [self.weight] if self.weight is not None else []
        if self.lora is not None:
            p.extend(self.lora.params())
        return p
