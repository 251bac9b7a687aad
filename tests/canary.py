"""Canary-padded device outputs for the GPU tests.

No memory checker can be run on the GPU kernels, so the tests carry their own:
an output tensor is allocated with a pad of known bytes behind its payload, and
after the kernel has run the pad must be unchanged.  The payload is pre-filled
with NaN so that an element the kernel failed to write shows up as well.
"""
import numpy as np

from rusty_b200 import DType, UnifiedTensor
from rusty_b200.backend import _Storage, bf16_bits_to_f32

PAD_BYTES = 4096
PAD_BYTE = 0xC3


class GuardedOutput:
    def __init__(self, ctx, shape, dtype=DType.FP32):
        self.ctx, self.shape, self.dtype = ctx, list(shape), dtype
        self.payload = int(np.prod(shape, dtype=np.int64)) * dtype.size_bytes()
        st = _Storage(ctx, self.payload + PAD_BYTES, pooled=False)
        self.tensor = UnifiedTensor(st, self.shape, dtype)
        fill = np.empty(self.payload + PAD_BYTES, np.uint8)
        if dtype == DType.FP32:
            fill[: self.payload].view(np.uint32)[:] = 0x7FC00000
        elif dtype == DType.BF16:
            fill[: self.payload].view(np.uint16)[:] = 0x7FC0
        else:
            fill[: self.payload] = 0xEE
        fill[self.payload:] = PAD_BYTE
        self.tensor.write_data(ctx, fill)

    def read(self):
        """The payload as float32 (bf16 widened) after checking the canary."""
        raw = self.tensor.to_bytes(self.ctx)
        pad = raw[self.payload:]
        bad = np.flatnonzero(pad != PAD_BYTE)
        assert bad.size == 0, f"kernel wrote {bad.size} bytes past the end of its output (first at +{int(bad[0])})"
        body = raw[: self.payload]
        if self.dtype == DType.BF16:
            return bf16_bits_to_f32(body.view(np.uint16)).reshape(self.shape)
        if self.dtype == DType.FP32:
            return body.view(np.float32).reshape(self.shape).copy()
        return body.copy()
