"""Host-side mirror of rusty-backend's tensor / engine surface over the C ABI.

Same names, argument meaning and error behaviour as the reference's Rust types,
so the parity tests read like tests of rusty itself:

    CudaContext    <- WgpuContext         (rusty-backend/src/lib.rs:11-53)
    DType          <- DType               (lib.rs:56-76), extended with BF16/I8/U8
    UnifiedTensor  <- UnifiedTensor       (lib.rs:78-241)
    ComputeEngine  <- ComputeEngine       (lib.rs:343; matmul :4403, matmul_bt :4299,
                                           dequantize :4872, affine_dequantize :4939,
                                           copy_tensor :4019)
    QLinear        <- (new) the fused int8 weight the engine multiplies in place of
                      the load-time-dequantised f32 copy (rusty-loader/src/lib.rs:155-218)

Everything here is glue: each method is one call into librusty_cuda.  numpy is
used for host arrays only.
"""
from __future__ import annotations

import ctypes as C
from enum import IntEnum
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import BackendError, check, lib


class DType(IntEnum):
    FP32 = capi.F32
    FP16 = capi.F16
    BF16 = capi.BF16
    I8 = capi.I8
    U8 = capi.U8

    def size_bytes(self) -> int:
        return {DType.FP32: 4, DType.FP16: 2, DType.BF16: 2, DType.I8: 1, DType.U8: 1}[self]


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as uint16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


class CudaContext:
    """One device, one in-order stream, one buffer pool (WgpuContext::new)."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        check(lib().rusty_cuda_ctx_create(device, C.byref(h)))
        self._h = h
        self.device = device

    @property
    def handle(self) -> C.c_void_p:
        if self._h is None:
            raise BackendError(capi.ERR_INVALID_OPERATION, "context already destroyed")
        return self._h

    def adapter_info(self) -> str:
        buf = C.create_string_buffer(256)
        check(lib().rusty_cuda_ctx_adapter_info(self.handle, buf, 256), self.handle)
        return buf.value.decode()

    def sync(self) -> None:
        check(lib().rusty_cuda_sync(self.handle), self.handle)

    def self_check(self) -> None:
        """Raises if a kernel wrote outside its region of the context's internal scratch (guard zones)."""
        check(lib().rusty_cuda_ctx_self_check(self.handle), self.handle)

    def launch_count(self) -> int:
        n = C.c_uint64()
        check(lib().rusty_cuda_ctx_launch_count(self.handle, C.byref(n)), self.handle)
        return n.value

    def stream(self) -> int:
        s = C.c_void_p()
        check(lib().rusty_cuda_ctx_stream(self.handle, C.byref(s)), self.handle)
        return s.value or 0

    def pool_idle_count(self, nbytes: int) -> int:
        n = C.c_size_t()
        check(lib().rusty_cuda_pool_idle_count(self.handle, nbytes, C.byref(n)), self.handle)
        return n.value

    def pool_clear(self) -> None:
        check(lib().rusty_cuda_pool_clear(self.handle), self.handle)

    def destroy(self) -> None:
        if self._h is not None:
            lib().rusty_cuda_ctx_destroy(self._h)
            self._h = None


class _Storage:
    """Reference-counted device buffer (the Arc<TensorData> of the reference)."""

    def __init__(self, ctx: CudaContext, nbytes: int, pooled: bool):
        h = C.c_void_p()
        check(lib().rusty_cuda_buf_alloc(ctx.handle, nbytes, 1 if pooled else 0, C.byref(h)), ctx.handle)
        self.h = h
        self.ctx = ctx
        self.nbytes = nbytes

    def __del__(self):
        try:
            if self.h is not None and self.ctx._h is not None:
                lib().rusty_cuda_buf_release(self.h)
        except Exception:
            pass
        self.h = None


class UnifiedTensor:
    """Buffer + shape + dtype tag."""

    def __init__(self, storage: _Storage, shape: Sequence[int], dtype: DType):
        self._data = storage
        self.shape = list(shape)
        self.dtype = dtype

    # -- constructors (lib.rs:115-196) --
    @staticmethod
    def new(ctx: CudaContext, data, shape: Sequence[int]) -> "UnifiedTensor":
        arr = np.ascontiguousarray(data, dtype=np.float32)
        return UnifiedTensor.from_bytes_with_dtype(ctx, arr, shape, DType.FP32)

    @staticmethod
    def empty(ctx: CudaContext, shape: Sequence[int]) -> "UnifiedTensor":
        return UnifiedTensor.empty_with_dtype(ctx, shape, DType.FP32)

    @staticmethod
    def empty_with_dtype(ctx: CudaContext, shape: Sequence[int], dtype: DType) -> "UnifiedTensor":
        n = int(np.prod(shape, dtype=np.int64)) * dtype.size_bytes()
        return UnifiedTensor(_Storage(ctx, n, pooled=True), shape, dtype)

    @staticmethod
    def zeros(ctx: CudaContext, shape: Sequence[int]) -> "UnifiedTensor":
        return UnifiedTensor.new(ctx, np.zeros(int(np.prod(shape, dtype=np.int64)), np.float32), shape)

    @staticmethod
    def from_bytes(ctx: CudaContext, data, shape: Sequence[int]) -> "UnifiedTensor":
        return UnifiedTensor.from_bytes_with_dtype(ctx, data, shape, DType.FP32)

    @staticmethod
    def from_bytes_with_dtype(ctx: CudaContext, data, shape: Sequence[int], dtype: DType) -> "UnifiedTensor":
        raw = np.ascontiguousarray(data).view(np.uint8).ravel()
        st = _Storage(ctx, raw.size, pooled=False)
        t = UnifiedTensor(st, shape, dtype)
        t.write_data(ctx, raw)
        return t

    @staticmethod
    def from_bf16(ctx: CudaContext, data_f32, shape: Sequence[int]) -> "UnifiedTensor":
        """Upload f32 host values rounded (RNE) to bf16."""
        return UnifiedTensor.from_bytes_with_dtype(ctx, f32_to_bf16_bits(np.asarray(data_f32, np.float32)), shape, DType.BF16)

    # -- accessors --
    def buffer(self) -> C.c_void_p:
        return self._data.h

    def size_in_bytes(self) -> int:
        return self._data.nbytes

    def device_ptr(self) -> int:
        p = C.c_void_p()
        check(lib().rusty_cuda_buf_device_ptr(self._data.h, C.byref(p)))
        return p.value or 0

    def write_data(self, ctx: CudaContext, data, offset: int = 0) -> None:
        raw = np.ascontiguousarray(data).view(np.uint8).ravel()
        check(lib().rusty_cuda_buf_upload(ctx.handle, self._data.h, offset, raw.ctypes.data_as(C.c_void_p), raw.size),
              ctx.handle)

    def reshaped(self, new_shape: Sequence[int]) -> "UnifiedTensor":
        cur = int(np.prod(self.shape, dtype=np.int64))
        new = int(np.prod(new_shape, dtype=np.int64))
        assert cur == new, f"Cannot reshape tensor of size {cur} to {list(new_shape)}"
        return UnifiedTensor(self._data, new_shape, self.dtype)

    def to_bytes(self, ctx: CudaContext) -> np.ndarray:
        out = np.empty(self._data.nbytes, np.uint8)
        check(lib().rusty_cuda_buf_download(ctx.handle, self._data.h, 0, out.ctypes.data_as(C.c_void_p), out.size),
              ctx.handle)
        return out

    def to_vec(self, ctx: CudaContext) -> np.ndarray:
        """Blocking readback.  FP32 tensors come back as float32 (the reference
        always reinterprets as f32); BF16 as float32 values; byte types as is."""
        raw = self.to_bytes(ctx)
        if self.dtype == DType.BF16:
            return bf16_bits_to_f32(raw.view(np.uint16))
        if self.dtype == DType.I8:
            return raw.view(np.int8)
        if self.dtype == DType.U8:
            return raw
        return raw[: raw.size // 4 * 4].view(np.float32)


def interleave_pairs(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Rows (or entries) a_0, b_0, a_1, b_1, ... of two equally shaped arrays."""
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    out = np.empty((2 * a.shape[0],) + a.shape[1:], a.dtype)
    out[0::2], out[1::2] = a, b
    return out


class QLinear:
    """A weight kept in its 1-byte quantised form on the device."""

    def __init__(self, ctx: CudaContext, weight: UnifiedTensor, scales: UnifiedTensor,
                 biases: Optional[UnifiedTensor], out_features: int, in_features: int,
                 layout: int = capi.LAYOUT_NK, qmode: int = capi.QMODE_SYM_ROW):
        h = C.c_void_p()
        check(lib().rusty_cuda_qlinear_create(ctx.handle, weight.buffer(), scales.buffer(),
                                              biases.buffer() if biases is not None else None,
                                              out_features, in_features, layout, qmode, C.byref(h)), ctx.handle)
        self._h = h
        self.ctx = ctx
        self.N, self.K = out_features, in_features
        self.layout, self.qmode = layout, qmode
        self._keep = (weight, scales, biases)

    @staticmethod
    def from_host(ctx: CudaContext, q: np.ndarray, scales: np.ndarray, biases: Optional[np.ndarray] = None,
                  layout: int = capi.LAYOUT_NK) -> "QLinear":
        """q: int8 (SYM_ROW, no biases) or uint8 (AFFINE_G64 with biases), 2-D in
        the storage order `layout` names."""
        q = np.ascontiguousarray(q)
        N, K = (q.shape if layout == capi.LAYOUT_NK else q.shape[::-1])
        affine = biases is not None
        wt = UnifiedTensor.from_bytes_with_dtype(ctx, q, list(q.shape), DType.U8 if affine else DType.I8)
        st = UnifiedTensor.new(ctx, np.asarray(scales, np.float32).ravel(), [int(np.size(scales))])
        bt = UnifiedTensor.new(ctx, np.asarray(biases, np.float32).ravel(), [int(np.size(biases))]) if affine else None
        return QLinear(ctx, wt, st, bt, N, K, layout, capi.QMODE_AFFINE_G64 if affine else capi.QMODE_SYM_ROW)

    def set_activation(self, act: int) -> "QLinear":
        """capi.ACT_SWIGLU_PAIRS: rows (2j, 2j+1) are (gate_j, up_j); every forward then writes silu(gate) * up,
        N/2 columns (MLP::forward, rusty-graph/src/lib.rs:317-323, with the activation in the kernel's epilogue)."""
        check(lib().rusty_cuda_qlinear_set_activation(self._h, act), self.ctx.handle)
        self.act = act
        return self

    @property
    def out_features(self) -> int:
        return self.N // 2 if getattr(self, "act", 0) == capi.ACT_SWIGLU_PAIRS else self.N

    @staticmethod
    def from_gate_up(ctx: CudaContext, gate_q: np.ndarray, gate_s: np.ndarray, up_q: np.ndarray,
                     up_s: np.ndarray) -> "QLinear":
        """Interleave two [F, K] int8 projections row by row (gate_0, up_0, gate_1, ...) and enable the pair epilogue."""
        q, s = interleave_pairs(gate_q, up_q), interleave_pairs(gate_s, up_s)
        return QLinear.from_host(ctx, q, s).set_activation(capi.ACT_SWIGLU_PAIRS)

    def plan(self, M: int, x_dtype: DType = DType.FP32, y_dtype: DType = DType.FP32) -> str:
        buf = C.create_string_buffer(64)
        check(lib().rusty_cuda_qlinear_plan(self._h, int(x_dtype), M, int(y_dtype), buf, 64))
        return buf.value.decode()

    def __del__(self):
        try:
            if self._h is not None and self.ctx._h is not None:
                lib().rusty_cuda_qlinear_destroy(self._h)
        except Exception:
            pass
        self._h = None


class ComputeEngine:
    """The operator surface of rusty-backend's ComputeEngine for this path.
    Methods enqueue on the context's stream and return; the caller allocates
    every output."""

    def __init__(self, ctx: CudaContext):
        self._ctx = ctx

    def matmul(self, ctx: CudaContext, a: UnifiedTensor, b: UnifiedTensor, out: UnifiedTensor) -> None:
        m, k, n = a.shape[0], a.shape[1], b.shape[1]
        check(lib().rusty_cuda_matmul_f32(ctx.handle, a.buffer(), b.buffer(), out.buffer(), m, k, n), ctx.handle)

    def matmul_bt(self, ctx: CudaContext, a: UnifiedTensor, b: UnifiedTensor, out: UnifiedTensor) -> None:
        m, k, n = a.shape[0], a.shape[1], b.shape[0]
        check(lib().rusty_cuda_matmul_bt_f32(ctx.handle, a.buffer(), b.buffer(), out.buffer(), m, k, n), ctx.handle)

    def dequantize(self, ctx: CudaContext, input: UnifiedTensor, out: UnifiedTensor) -> None:
        total = int(np.prod(input.shape, dtype=np.int64))
        check(lib().rusty_cuda_dequantize_u8(ctx.handle, input.buffer(), out.buffer(), total), ctx.handle)

    def affine_dequantize(self, ctx: CudaContext, weight: UnifiedTensor, scales: UnifiedTensor,
                          biases: UnifiedTensor, out: UnifiedTensor) -> None:
        total = int(np.prod(out.shape, dtype=np.int64))
        check(lib().rusty_cuda_affine_dequantize_g64(ctx.handle, weight.buffer(), scales.buffer(), biases.buffer(),
                                                     out.buffer(), total), ctx.handle)

    def add(self, ctx: CudaContext, a: UnifiedTensor, b: UnifiedTensor, out: UnifiedTensor) -> None:
        total = int(np.prod(out.shape, dtype=np.int64))
        check(lib().rusty_cuda_add_f32(ctx.handle, a.buffer(), b.buffer(), out.buffer(), total), ctx.handle)

    def copy_tensor(self, ctx: CudaContext, src: UnifiedTensor, dst: UnifiedTensor, dst_offset: int) -> None:
        check(lib().rusty_cuda_buf_copy(ctx.handle, src.buffer(), dst.buffer(), dst_offset), ctx.handle)

    def silu(self, ctx: CudaContext, x: UnifiedTensor, out: UnifiedTensor) -> None:
        total = int(np.prod(out.shape, dtype=np.int64))
        check(lib().rusty_cuda_silu_f32(ctx.handle, x.buffer(), out.buffer(), total), ctx.handle)

    def mul(self, ctx: CudaContext, a: UnifiedTensor, b: UnifiedTensor, out: UnifiedTensor) -> None:
        total = int(np.prod(out.shape, dtype=np.int64))
        check(lib().rusty_cuda_mul_f32(ctx.handle, a.buffer(), b.buffer(), out.buffer(), total), ctx.handle)

    def rms_norm(self, ctx: CudaContext, input: UnifiedTensor, weight: UnifiedTensor, out: UnifiedTensor,
                 eps: float = 1e-5) -> None:
        """ComputeEngine::rms_norm (rusty-backend/src/lib.rs:4492): every row of input[..., K] normalised."""
        K = int(input.shape[-1])
        M = int(np.prod(input.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_rms_norm_f32(ctx.handle, input.buffer(), None, weight.buffer(), out.buffer(), None, M, K, eps),
              ctx.handle)

    def rms_norm_residual(self, ctx: CudaContext, x: UnifiedTensor, residual: UnifiedTensor, weight: UnifiedTensor,
                          out: UnifiedTensor, sum_out: Optional[UnifiedTensor] = None, eps: float = 1e-5) -> None:
        """ComputeEngine::rms_norm_residual (rusty-backend/src/lib.rs:5320), row by row; sum_out receives x + residual."""
        K = int(x.shape[-1])
        M = int(np.prod(x.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_rms_norm_f32(ctx.handle, x.buffer(), residual.buffer(), weight.buffer(), out.buffer(),
                                            sum_out.buffer() if sum_out is not None else None, M, K, eps), ctx.handle)

    def embedding(self, ctx: CudaContext, table: UnifiedTensor, ids: UnifiedTensor, out: UnifiedTensor) -> None:
        """Embedding::forward (rusty-graph/src/lib.rs:121-135) with the ids (u32) already on the device."""
        vocab, dim = int(table.shape[0]), int(table.shape[1])
        n = ids.size_in_bytes() // 4
        check(lib().rusty_cuda_embedding_f32(ctx.handle, table.buffer(), ids.buffer(), out.buffer(), n, vocab, dim), ctx.handle)

    def qlinear_normed(self, ctx: CudaContext, x: UnifiedTensor, norm_weight: UnifiedTensor, w: "QLinear", out: UnifiedTensor,
                       residual: Optional[UnifiedTensor] = None, normed_out: Optional[UnifiedTensor] = None,
                       sum_out: Optional[UnifiedTensor] = None, eps: float = 1e-5) -> None:
        """out = w(RMSNorm(x [+ residual]) * norm_weight): norm1 -> q|k|v, norm2 -> gate|up of a transformer block."""
        M = int(np.prod(x.shape[:-1], dtype=np.int64))
        b = lambda t: t.buffer() if t is not None else None
        check(lib().rusty_cuda_qlinear_forward_normed(ctx.handle, w._h, x.buffer(), b(residual), norm_weight.buffer(), eps, M,
                                                      b(normed_out), b(sum_out), out.buffer(), int(out.dtype)), ctx.handle)

    def qlinear_residual(self, ctx: CudaContext, x: UnifiedTensor, w: "QLinear", residual: UnifiedTensor,
                         out: UnifiedTensor) -> None:
        """out = residual + w(x): the residual add after o_proj / down_proj inside the Linear's epilogue (out may be
        the residual tensor itself)."""
        M = int(np.prod(x.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_qlinear_forward_residual(ctx.handle, w._h, x.buffer(), int(x.dtype), M, residual.buffer(),
                                                        out.buffer(), int(out.dtype)), ctx.handle)

    def argmax_rows(self, ctx: CudaContext, logits: UnifiedTensor, out_idx: UnifiedTensor,
                    out_val: Optional[UnifiedTensor] = None) -> None:
        """Greedy token per row (Sampler::sample with temperature <= 0, rusty-loader/src/tokenizer.rs:151-158):
        out_idx is u32[M] (allocate it with 4*M bytes), out_val the optional f32[M] maxima."""
        m = int(np.prod(logits.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_argmax_rows_f32(ctx.handle, logits.buffer(), m, int(logits.shape[-1]), out_idx.buffer(),
                                               out_val.buffer() if out_val is not None else None), ctx.handle)

    def top_k(self, ctx: CudaContext, input: UnifiedTensor, out_idx: UnifiedTensor, k: int,
              out_val: Optional[UnifiedTensor] = None) -> None:
        """ComputeEngine::top_k (rusty-backend/src/lib.rs:4901) for every row of input[..., N]: out_idx u32 [M, k]."""
        N = int(input.shape[-1])
        M = int(np.prod(input.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_top_k_rows_f32(ctx.handle, input.buffer(), M, N, k, out_idx.buffer(),
                                              out_val.buffer() if out_val is not None else None), ctx.handle)

    def softmax_stats(self, ctx: CudaContext, input: UnifiedTensor, temperature: float, out_max: UnifiedTensor,
                      out_sum: UnifiedTensor) -> None:
        """Per row of input[..., N]: the largest logit and sum exp((x - max) / temperature) (the first half of
        Sampler::sample, rusty-loader/src/tokenizer.rs:161-170)."""
        N = int(input.shape[-1])
        M = int(np.prod(input.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_softmax_stats_rows_f32(ctx.handle, input.buffer(), M, N, float(temperature), out_max.buffer(),
                                                      out_sum.buffer()), ctx.handle)

    def qlinear(self, ctx: CudaContext, x: UnifiedTensor, w: QLinear, out: UnifiedTensor) -> None:
        """out[M,N] = x[M,K] (.) w, fused dequantise + multiply."""
        m = int(np.prod(x.shape[:-1], dtype=np.int64))
        check(lib().rusty_cuda_qlinear_forward(ctx.handle, w._h, x.buffer(), int(x.dtype), m, out.buffer(),
                                               int(out.dtype)), ctx.handle)


class Event:
    """Device timestamp on the context's stream."""

    def __init__(self, ctx: CudaContext):
        h = C.c_void_p()
        check(lib().rusty_cuda_event_create(ctx.handle, C.byref(h)), ctx.handle)
        self._h, self.ctx = h, ctx

    def record(self) -> None:
        check(lib().rusty_cuda_event_record(self.ctx.handle, self._h), self.ctx.handle)

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        check(lib().rusty_cuda_event_elapsed_ms(self.ctx.handle, self._h, stop._h, C.byref(ms)), self.ctx.handle)
        return float(ms.value)

    def __del__(self):
        try:
            if self._h is not None and self.ctx._h is not None:
                lib().rusty_cuda_event_destroy(self._h)
        except Exception:
            pass
        self._h = None


class Graph:
    """A recorded sequence of operator calls, replayed with one launch."""

    def __init__(self, ctx: CudaContext):
        self.ctx = ctx
        self._h = None

    def __enter__(self) -> "Graph":
        check(lib().rusty_cuda_graph_begin(self.ctx.handle), self.ctx.handle)
        return self

    def __exit__(self, et, ev, tb) -> bool:
        h = C.c_void_p()
        rc = lib().rusty_cuda_graph_end(self.ctx.handle, C.byref(h))
        if et is None:
            check(rc, self.ctx.handle)
            self._h = h
        return False

    def launch(self) -> None:
        check(lib().rusty_cuda_graph_launch(self.ctx.handle, self._h), self.ctx.handle)

    def __del__(self):
        try:
            if self._h is not None and self.ctx._h is not None:
                lib().rusty_cuda_graph_destroy(self._h)
        except Exception:
            pass
        self._h = None


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (for asynchronous copies)."""

    def __init__(self, shape, dtype):
        self.nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        check(lib().rusty_cuda_host_alloc(self.nbytes, C.byref(p)))
        self._p = p
        buf = (C.c_uint8 * max(self.nbytes, 1)).from_address(p.value)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)

    def ptr(self) -> C.c_void_p:
        return self._p

    def free(self) -> None:
        if self._p is not None:
            self.array = None
            lib().rusty_cuda_host_free(self._p)
            self._p = None


def upload_async(ctx: CudaContext, dst: UnifiedTensor, src: PinnedArray, offset: int = 0) -> None:
    check(lib().rusty_cuda_buf_upload_async(ctx.handle, dst.buffer(), offset, src.ptr(), src.nbytes), ctx.handle)


def download_async(ctx: CudaContext, src: UnifiedTensor, dst: PinnedArray, offset: int = 0) -> None:
    check(lib().rusty_cuda_buf_download_async(ctx.handle, src.buffer(), offset, dst.ptr(), dst.nbytes), ctx.handle)


def fill_u8(ctx: CudaContext, t: UnifiedTensor, value: int = 0) -> None:
    check(lib().rusty_cuda_buf_fill_u8(ctx.handle, t.buffer(), 0, value, t.size_in_bytes()), ctx.handle)


def qlinear_forward_batch(ctx: CudaContext, qls, xs, ys, M: int, x_dtype: DType, y_dtype: DType) -> None:
    """One host call for a sequence of fused linears (a model forward's Linear loop)."""
    n = len(qls)
    arr = C.c_void_p * n
    check(lib().rusty_cuda_qlinear_forward_batch(
        ctx.handle, n, arr(*[q._h for q in qls]), arr(*[x.buffer() for x in xs]), int(x_dtype), M,
        arr(*[y.buffer() for y in ys]), int(y_dtype)), ctx.handle)
