"""ctypes binding of ``librusty_cuda.so`` — the C ABI in ``include/rusty_cuda.h``.

The signatures below are the same ones a Rust ``extern "C"`` block inside
rusty-backend would declare.  Loading fails loudly when the shared library has
not been built; there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "librusty_cuda.so")

# status codes (rusty_cuda.h)
OK = 0
ERR_GPU_INITIALIZATION = 1
ERR_MEMORY_ALLOCATION = 2
ERR_INVALID_DIMENSIONS = 3
ERR_INVALID_DATA_TYPE = 4
ERR_BUFFER_OPERATION = 5
ERR_KERNEL_EXECUTION = 6
ERR_UNSUPPORTED = 7
ERR_DATA_TRANSFER = 8
ERR_INVALID_OPERATION = 9
ERR_TIMEOUT = 10
ERR_OTHER = 11

STATUS_NAMES = {
    0: "Ok", 1: "GpuInitialization", 2: "MemoryAllocation", 3: "InvalidDimensions", 4: "InvalidDataType",
    5: "BufferOperation", 6: "KernelExecution", 7: "UnsupportedOperation", 8: "DataTransfer",
    9: "InvalidOperation", 10: "Timeout", 11: "Other",
}

F32, F16, BF16, I8, U8 = 0, 1, 2, 3, 4
QMODE_AFFINE_G64, QMODE_SYM_ROW = 0, 1
LAYOUT_NK, LAYOUT_KN = 0, 1
ACT_NONE, ACT_SWIGLU_PAIRS = 0, 1

_vp = C.c_void_p
_vpp = C.POINTER(C.c_void_p)
_sz = C.c_size_t
_u32 = C.c_uint32
_int = C.c_int

# name -> (argtypes, restype); every symbol rusty_cuda.h declares.
SIGNATURES = {
    "rusty_cuda_device_count": ([C.POINTER(_int)], _int),
    "rusty_cuda_ctx_create": ([_int, _vpp], _int),
    "rusty_cuda_ctx_destroy": ([_vp], _int),
    "rusty_cuda_ctx_adapter_info": ([_vp, C.c_char_p, _sz], _int),
    "rusty_cuda_last_error": ([_vp], C.c_char_p),
    "rusty_cuda_sync": ([_vp], _int),
    "rusty_cuda_ctx_self_check": ([_vp], _int),
    "rusty_cuda_ctx_launch_count": ([_vp, C.POINTER(C.c_uint64)], _int),
    "rusty_cuda_ctx_stream": ([_vp, _vpp], _int),
    "rusty_cuda_buf_alloc": ([_vp, _sz, _int, _vpp], _int),
    "rusty_cuda_buf_retain": ([_vp], _int),
    "rusty_cuda_buf_release": ([_vp], _int),
    "rusty_cuda_buf_size": ([_vp, C.POINTER(_sz)], _int),
    "rusty_cuda_buf_device_ptr": ([_vp, _vpp], _int),
    "rusty_cuda_buf_upload": ([_vp, _vp, _sz, _vp, _sz], _int),
    "rusty_cuda_buf_download": ([_vp, _vp, _sz, _vp, _sz], _int),
    "rusty_cuda_buf_copy": ([_vp, _vp, _vp, _sz], _int),
    "rusty_cuda_pool_clear": ([_vp], _int),
    "rusty_cuda_pool_idle_count": ([_vp, _sz, C.POINTER(_sz)], _int),
    "rusty_cuda_host_alloc": ([_sz, _vpp], _int),
    "rusty_cuda_host_free": ([_vp], _int),
    "rusty_cuda_buf_upload_async": ([_vp, _vp, _sz, _vp, _sz], _int),
    "rusty_cuda_buf_download_async": ([_vp, _vp, _sz, _vp, _sz], _int),
    "rusty_cuda_matmul_f32": ([_vp, _vp, _vp, _vp, _u32, _u32, _u32], _int),
    "rusty_cuda_matmul_bt_f32": ([_vp, _vp, _vp, _vp, _u32, _u32, _u32], _int),
    "rusty_cuda_dequantize_u8": ([_vp, _vp, _vp, _sz], _int),
    "rusty_cuda_affine_dequantize_g64": ([_vp, _vp, _vp, _vp, _vp, _sz], _int),
    "rusty_cuda_add_f32": ([_vp, _vp, _vp, _vp, _sz], _int),
    "rusty_cuda_qlinear_create": ([_vp, _vp, _vp, _vp, _u32, _u32, _int, _int, _vpp], _int),
    "rusty_cuda_qlinear_destroy": ([_vp], _int),
    "rusty_cuda_qlinear_forward": ([_vp, _vp, _vp, _int, _u32, _vp, _int], _int),
    "rusty_cuda_qlinear_forward_batch": ([_vp, _sz, _vpp, _vpp, _int, _u32, _vpp, _int], _int),
    "rusty_cuda_qlinear_i8_forward_static": ([_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp], _int),
    "rusty_cuda_qlinear_i8_static_status": ([_vp], _int),
    "rusty_cuda_qlinear_i8_static_status_decode": ([C.c_uint, C.c_uint], _int),
    "rusty_cuda_comm_unique_id": ([_vp], _int),
    "rusty_cuda_comm_create": ([_vp, _int, _int, _vp, _vpp], _int),
    "rusty_cuda_comm_destroy": ([_vp], _int),
    "rusty_cuda_comm_check": ([_vp], _int),
    "rusty_cuda_qlinear_forward_sharded": ([_vp, _vp, _vp, _vp, _int, _u32, _vp, _vp, _int], _int),
    "rusty_cuda_qlinear_forward_sharded_batch": ([_vp, _vp, _sz, _vpp, _vpp, _int, _u32, _vp, _vpp, _int], _int),
    "rusty_cuda_silu_f32": ([_vp, _vp, _vp, _sz], _int),
    "rusty_cuda_mul_f32": ([_vp, _vp, _vp, _vp, _sz], _int),
    "rusty_cuda_qlinear_set_activation": ([_vp, _int], _int),
    "rusty_cuda_arena_create": ([_vp, _sz, _int, _int, _vpp], _int),
    "rusty_cuda_arena_export": ([_vp, _vp], _int),
    "rusty_cuda_arena_attach": ([_vp, _vp], _int),
    "rusty_cuda_arena_buf": ([_vp, _sz, _sz, _vpp], _int),
    "rusty_cuda_arena_wait": ([_vp, _vp], _int),
    "rusty_cuda_arena_destroy": ([_vp], _int),
    "rusty_cuda_qlinear_forward_pushed": ([_vp, _vp, _vp, _vp, _int, _u32, _vp, _int], _int),
    "rusty_cuda_qlinear_forward_pushed_batch": ([_vp, _vp, _sz, _vpp, _vpp, _int, _u32, _vpp, _int], _int),
    "rusty_cuda_embedding_f32": ([_vp, _vp, _vp, _vp, _sz, _u32, _u32], _int),
    "rusty_cuda_rms_norm_f32": ([_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, C.c_float], _int),
    "rusty_cuda_qlinear_forward_normed": ([_vp, _vp, _vp, _vp, _vp, C.c_float, _u32, _vp, _vp, _vp, _int], _int),
    "rusty_cuda_qlinear_forward_residual": ([_vp, _vp, _vp, _int, _u32, _vp, _vp, _int], _int),
    "rusty_cuda_argmax_rows_f32": ([_vp, _vp, _u32, _u32, _vp, _vp], _int),
    "rusty_cuda_argmax_rows_sharded": ([_vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp], _int),
    "rusty_cuda_top_k_rows_f32": ([_vp, _vp, _u32, _u32, _u32, _vp, _vp], _int),
    "rusty_cuda_softmax_stats_rows_f32": ([_vp, _vp, _u32, _u32, C.c_float, _vp, _vp], _int),
    "rusty_cuda_top_k_rows_sharded": ([_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp], _int),
    "rusty_cuda_graph_begin": ([_vp], _int),
    "rusty_cuda_graph_end": ([_vp, _vpp], _int),
    "rusty_cuda_graph_launch": ([_vp, _vp], _int),
    "rusty_cuda_graph_destroy": ([_vp], _int),
    "rusty_cuda_event_create": ([_vp, _vpp], _int),
    "rusty_cuda_event_record": ([_vp, _vp], _int),
    "rusty_cuda_event_elapsed_ms": ([_vp, _vp, _vp, C.POINTER(C.c_float)], _int),
    "rusty_cuda_event_destroy": ([_vp], _int),
    "rusty_cuda_buf_fill_u8": ([_vp, _vp, _sz, _int, _sz], _int),
    "rusty_cuda_qlinear_plan": ([_vp, _int, _u32, _int, C.c_char_p, _sz], _int),
}

_lib = None


class BackendError(RuntimeError):
    """A non-zero status from the C ABI; ``code`` is the RUSTY_CUDA_ERR_* value
    and ``kind`` the matching rusty BackendError variant name."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.kind = STATUS_NAMES.get(code, "Other")
        super().__init__(f"{self.kind} ({code}): {message}")


def lib() -> C.CDLL:
    """Load librusty_cuda.so (once) and attach the declared signatures."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m rusty_b200.build` "
                "(needs nvcc; there is no CPU or PyTorch fallback)")
        l = C.CDLL(LIB_PATH)
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(l, name)  # AttributeError here = header and library disagree
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = l
    return _lib


def check(rc: int, ctx=None) -> None:
    if rc != OK:
        msg = lib().rusty_cuda_last_error(ctx)
        raise BackendError(rc, msg.decode("utf-8", "replace") if msg else "")
