"""rusty_b200 — B200 (sm_100a) backend for rusty's quantized-linear path.

``csrc/``      CUDA kernels and the C ABI (include/rusty_cuda.h), built into
               ``librusty_cuda.so`` / ``.a`` by ``python -m rusty_b200.build``.
``capi``       ctypes binding of that ABI.
``backend``    host mirror of rusty-backend's WgpuContext / UnifiedTensor /
               ComputeEngine surface.
``graph``      host mirror of rusty-graph's Linear / LoRAAdapter.
``workloads``  seeded synthetic inputs with the shapes the benchmarks name.
"""
from .capi import BackendError, LIB_PATH  # noqa: F401
from .backend import CudaContext, ComputeEngine, DType, QLinear, UnifiedTensor  # noqa: F401
from .graph import Linear, LoRAAdapter  # noqa: F401
