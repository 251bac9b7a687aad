"""Quantised weights from safetensors files, without the f32 detour.

Host-side mirror of rusty-loader's WeightsContext (rusty-loader/src/lib.rs:97-218)
for the quantised-linear path.  The on-disk contract is the reference's: a
quantised tensor `name` is three tensors `name.weight` (bytes, shape taken
verbatim), `name.scales` and `name.biases` (f32, one pair per 64 consecutive
flat elements, lib.rs:161-187); a weight is quantised iff `name.scales` exists
(rusty-graph/src/model_builder.rs:68-72).

  * `upload_quantized(name, ctx, engine)` does what the reference does: three
    uploads, then the affine_dequantize kernel into a full f32 tensor.
  * `upload_qlinear(name, ctx, ...)` keeps the weight at one byte per element
    and returns the fused linear; with (rank, world) it uploads only this
    rank's output rows and their groups.

The safetensors container is parsed here (8-byte little-endian header length,
JSON header with dtype / shape / data_offsets, then the byte buffer); files are
memory-mapped and tensors are views, as in the reference.  `save_file` writes
the same container (synthetic checkpoints for tests, like
rusty-loader/examples/gen_dummy.rs).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from . import capi
from .backend import ComputeEngine, CudaContext, DType, QLinear, UnifiedTensor

_NP_DTYPES = {
    "U8": np.uint8, "I8": np.int8, "BOOL": np.bool_, "I16": np.int16, "U16": np.uint16, "F16": np.float16,
    "BF16": np.uint16,  # raw bits; numpy has no bfloat16
    "I32": np.int32, "U32": np.uint32, "F32": np.float32, "I64": np.int64, "U64": np.uint64, "F64": np.float64,
}
_ST_NAMES = {np.dtype(np.uint8): "U8", np.dtype(np.int8): "I8", np.dtype(np.int16): "I16", np.dtype(np.uint16): "U16",
             np.dtype(np.float16): "F16", np.dtype(np.int32): "I32", np.dtype(np.uint32): "U32",
             np.dtype(np.float32): "F32", np.dtype(np.int64): "I64", np.dtype(np.uint64): "U64",
             np.dtype(np.float64): "F64", np.dtype(np.bool_): "BOOL"}

GROUP = 64  # elements per (scale, bias) pair: hard-coded in the reference shader (kernels.wgsl:395)


class LoaderError(RuntimeError):
    """Io / Safetensors / MissingWeight of rusty-loader's LoaderError (lib.rs:15-25)."""

    def __init__(self, kind: str, message: str):
        self.kind = kind
        super().__init__(f"{kind}: {message}")


def save_file(path: str, tensors: Dict[str, np.ndarray], metadata: Optional[Dict[str, str]] = None,
              dtype_names: Optional[Dict[str, str]] = None) -> None:
    """Write a safetensors file.  `dtype_names` overrides the dtype tag of a tensor (e.g. "BF16" for uint16 bits)."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    blobs: List[bytes] = []
    off = 0
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr)
        tag = (dtype_names or {}).get(name) or _ST_NAMES.get(a.dtype)
        if tag is None:
            raise LoaderError("Safetensors", f"{name}: dtype {a.dtype} has no safetensors name")
        raw = a.tobytes()
        header[name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)  # data starts 8-byte aligned, as the reference crate writes it
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class _File:
    def __init__(self, path: str):
        try:
            size = os.path.getsize(path)
            with open(path, "rb") as f:
                head = f.read(8)
                if len(head) != 8:
                    raise LoaderError("Safetensors", f"{path}: shorter than the 8-byte header length")
                (n,) = struct.unpack("<Q", head)
                if n > size - 8 or n > (100 << 20):
                    raise LoaderError("Safetensors", f"{path}: header length {n} does not fit the file")
                raw = f.read(n)
        except OSError as e:
            raise LoaderError("Io", str(e)) from e
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise LoaderError("Json", f"{path}: {e}") from e
        if not isinstance(header, dict):
            raise LoaderError("Safetensors", f"{path}: header is not a JSON object")
        self.path = path
        self.data_start = 8 + n
        self.data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            try:
                tag, shape, (b, e) = info["dtype"], tuple(int(d) for d in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise LoaderError("Safetensors", f"{path}: malformed entry {name!r}") from ex
            if tag not in _NP_DTYPES:
                raise LoaderError("Safetensors", f"{path}: {name}: unknown dtype {tag}")
            want = int(np.prod(shape, dtype=np.int64)) * np.dtype(_NP_DTYPES[tag]).itemsize
            if not (0 <= b <= e <= self.data_len) or e - b != want:
                raise LoaderError("Safetensors", f"{path}: {name}: data_offsets [{b},{e}) do not match shape {list(shape)} {tag}")
            self.entries[name] = (tag, shape, int(b), int(e))
        # no two tensors may share bytes (the reference's safetensors crate validates the same)
        spans = sorted((b, e) for _t, _s, b, e in self.entries.values() if e > b)
        for (b0, e0), (b1, _e1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise LoaderError("Safetensors", f"{path}: tensor byte ranges overlap")
        self.mmap = np.memmap(path, dtype=np.uint8, mode="r") if size > 0 else np.zeros(0, np.uint8)

    def view(self, name: str) -> Tuple[np.ndarray, Tuple[int, ...], str]:
        tag, shape, b, e = self.entries[name]
        raw = self.mmap[self.data_start + b:self.data_start + e]
        return raw, shape, tag


class WeightsContext:
    """Memory-mapped safetensors files and a name -> file map (lib.rs:97-150)."""

    def __init__(self):
        self._files: Dict[str, _File] = {}
        self.weight_map: Dict[str, str] = {}

    def load_file(self, path: str) -> None:
        f = _File(path)
        key = os.path.basename(path)
        self._files[key] = f
        for name in f.entries:
            self.weight_map[name] = key

    def names(self) -> Iterable[str]:
        return self.weight_map.keys()

    def get_tensor_info(self, name: str) -> Optional[Tuple[List[int], str]]:
        key = self.weight_map.get(name)
        if key is None:
            return None
        tag, shape, _b, _e = self._files[key].entries[name]
        return list(shape), tag

    def read_bytes(self, name: str) -> Tuple[np.ndarray, List[int]]:
        """The tensor's bytes (a read-only view of the mapping) and its shape."""
        key = self.weight_map.get(name)
        if key is None:
            raise LoaderError("MissingWeight", name)
        raw, shape, _tag = self._files[key].view(name)
        return raw, list(shape)

    def read_array(self, name: str) -> np.ndarray:
        key = self.weight_map.get(name)
        if key is None:
            raise LoaderError("MissingWeight", name)
        raw, shape, tag = self._files[key].view(name)
        return raw.view(_NP_DTYPES[tag]).reshape(shape)

    def is_quantized(self, name: str) -> bool:
        return f"{name}.scales" in self.weight_map

    # -- the reference's load path: f32 copy made by the dequantize kernel (lib.rs:155-218) --
    def upload_quantized(self, name: str, ctx: CudaContext, engine: ComputeEngine) -> UnifiedTensor:
        q, shape, s, b = self._quantized_parts(name)
        qt = UnifiedTensor.from_bytes_with_dtype(ctx, q, [q.size], DType.U8)
        st = UnifiedTensor.new(ctx, s, [s.size])
        bt = UnifiedTensor.new(ctx, b, [b.size])
        out = UnifiedTensor.empty(ctx, shape)
        engine.affine_dequantize(ctx, qt, st, bt, out)
        return out

    # -- the fused path: the weight stays one byte per element --
    def upload_qlinear(self, name: str, ctx: CudaContext, layout: int = capi.LAYOUT_KN, rank: int = 0,
                       world: int = 1) -> QLinear:
        """`layout`: LAYOUT_KN when the stored matrix is [in,out] (what rusty's Linear multiplies by, lib.rs:69-70),
        LAYOUT_NK when it is [out,in] (HF / MLX checkpoints).  A rank's shard is a block of output features made of
        whole groups: rows of an [out,in] matrix whose input width is a multiple of 64, or columns of an [in,out] matrix
        whose output width is a multiple of 64 * world."""
        q2, s, b = self.quantized_shard(name, layout, rank, world)
        return QLinear.from_host(ctx, q2, s, b, layout=layout)

    def quantized_shard(self, name: str, layout: int = capi.LAYOUT_KN, rank: int = 0, world: int = 1):
        """Host views (weight bytes as a 2-D array, scales, biases) of the part of `name` that `rank` of `world` keeps."""
        q, shape, s, b = self._quantized_parts(name)
        if len(shape) != 2:
            raise LoaderError("Safetensors", f"{name}.weight: a linear weight has two dimensions, got {shape}")
        q2 = q.reshape(shape)
        if world > 1 and layout == capi.LAYOUT_KN:
            # [in,out] storage: the output features are the columns and the groups of 64 run along them, so a rank keeps
            # whole groups of every input row (copied: a column block is not contiguous in the file)
            k, n = shape
            if n % (world * GROUP) != 0:
                raise LoaderError("Safetensors", f"{name}: [{k},{n}] cannot be cut into {world} column shards of whole groups")
            nl, gpr = n // world, n // GROUP
            gl = nl // GROUP
            q2 = np.ascontiguousarray(q2[:, rank * nl:(rank + 1) * nl])
            s = np.ascontiguousarray(s.reshape(k, gpr)[:, rank * gl:(rank + 1) * gl]).ravel()
            b = np.ascontiguousarray(b.reshape(k, gpr)[:, rank * gl:(rank + 1) * gl]).ravel()
        elif world > 1:
            n, k = shape
            if n % world != 0 or k % GROUP != 0:
                raise LoaderError("Safetensors", f"{name}: [{n},{k}] cannot be cut into {world} row shards of whole groups")
            nl = n // world
            gpr = k // GROUP  # groups per row
            q2 = q2[rank * nl:(rank + 1) * nl]
            s = s[rank * nl * gpr:(rank + 1) * nl * gpr]
            b = b[rank * nl * gpr:(rank + 1) * nl * gpr]
        return q2, s, b

    def _quantized_parts(self, name: str):
        wn, sn, bn = f"{name}.weight", f"{name}.scales", f"{name}.biases"
        if wn not in self.weight_map:
            raise LoaderError("MissingWeight", wn)
        q, shape = self.read_bytes(wn)
        s_raw, _ = self.read_bytes(sn)
        b_raw, _ = self.read_bytes(bn)
        if s_raw.size % 4 or b_raw.size % 4:
            raise LoaderError("Safetensors", f"{name}: scales / biases are not whole f32 values")
        s, b = s_raw.view(np.float32), b_raw.view(np.float32)  # assumed f32, as lib.rs:184-187 does
        total = int(np.prod(shape, dtype=np.int64))
        if q.size != total:
            raise LoaderError("Safetensors", f"{wn}: {q.size} bytes for shape {shape}: not one byte per element")
        groups = (total + GROUP - 1) // GROUP
        if s.size < groups or b.size < groups:
            raise LoaderError("Safetensors", f"{name}: {total} elements need {groups} (scale, bias) pairs, found {s.size}/{b.size}")
        return q, shape, s[:groups] if s.size > groups else s, b[:groups] if b.size > groups else b
