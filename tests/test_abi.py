"""CPU tests of the C-ABI boundary: the shared library loads, exports every
symbol the header declares, and refuses to work without a CUDA device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"RUSTY_CUDA_API\s+[\w\s\*]+?\b(rusty_cuda_\w+)\s*\(", text)
    return names


def test_header_declares_entry_points():
    names = _declared_symbols()
    for must in ("rusty_cuda_ctx_create", "rusty_cuda_matmul_f32", "rusty_cuda_matmul_bt_f32", "rusty_cuda_dequantize_u8",
                 "rusty_cuda_affine_dequantize_g64", "rusty_cuda_qlinear_forward"):
        assert must in names
    assert len(names) == len(set(names))


def test_library_exports_every_declared_symbol():
    from rusty_b200 import capi
    assert os.path.exists(capi.LIB_PATH), "librusty_cuda.so is not built (python -m rusty_b200.build)"
    raw = C.CDLL(capi.LIB_PATH)
    for name in _declared_symbols():
        assert hasattr(raw, name), f"{name} declared in include/ but not exported"


def test_binding_covers_every_declared_symbol():
    from rusty_b200 import capi
    assert set(capi.SIGNATURES) == set(_declared_symbols())
    capi.lib()


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "rusty_cuda.h"\nint main(void){return RUSTY_CUDA_OK;}\n')
    import subprocess
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                           str(tmp_path / "t.o")])


def test_static_archive_holds_the_same_entry_points():
    import subprocess
    ar = os.path.join(ROOT, "rusty_b200", "librusty_cuda.a")
    assert os.path.exists(ar)
    syms = subprocess.run(["nm", "-g", "--defined-only", ar], capture_output=True, text=True).stdout
    for name in _declared_symbols():
        assert re.search(rf"\bT {name}\b", syms), name


def test_no_device_means_loud_failure():
    """Without a GPU nothing computes: context creation reports GpuInitialization."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import rusty_b200
    with pytest.raises(rusty_b200.BackendError) as e:
        rusty_b200.CudaContext(0)
    assert e.value.kind == "GpuInitialization"


def test_null_handles_are_rejected_not_dereferenced():
    from rusty_b200 import capi
    l = capi.lib()
    assert l.rusty_cuda_sync(None) == capi.ERR_INVALID_OPERATION
    assert l.rusty_cuda_buf_release(None) == capi.OK
    assert l.rusty_cuda_qlinear_destroy(None) == capi.OK
    n = C.c_size_t()
    assert l.rusty_cuda_buf_size(None, C.byref(n)) == capi.ERR_INVALID_OPERATION
    assert b"null" in l.rusty_cuda_last_error(None)


def test_product_package_does_not_import_the_oracle():
    """The oracle is test infrastructure; nothing under rusty_b200/ may touch it."""
    pkg = os.path.join(ROOT, "rusty_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        if "build" in dirpath.split(os.sep)[-1:]:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".hpp", ".cuh", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f
                assert "liboracle" not in text and "rusty_oracle" not in text, f


def test_static_entry_status_word_decodes_on_the_host():
    """The allocation-free entry point reports a device-side wait that gave up through a status word; the mapping
    from that word to a status code is host code and needs no GPU."""
    from rusty_b200 import capi
    lib = capi.lib()
    assert lib.rusty_cuda_qlinear_i8_static_status_decode(0, 0) == capi.OK
    assert lib.rusty_cuda_qlinear_i8_static_status_decode(1, 8) == capi.ERR_TIMEOUT
    assert b"site 8" in lib.rusty_cuda_last_error(None)
