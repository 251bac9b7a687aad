"""Builds librusty_cuda (shared + static) for sm_100a with nvcc, in-tree.

    python -m rusty_b200.build [--force] [--verbose]

Every .cu under rusty_b200/csrc is compiled to an object with
``-gencode arch=compute_100a,code=sm_100a`` and linked into
``rusty_b200/librusty_cuda.so`` (what ctypes and the tests load) and archived
into ``rusty_b200/librusty_cuda.a`` (what a Rust build script would link).
The CUDA runtime is linked statically, so the shared library depends only on
libdl/libpthread/librt and the driver's libcuda found at run time.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
SO = os.path.join(PKG, "librusty_cuda.so")
AR = os.path.join(PKG, "librusty_cuda.a")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-I", os.path.join(ROOT, "include"),
    "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: librusty_cuda cannot be built")


def _deps_mtime() -> float:
    hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(
        os.path.join(ROOT, "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    # RUSTY_TIMELINE=1 in the environment: a development build whose kernels can write %globaltimer stamps
    extra = ["-DRUSTY_TIMELINE"] if os.environ.get("RUSTY_TIMELINE") == "1" else []
    os.makedirs(OBJ, exist_ok=True)
    # objects built with other flags (a development build before a regular one, or the reverse) are all stale
    stamp = os.path.join(OBJ, "flags.txt")
    flags_now = " ".join(NVCC_FLAGS + extra)
    if not os.path.exists(stamp) or open(stamp).read() != flags_now:
        force = True
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_t = _deps_mtime()
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    with open(stamp, "w") as f:
        f.write(flags_now)
    need_link = force or jobs or not os.path.exists(SO) or not os.path.exists(AR)
    if need_link:
        subprocess.check_call([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", SO] + objs
                              + ["-cudart", "static", "-ldl", "-lpthread", "-lrt"])
        if os.path.exists(AR):
            os.remove(AR)
        subprocess.check_call(["ar", "rcs", AR] + objs)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
