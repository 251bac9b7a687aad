"""The C++ host mirror (rusty_b200/host/rusty_host.hpp): it must compile against the C ABI on any machine, and its
test program must pass on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")


def _build(tmp_path):
    exe = str(tmp_path / "host_mirror_test")
    pkg = os.path.join(ROOT, "rusty_b200")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-I",
                           os.path.join(pkg, "host"), SRC, "-o", exe, "-L", pkg, "-lrusty_cuda", f"-Wl,-rpath,{pkg}"])
    return exe


def test_host_mirror_compiles_and_links(tmp_path):
    _build(tmp_path)


@pytest.mark.gpu
def test_host_mirror_program(tmp_path):
    r = subprocess.run([_build(tmp_path)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
