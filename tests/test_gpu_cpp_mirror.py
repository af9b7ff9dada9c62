"""Builds the C++ host mirror test (tests/cpp/kvcache_test.cpp over include/relux_cuda.hpp) against
librelux_cuda.so; the CPU test checks that it compiles and links, the GPU test runs it."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "kvcache_test")


def _build():
    import __graft_entry__ as g
    g.build()
    so_dir = os.path.join(ROOT, "relux_b200")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "kvcache_test.cpp"),
                           "-o", EXE, "-L", so_dir, "-l:librelux_cuda.so", "-Wl,-rpath," + so_dir])
    return EXE


def test_cpp_mirror_compiles_and_links():
    assert os.path.exists(_build())


@pytest.mark.gpu
def test_cpp_mirror_replays_reference_kvcache_tests():
    exe = _build()
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "ALL PASSED" in out.stdout, out.stdout + out.stderr
