"""The device header library under a plain host compiler.

``include/iris/*.cuh`` compiles for sm_100a with nvcc and, with the same source, for the host (the
CPU backend is built that way). ``tests/kernels/host_header_checks.cpp`` exercises the parts with
no device dependency: tile and tensor views, the tile-order swizzle, context decoding from the int64
tensor, address translation, every RMA function and atomic on two windows of one array, and the
bounded waits (a flag nothing sets, a barrier round nobody signals). The reference has no host
build of its device API (Triton only; iris/mem/triton/types.py, context.py).
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_headers_compile_and_behave_on_the_host(tmp_path):
    from iris_b200 import _build

    exe = tmp_path / "host_header_checks"
    cmd = ["g++", "-O1", "-std=c++17", "-Wall", "-Werror", "-Wno-unused-function", f"-I{_build.INCLUDE}", f"-I{_build._cuda_include()}",
           os.path.join(ROOT, "tests", "kernels", "host_header_checks.cpp"), "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-4000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout[-4000:] + run.stderr[-2000:]
    assert "all host header checks passed" in run.stdout
