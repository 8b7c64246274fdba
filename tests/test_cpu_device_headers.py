"""The device header library under a plain host compiler.

``include/iris/*.cuh`` compiles for sm_100a with nvcc and, with the same source, for the host (the
CPU backend is built that way). ``tests/kernels/host_header_checks.cpp`` exercises the parts with
no device dependency: tile and tensor views, the tile-order swizzle, context decoding from the int64
tensor, address translation, every RMA function and atomic on two windows of one array, and the
bounded waits (a flag nothing sets, a barrier round nobody signals). Built a second time with
``-DIRIS_DEBUG``, the object API skips and records accesses outside the heap or to a rank that does
not exist. The reference has no host build of its device API (Triton only;
iris/mem/triton/types.py, context.py) and no debug build.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
@pytest.mark.parametrize("debug", [False, True])
def test_headers_compile_and_behave_on_the_host(tmp_path, debug):
    from iris_b200 import _build

    exe = tmp_path / "host_header_checks"
    cmd = ["g++", "-O1", "-std=c++17", "-Wall", "-Werror", "-Wno-unused-function", *(["-DIRIS_DEBUG"] if debug else []),
           f"-I{_build.INCLUDE}", f"-I{_build._cuda_include()}",
           os.path.join(ROOT, "tests", "kernels", "host_header_checks.cpp"), "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-4000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout[-4000:] + run.stderr[-2000:]
    assert "all host header checks passed" in run.stdout
    assert ("debug bounds checks active" in run.stdout) == debug


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"), reason="needs nvcc")
def test_user_kernels_cross_compile_in_debug_mode(tmp_path):
    """nvcc builds the sample user kernels for sm_100a with the bounds checks on (no GPU needed to
    compile or to load the library); the debug library is a separate file from the regular one."""
    from iris_b200 import jit

    out = tmp_path / "libuser_kernels_debug.so"
    mod = jit.compile_file(os.path.join(ROOT, "tests", "kernels", "user_kernels.cu"), out=out, debug=True)
    assert mod.path == out and out.exists() and out.stat().st_size > 0
    assert callable(mod.fn("store_blocks")) and callable(mod.fn("tile_collective"))
    log = [p for p in tmp_path.iterdir() if "ptxas" in p.name]
    assert log and "sm_100a" in log[0].read_text()
    assert jit._debug_default(None) is False and jit._debug_default(True) is True
