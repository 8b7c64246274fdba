"""ctypes bindings of the two native libraries (see ``_build.py``).

``kernels()`` returns ``libiris_b200_kernels.so`` (sm_100a kernels, needs a GPU to be useful),
``runtime()`` returns ``libiris_b200_runtime.so`` (heap / fd mesh / CPU backend, loads anywhere).
Both are built in-tree on first use when the shared object is missing; on a machine with a GPU a
missing or unloadable kernel library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

from . import _build

MAX_RANKS = 72

_lock = threading.Lock()
_kernels = None
_runtime = None


class IrisCtx(C.Structure):
    """Mirror of ``IrisCtx`` in include/iris/host_api.h (= iris::DeviceContext)."""

    _fields_ = [
        ("rank", C.c_int32),
        ("world", C.c_int32),
        ("heap_size", C.c_uint64),
        ("mc_base", C.c_uint64),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("trace_enabled", C.c_int32),
        ("trace_max_events", C.c_int32),
        ("trace_ptrs", C.c_void_p * 15),
        ("bases", C.c_uint64 * MAX_RANKS),
    ]


class IrisGemmDesc(C.Structure):
    _fields_ = [
        ("op", C.c_int32),
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("dtype", C.c_int32),
        ("b_kmajor", C.c_int32),
        ("bn", C.c_int32),
        ("group_m", C.c_int32),
        ("gemm_ctas", C.c_int32),
        ("comm_ctas", C.c_int32),
        ("use_mc", C.c_int32),
        ("two_sm", C.c_int32),
        ("A", C.c_void_p), ("lda", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64),
        ("C", C.c_void_p), ("ldc", C.c_int64),
        ("bias_row", C.c_void_p),
        ("bias_col", C.c_void_p),
        ("ctx", IrisCtx),
        ("sync_block", C.c_void_p),
        ("inbox", C.c_void_p),
        ("flags", C.c_void_p),
        ("staging", C.c_void_p),
        ("M_local", C.c_int32),
        ("K_local", C.c_int32),
        ("timeline", C.c_void_p),
        ("in_dtype", C.c_int32),
        ("sf_a", C.c_void_p),
        ("sf_b", C.c_void_p),
        ("sf_inbox", C.c_void_p),
        ("overlap", C.c_int32),
    ]


DTYPE_CODE = {
    torch.float16: 0, torch.bfloat16: 1, torch.float32: 2, torch.int32: 3, torch.int8: 4,
    torch.int64: 6,
}
if hasattr(torch, "float8_e4m3fn"):
    DTYPE_CODE[torch.float8_e4m3fn] = 5

GEMM_LOCAL, GEMM_AG_M, GEMM_AG_K, GEMM_ALL_GATHER, GEMM_REDUCE_SCATTER, GEMM_ALL_REDUCE, GEMM_ALL_SCATTER, GEMM_RS_TILES = range(8)
GEMM_AR_ONE_SHOT, GEMM_AR_ATOMIC = 8, 9


def _load(path, builder):
    if not os.path.exists(path) or os.environ.get("IRIS_B200_REBUILD") == "1":
        builder(verbose=os.environ.get("IRIS_B200_BUILD_VERBOSE", "0") == "1")
    return C.CDLL(str(path), mode=C.RTLD_GLOBAL)


def runtime() -> C.CDLL:
    global _runtime
    with _lock:
        if _runtime is None:
            _runtime = _load(_build.runtime_lib(), _build.build_runtime)
        return _runtime


def kernels() -> C.CDLL:
    """The sm_100a kernel library. Raises if it cannot be built or loaded."""
    global _kernels
    with _lock:
        if _kernels is None:
            lib = _load(_build.kernels_lib(), _build.build_kernels)
            lib.iris_gemm_launch.argtypes = [C.POINTER(IrisGemmDesc), C.c_void_p]
            lib.iris_gemm_launch.restype = C.c_int
            lib.iris_gemm_workspace.argtypes = [C.POINTER(IrisGemmDesc), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                                C.POINTER(C.c_uint64), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
            lib.iris_gemm_workspace.restype = C.c_int
            lib.iris_gemm_sf_inbox_bytes.argtypes = [C.POINTER(IrisGemmDesc)]
            lib.iris_gemm_sf_inbox_bytes.restype = C.c_uint64
            _kernels = lib
        return _kernels


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


# Kernels of this library launched by this process, by entry point ("all_gather_matmul",
# "collective", "gemm", ...). Every launch path goes through `check(..., kernels=n)`; benchmarks report
# the difference of `launch_count()` around their timed region.
LAUNCHES: dict = {}


def launch_count() -> int:
    return sum(LAUNCHES.values())


def check(code: int, what: str, kernels: int = 0) -> None:
    """Raise on a non-zero return code of a native call; `kernels` is the number of GPU kernels the
    call launched when it succeeded (counted in `LAUNCHES` under `what`)."""
    if code != 0:
        raise RuntimeError(f"iris_b200: {what} failed with code {code}")
    if kernels:
        LAUNCHES[what] = LAUNCHES.get(what, 0) + kernels
