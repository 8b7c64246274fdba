"""Compile and call user kernels written against the device library.

The reference's users write Triton kernels that call ``iris.load`` / ``iris.store``; here a user
kernel is CUDA C++ that includes ``<iris/iris.cuh>`` and exports a C launcher::

    #include <iris/iris.cuh>
    #include <iris/host_api.h>
    __global__ void k(iris::DeviceContext ctx, float* buf, int n, int to) {
      int i = blockIdx.x * blockDim.x + threadIdx.x;
      iris::Ctx(ctx).store(buf + i, 1.0f, to, i < n);
    }
    extern "C" int launch(const IrisCtx* c, float* buf, int n, int to, void* stream) {
      iris::DeviceContext ctx; memcpy(&ctx, c, sizeof(ctx));
      k<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(ctx, buf, n, to);
      return (int)cudaGetLastError();
    }

``compile_source`` / ``compile_file`` run nvcc for sm_100a (once per content hash, cached next to
the source or under ``~/.cache/iris_b200``) and return a ``Module``; ``module.fn("launch")(ctx, ...)``
calls the launcher, converting an ``Iris`` context to ``IrisCtx*``, tensors to device pointers and
``None`` to the current stream for a trailing ``void* stream`` argument.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
from pathlib import Path

import torch

from . import _build, _lib


class Module:
    def __init__(self, path: Path):
        self.path = Path(path)
        self.lib = C.CDLL(str(path))

    def fn(self, name: str, restype=C.c_int):
        f = getattr(self.lib, name)
        f.restype = restype

        def call(*args, stream=None):
            conv, keep = [], []
            for a in args:
                if hasattr(a, "ctx_struct"):
                    s = a.ctx_struct()
                    keep.append(s)
                    conv.append(C.byref(s))
                elif isinstance(a, _lib.IrisCtx):
                    conv.append(C.byref(a))
                elif isinstance(a, torch.Tensor):
                    conv.append(C.c_void_p(a.data_ptr()))
                elif isinstance(a, float):
                    conv.append(C.c_float(a))
                elif isinstance(a, bool):
                    conv.append(C.c_int(int(a)))
                elif isinstance(a, int):
                    conv.append(C.c_longlong(a) if abs(a) >= 2**31 else C.c_int(a))
                elif a is None:
                    conv.append(C.c_void_p(0))
                else:
                    conv.append(a)
            sp = stream.cuda_stream if stream is not None else (_lib.current_stream_ptr() if torch.cuda.is_available() else 0)
            rc = f(*conv, C.c_void_p(sp))
            if restype is C.c_int and rc != 0:
                raise RuntimeError(f"{name} returned {rc}")
            return rc

        return call


def _debug_default(debug: bool | None) -> bool:
    return (os.environ.get("IRIS_DEBUG", "0") not in ("", "0")) if debug is None else bool(debug)


def compile_file(src: str | os.PathLike, out: str | os.PathLike | None = None, verbose: bool = False,
                 debug: bool | None = None) -> Module:
    """``debug=True`` (default: ``IRIS_DEBUG=1`` in the environment) compiles with ``-DIRIS_DEBUG``: the
    object API (``iris::Ctx``) then skips and records, as status ``kBadTranslate``, every access whose
    pointer is outside the heap or whose rank does not exist; the library is written next to the
    regular one as ``lib<name>_debug.so``."""
    src = Path(src)
    debug = _debug_default(debug)
    out = Path(out) if out is not None else src.with_name("lib" + src.stem + ("_debug" if debug else "") + ".so")
    _build.build_user_kernel(src, out, verbose=verbose, defines=("IRIS_DEBUG",) if debug else ())
    return Module(out)


def compile_source(source: str, name: str = "kernel", cache_dir: str | os.PathLike | None = None, verbose: bool = False,
                   debug: bool | None = None) -> Module:
    digest = hashlib.sha256(source.encode()).hexdigest()[:16]
    cache = Path(cache_dir) if cache_dir else Path(os.environ.get("IRIS_B200_CACHE", Path.home() / ".cache" / "iris_b200"))
    cache.mkdir(parents=True, exist_ok=True)
    src = cache / f"{name}_{digest}.cu"
    if not src.exists():
        src.write_text(source)
    debug = _debug_default(debug)
    return compile_file(src, cache / f"lib{name}_{digest}{'_debug' if debug else ''}.so", verbose=verbose, debug=debug)
