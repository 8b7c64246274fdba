"""In-tree build of the native libraries.

Two shared objects are produced under ``iris_b200/lib``:

* ``libiris_b200_kernels.so`` - every ``csrc/kernels/*.cu`` compiled by nvcc for sm_100a
  (``-gencode arch=compute_100a,code=sm_100a``), exported through the C ABI of
  ``include/iris/host_api.h``.
* ``libiris_b200_runtime.so`` - ``csrc/runtime/*.cpp`` (symmetric heap over CUDA VMM / IPC, fd
  mesh, multicast objects, CPU shared-memory backend); plain g++, libcuda is resolved at run time
  so the library also loads on a machine without a GPU.

Objects are rebuilt only when the hash of their source, the headers and the flags changes.
``python -m iris_b200._build`` builds everything; ``build_all()`` is what ``__graft_entry__.build``
calls. The reference has no native build at all (pure setuptools, pyproject.toml:4-6).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
INCLUDE = ROOT / "include"
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _cuda_include() -> str:
    return str(Path(_nvcc()).resolve().parent.parent / "include")


def _headers_hash() -> str:
    h = hashlib.sha256()
    files = [p for p in INCLUDE.rglob("*") if p.is_file()]
    files += [p for p in CSRC.rglob("*") if p.is_file() and p.suffix in (".h", ".hpp", ".cuh")]
    for p in sorted(files):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _needs(obj: Path, key: str) -> bool:
    stamp = obj.with_suffix(obj.suffix + ".hash")
    return not obj.exists() or not stamp.exists() or stamp.read_text() != key


def _stamp(obj: Path, key: str) -> None:
    obj.with_suffix(obj.suffix + ".hash").write_text(key)


def _run(cmd: list[str], log: Path | None = None) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout[-4000:], proc.stderr[-8000:]))


def _compile_cu(src: Path, hh: str, verbose: bool) -> Path:
    obj = OBJDIR / (src.stem + ".cu.o")
    key = hashlib.sha256((hh + src.read_text() + " ".join(NVCC_FLAGS)).encode()).hexdigest()
    if _needs(obj, key):
        if verbose:
            print(f"[iris_b200 build] nvcc {src.name}", flush=True)
        _run([_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{src.parent}", "-c", str(src), "-o", str(obj)], log=obj.with_suffix(".ptxas.log"))
        _stamp(obj, key)
    return obj


def _compile_cpp(src: Path, hh: str, verbose: bool) -> Path:
    obj = OBJDIR / (src.stem + ".cpp.o")
    key = hashlib.sha256((hh + src.read_text() + " ".join(CXX_FLAGS)).encode()).hexdigest()
    if _needs(obj, key):
        if verbose:
            print(f"[iris_b200 build] g++ {src.name}", flush=True)
        _run(["g++", *CXX_FLAGS, f"-I{INCLUDE}", f"-I{_cuda_include()}", "-c", str(src), "-o", str(obj)])
        _stamp(obj, key)
    return obj


def _link(objs: list[Path], out: Path, cuda: bool, verbose: bool) -> None:
    key = hashlib.sha256("".join(sorted(o.with_suffix(o.suffix + ".hash").read_text() for o in objs)).encode()).hexdigest()
    if not _needs(out, key):
        return
    if verbose:
        print(f"[iris_b200 build] link {out.name}", flush=True)
    tmp = out.with_name(out.name + f".tmp{os.getpid()}")       # processes that have the library loaded keep their copy
    if cuda:
        _run([_nvcc(), "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static", "-Xcompiler", "-fPIC"])
    else:
        _run(["g++", "-shared", "-o", str(tmp), *map(str, objs), "-ldl", "-lpthread", "-lrt"])
    os.replace(tmp, out)
    _stamp(out, key)


def kernels_lib() -> Path:
    return LIBDIR / "libiris_b200_kernels.so"


def runtime_lib() -> Path:
    return LIBDIR / "libiris_b200_runtime.so"


def build_kernels(verbose: bool = True, extra_dirs: tuple[Path, ...] = ()) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hh = _headers_hash()
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    for d in extra_dirs:
        srcs += sorted(Path(d).glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile_cu(s, hh, verbose), srcs))
    _link(objs, kernels_lib(), cuda=True, verbose=verbose)
    return kernels_lib()


def build_runtime(verbose: bool = True) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hh = _headers_hash()
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile_cpp(s, hh, verbose), srcs))
    _link(objs, runtime_lib(), cuda=False, verbose=verbose)
    return runtime_lib()


def build_user_kernel(src: Path, out: Path, verbose: bool = False, defines: tuple = ()) -> Path:
    """Compile one user ``.cu`` that includes ``<iris/iris.cuh>`` into a shared object; ``defines``
    are passed as ``-D`` (``IRIS_DEBUG`` turns on the device API's bounds checks)."""
    src, out = Path(src), Path(out)
    dflags = [f"-D{d}" for d in defines]
    key = hashlib.sha256((_headers_hash() + src.read_text() + " ".join(NVCC_FLAGS + dflags)).encode()).hexdigest()
    if _needs(out, key):
        if verbose:
            print(f"[iris_b200 build] nvcc {src.name} -> {out.name}", flush=True)
        out.parent.mkdir(parents=True, exist_ok=True)
        tmp = out.with_name(out.name + f".tmp{os.getpid()}")     # ranks may compile the same file at once
        _run([_nvcc(), *NVCC_FLAGS, *dflags, f"-I{INCLUDE}", "-shared", "-cudart", "static", str(src), "-o", str(tmp)],
             log=out.with_suffix(f".ptxas{os.getpid()}.log"))
        os.replace(tmp, out)
        _stamp(out, key)
    return out


def build_all(verbose: bool = True) -> None:
    build_runtime(verbose)
    build_kernels(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
    print("ok", kernels_lib(), runtime_lib())
    sys.exit(0)
