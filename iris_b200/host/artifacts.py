"""Kernel build artifacts (reference: iris/host/tracing/kernel_artifacts.py:42-281, which dumps the
Triton IR stages of every launched kernel when ``IRIS_KERNEL_ARTIFACTS_DIR`` is set).

Kernels here are compiled ahead of time by nvcc, so the artifacts are what the compiler reports:
for every translation unit the ``ptxas -v`` log and a ``metadata.json`` listing each kernel's
registers, spills, stack and static shared memory. ``collect()`` parses the logs the build left in
``build/obj``; ``export(dir)`` (or setting ``IRIS_KERNEL_ARTIFACTS_DIR`` before the first launch)
copies them under ``<dir>/<source>/``. Nothing is disassembled.

Launch records follow the reference's directory scheme: with ``IRIS_KERNEL_ARTIFACTS_DIR`` set,
every collective and fused-op launch with a configuration not seen before writes
``<dir>/<algo>/<kernel>/rank_<r>/<M>x<N>_<dtype>_w<world>/<sha12>/metadata.json`` holding the launch
parameters and what the compiler reported for the kernels of that source file, next to a copy of
its ``ptxas.log``. A configuration is written once per process; replayed launches cost one
attribute test when the directory is not set.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from pathlib import Path

import hashlib

from .. import _build

ACTIVE = bool(os.environ.get("IRIS_KERNEL_ARTIFACTS_DIR"))     # tested on the launch path
_seen: set = set()
_build_exported = False

_FUNC = re.compile(r"Compiling entry function '([^']+)' for 'sm_100a'")
_USED = re.compile(r"Used (\d+) registers(?:, used (\d+) barriers)?(?:, (\d+) bytes cumulative stack size)?(?:, (\d+) bytes smem)?")
_SPILL = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")


def parse_ptxas_log(text: str) -> list:
    """``[{name, registers, barriers, stack_bytes, spill_stores, spill_loads, smem_bytes}]`` per kernel."""
    out, cur = [], None
    for line in text.splitlines():
        m = _FUNC.search(line)
        if m:
            cur = {"name": m.group(1), "registers": None, "barriers": 0, "stack_bytes": 0, "spill_stores": 0,
                   "spill_loads": 0, "smem_bytes": 0}
            out.append(cur)
            continue
        if cur is None:
            continue
        m = _SPILL.search(line)
        if m:
            cur["stack_bytes"], cur["spill_stores"], cur["spill_loads"] = int(m.group(1)), int(m.group(2)), int(m.group(3))
        m = _USED.search(line)
        if m:
            cur["registers"] = int(m.group(1))
            cur["barriers"] = int(m.group(2) or 0)
            cur["smem_bytes"] = int(m.group(4) or 0)
    return out


def collect() -> dict:
    """Kernel metadata per source file, from the logs of the last build."""
    res = {}
    for log in sorted(_build.OBJDIR.glob("*.ptxas.log")):
        res[log.name.replace(".cu.ptxas.log", ".cu")] = parse_ptxas_log(log.read_text())
    return res


def export(directory: str | os.PathLike | None = None) -> Path | None:
    directory = directory or os.environ.get("IRIS_KERNEL_ARTIFACTS_DIR")
    if not directory:
        return None
    root = Path(directory)
    for log in sorted(_build.OBJDIR.glob("*.ptxas.log")):
        src = log.name.replace(".cu.ptxas.log", "")
        d = root / src
        d.mkdir(parents=True, exist_ok=True)
        shutil.copy(log, d / "ptxas.log")
        (d / "metadata.json").write_text(json.dumps({"source": src + ".cu", "arch": "sm_100a", "flags": _build.NVCC_FLAGS,
                                                     "kernels": parse_ptxas_log(log.read_text())}, indent=1))
    return root


def configure(directory: str | os.PathLike | None) -> None:
    """Turn launch records on (a directory) or off (``None``) for this process."""
    global ACTIVE, _build_exported
    if directory:
        os.environ["IRIS_KERNEL_ARTIFACTS_DIR"] = str(directory)
    else:
        os.environ.pop("IRIS_KERNEL_ARTIFACTS_DIR", None)
    ACTIVE = bool(directory)
    _seen.clear()
    _build_exported = False


def record_launch(algo: str, kernel: str, rank: int, params: dict, source: str | None = None) -> Path | None:
    """Write the record of one launch configuration (see the module docstring). ``params`` must be
    JSON-serialisable; ``M``, ``N``, ``dtype`` and ``world`` name the directory. ``source`` is the
    ``.cu`` file whose compile report is attached. Returns the record's directory, ``None`` when the
    configuration was already recorded or records are off."""
    global _build_exported
    directory = os.environ.get("IRIS_KERNEL_ARTIFACTS_DIR")
    if not directory:
        return None
    blob = json.dumps({"algo": algo, "kernel": kernel, "rank": rank, "params": params}, sort_keys=True, default=str)
    sha = hashlib.sha256(blob.encode()).hexdigest()[:12]
    if sha in _seen:
        return None
    _seen.add(sha)
    key = f"{params.get('M', 0)}x{params.get('N', 0)}_{str(params.get('dtype', '')).replace('torch.', '')}_w{params.get('world', 1)}"
    d = Path(directory) / algo / kernel / f"rank_{rank}" / key / sha
    d.mkdir(parents=True, exist_ok=True)
    meta = {"algo": algo, "kernel": kernel, "rank": rank, "arch": "sm_100a", "params": json.loads(json.dumps(params, default=str)),
            "source": source, "compiled": []}
    if source:
        log = _build.OBJDIR / (source + ".ptxas.log")
        if log.exists():
            shutil.copy(log, d / "ptxas.log")
            meta["compiled"] = parse_ptxas_log(log.read_text())
    (d / "metadata.json").write_text(json.dumps(meta, indent=1))
    if not _build_exported and rank == 0:
        _build_exported = True
        export(Path(directory) / "build")
    return d
