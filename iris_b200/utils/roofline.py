"""Roofline arithmetic against MEASURED peaks of the machine.

The denominators are measurements, not data-sheet figures: a STREAM-style copy for HBM, a cuBLAS
bf16 GEMM as a burst and as a seconds-long loop under the power cap, and a peer copy for NVLink.
``load_peaks`` reads them from ``MEASURED_PEAKS.json`` (searched in ``$IRIS_PEAKS_FILE``, the
current directory and the repository root) and falls back to earlier measurements of the same
kind of machine, flagged as such. The reference reports raw TFLOPS and GB/s only
(iris/bench/_runner.py:172-310); fractions of a measured peak are what its numbers lack.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_PEER_GBS = 770.0        # measured peer copy, per direction per GPU (nominal 900)
NVLINK_ALLREDUCE_BUS_GBS = 725.0   # measured 8-rank all-reduce bus bandwidth at 1 GiB


@dataclass
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    nvlink_gbs: float = NVLINK_PEER_GBS
    source: str = "fallback"

    @property
    def label(self) -> str:
        """The words to put beside a fraction."""
        return "of measured" if self.source != "fallback" else "of fallback"


def load_peaks(path: str | os.PathLike | None = None) -> Peaks:
    candidates = [path, os.environ.get("IRIS_PEAKS_FILE"), Path.cwd() / "MEASURED_PEAKS.json",
                  Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"]
    for c in candidates:
        if c and Path(c).is_file():
            try:
                d = json.loads(Path(c).read_text())
                return Peaks(float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                             source=str(c))
            except (ValueError, KeyError):
                continue
    return Peaks(**FALLBACK)


def gemm_flops(M: int, N: int, K: int) -> float:
    return 2.0 * M * N * K


def attention_flops(seq_q: int, seq_k: int, heads: int, head_dim: int, causal: bool = False) -> float:
    """QK^T and PV: 4 S_q S_k D per head; a causal mask keeps about half of the pairs."""
    f = 4.0 * seq_q * seq_k * heads * head_dim
    return f / 2 if causal else f


def compute_fraction(flops: float, seconds: float, peaks: Peaks | None = None, sustained: bool = False) -> float:
    """Achieved FLOP/s over the measured bf16 GEMM rate (burst for a kernel timed alone, sustained
    for a kernel inside a long step)."""
    p = peaks or load_peaks()
    peak = (p.bf16_tflops_sustained if sustained else p.bf16_tflops) * 1e12
    return flops / seconds / peak


def memory_fraction(nbytes: float, seconds: float, peaks: Peaks | None = None) -> float:
    p = peaks or load_peaks()
    return nbytes / seconds / (p.hbm_gbs * 1e9)


def fused_target_seconds(flops: float, link_bytes: float, peaks: Peaks | None = None, sustained: bool = True) -> float:
    """Roofline of a fused compute + collective kernel: the slower of the math at the measured GEMM
    rate and the bytes that must cross NVLink (per direction, per GPU) at the measured link rate."""
    p = peaks or load_peaks()
    peak = (p.bf16_tflops_sustained if sustained else p.bf16_tflops) * 1e12
    return max(flops / peak, link_bytes / (p.nvlink_gbs * 1e9))


def collective_link_bytes(op: str, nbytes: float, world: int) -> float:
    """Bytes each GPU must send (= receive) for a collective over ``nbytes`` of payload per rank:
    all_gather / reduce_scatter / all_to_all move (W-1)/W of the full payload, all_reduce twice that
    (once with in-switch reduction, which halves what crosses each link)."""
    if world <= 1:
        return 0.0
    frac = (world - 1) / world
    if op == "all_reduce":
        return 2 * frac * nbytes
    if op == "all_reduce_nvls":
        return nbytes
    if op in ("all_gather", "reduce_scatter", "all_to_all"):
        return frac * nbytes
    raise ValueError(f"unknown collective {op!r}")
