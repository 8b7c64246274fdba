"""Benchmark registry: ``@register`` + ``@axis`` declare a sweep, ``State`` carries one point of it.

Usage mirrors the reference harness (iris/bench/_core.py:13-232)::

    @bench.register
    @bench.axis("num_ranks", [2, 4, 8])
    @bench.axis("M", bench.power_of_two(10, 14))
    def all_reduce(state, ctx):
        ...                      # untimed set-up for state["M"]
        state.set_bytes(nbytes)
        state.exec(lambda: ctx.ccl.all_reduce(out, inp, async_op=True))
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Callable


@dataclass
class AxisDef:
    name: str
    values: list


@dataclass
class BenchmarkDef:
    name: str
    fn: Callable
    axes: list


@dataclass
class Result:
    benchmark_name: str
    params: dict
    gpu_time_ms: float
    all_times_ms: list
    bandwidth_gbps: float | None = None
    tflops: float | None = None
    counters: dict = field(default_factory=dict)
    skipped: bool = False
    skip_reason: str = ""
    world_size: int = 1
    # additions: the timing that counts for a multi-GPU number and the roofline it is held against
    device_time_us_max_over_ranks: float | None = None
    roofline_us: float | None = None
    roofline_frac: float | None = None
    nccl_baseline_us: float | None = None       # the library form of the same work, timed by the same loop
    speedup_vs_baseline: float | None = None


registry: list[BenchmarkDef] = []


class SkipCombination(Exception):
    def __init__(self, reason: str = ""):
        super().__init__(reason)
        self.reason = reason


class State:
    """One parameter combination of a benchmark; the benchmark body is its untimed set-up."""

    def __init__(self, params: dict, n_warmup: int = 25, n_repeat: int = 100):
        self._params = dict(params)
        self._bytes = None
        self._flops = None
        self._roofline_us = None
        self._counters: dict[str, float] = {}
        self._exec_fn = None
        self._preamble_fn = None
        self._baseline_fn = None
        self._baseline_preamble_fn = None
        self.n_warmup, self.n_repeat = n_warmup, n_repeat
        self.timing = "per_call"

    def __getitem__(self, key):
        return self._params[key]

    def get(self, key, default=None):
        return self._params.get(key, default)

    @property
    def params(self) -> dict:
        return dict(self._params)

    def set_bytes(self, n: int) -> None:
        self._bytes = int(n)

    def set_flops(self, n: int) -> None:
        self._flops = int(n)

    def set_roofline_us(self, us: float) -> None:
        """Time the point cannot beat (slower of FLOPs / measured peak and link bytes / link rate)."""
        self._roofline_us = float(us)

    def add_counter(self, name: str, value: float) -> None:
        self._counters[name] = float(value)

    def set_warmup(self, n: int) -> None:
        self.n_warmup = int(n)

    def set_repeat(self, n: int) -> None:
        self.n_repeat = int(n)

    def set_timing(self, mode: str) -> None:
        """``"per_call"``: every timed call is preceded by a barrier, the preamble and an L2 flush (the
        reference's do_bench protocol; below about 1 MB it mostly measures launch skew between the ranks).
        ``"back_to_back"``: one pair of CUDA events around ``n_repeat`` calls issued without a gap after one
        barrier: the steady-state time per call, caches warm."""
        if mode not in ("per_call", "back_to_back"):
            raise ValueError("timing is 'per_call' or 'back_to_back'")
        self.timing = mode

    def exec(self, fn: Callable, preamble_fn: Callable | None = None) -> None:
        self._exec_fn, self._preamble_fn = fn, preamble_fn

    def exec_baseline(self, fn: Callable, preamble_fn: Callable | None = None) -> None:
        """Register the library form of the same work (NCCL collective, cuBLAS GEMM + NCCL, ...). It is
        timed right after ``exec``'s function with the same warm-up, repeats, cache flush and
        maximum over ranks, and reported as ``nccl_baseline_us`` with the ratio next to it."""
        self._baseline_fn, self._baseline_preamble_fn = fn, preamble_fn

    def skip(self, reason: str = "") -> None:
        raise SkipCombination(reason)


def axis(name: str, values) -> Callable:
    """Add a sweep axis; decorators closer to the function vary fastest."""
    values = list(values)

    def deco(fn):
        axes = getattr(fn, "_bench_axes", [])
        fn._bench_axes = [AxisDef(name, values)] + axes
        return fn

    return deco


def register(fn: Callable) -> Callable:
    registry.append(BenchmarkDef(fn.__name__, fn, list(getattr(fn, "_bench_axes", []))))
    return fn


def power_of_two(lo_exp: int, hi_exp: int) -> list:
    return [1 << e for e in range(lo_exp, hi_exp + 1)]


def linear_range(start: int, stop: int, step: int = 1) -> list:
    return list(range(start, stop + 1, step))


def combinations(axes: list, overrides: dict | None = None, skips: dict | None = None):
    """Cartesian product of the axes (after overrides / skips) as dicts."""
    overrides, skips = overrides or {}, skips or {}
    names, lists = [], []
    for a in axes:
        vals = list(overrides.get(a.name, a.values))
        vals = [v for v in vals if v not in skips.get(a.name, [])]
        names.append(a.name)
        lists.append(vals)
    for combo in itertools.product(*lists):
        yield dict(zip(names, combo))
