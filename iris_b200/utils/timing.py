"""Timing of multi-GPU work: on the device, after warm-up, maximum over ranks.

``iris_b200.do_bench`` follows the reference's protocol and returns THIS rank's times
(iris/host/platform/utils.py:137-201). A collective or a fused op is only as fast as its slowest
rank, so the figure to report is the maximum over ranks of the device-side duration;
``time_max_over_ranks`` measures that: CUDA events on the launching stream, a synchronise and a
barrier on both sides of the timed region, and one reduction of the per-rank means at the end.
On the CPU backend the host clock stands in for the events.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


def time_max_over_ranks(fn, ctx=None, n_warmup: int = 5, n_repeat: int = 20, flush_l2: bool = True, group=None) -> dict:
    """Run ``fn`` ``n_warmup + n_repeat`` times; returns ``{"ms": max over ranks of the mean time
    per call, "ms_this_rank": ..., "ms_min_over_ranks": ..., "n_repeat": ...}``.

    ``n_warmup`` is raised to 3 if smaller. With ``flush_l2`` a buffer larger than the L2 cache is
    overwritten before every timed call (outside the timed interval), so each call starts cold.
    """
    n_warmup = max(int(n_warmup), 3)
    cuda = torch.cuda.is_available() and (ctx is None or not ctx.is_cpu)
    multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1

    def sync():
        if cuda:
            torch.cuda.synchronize()
        if multi:
            dist.barrier(group=group)

    flush = None
    if cuda and flush_l2:
        from ..host.platform import _flush_l2

        dev = torch.device("cuda", torch.cuda.current_device())
        flush = lambda: _flush_l2(dev)  # noqa: E731
    for _ in range(n_warmup):
        fn()
    sync()
    total = 0.0
    if cuda:
        pairs = []
        for _ in range(n_repeat):
            if flush is not None:
                flush()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            pairs.append((s, e))
        sync()
        total = sum(s.elapsed_time(e) for s, e in pairs)
    else:
        for _ in range(n_repeat):
            t0 = time.perf_counter()
            fn()
            total += (time.perf_counter() - t0) * 1e3
        sync()
    mine = total / n_repeat
    hi = lo = mine
    if multi:
        dev = torch.device("cuda", torch.cuda.current_device()) if (cuda and "nccl" in str(dist.get_backend(group))) else "cpu"
        t = torch.tensor([mine, -mine], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        hi, lo = float(t[0]), -float(t[1])
    return {"ms": hi, "ms_this_rank": mine, "ms_min_over_ranks": lo, "n_repeat": n_repeat, "n_warmup": n_warmup}
