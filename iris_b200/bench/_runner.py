"""Runner of the benchmark harness: command line, one process per rank, timing, formatting.

``bench.main()`` parses ``--benchmark_filter --benchmark_format --benchmark_out --heap_size
--n_warmup --n_repeat --axis_<name>=... --skip_<name>=...`` (axis values: a comma list,
``pow2:a:b`` or ``lin:a:b:s``; dtype names are resolved), launches ``num_ranks`` processes on this
host with ``torch.multiprocessing`` for each distinct rank count and prints console / JSON / CSV
(reference: iris/bench/_runner.py:35-595). When the program is already running under ``torchrun``
(``WORLD_SIZE`` set) the existing ranks are used instead of spawning. Times are CUDA-event times;
the figure reported for a multi-rank point is the maximum over ranks of the per-rank mean.
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import os
import re
import socket
import sys

import torch

from ._core import Result, SkipCombination, State, combinations, registry

_DTYPES = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "int32": torch.int32, "int8": torch.int8}


def dtype_str(v) -> str:
    return str(v).replace("torch.", "") if isinstance(v, torch.dtype) else str(v)


def parse_axis_values(raw: str, axis_name: str = "") -> list:
    """``"1,2,4"`` | ``"pow2:10:14"`` | ``"lin:0:64:16"`` | ``"bf16,fp32"``."""
    raw = raw.strip()
    m = re.fullmatch(r"pow2:(-?\d+):(-?\d+)", raw)
    if m:
        return [1 << e for e in range(int(m.group(1)), int(m.group(2)) + 1)]
    m = re.fullmatch(r"lin:(-?\d+):(-?\d+)(?::(-?\d+))?", raw)
    if m:
        return list(range(int(m.group(1)), int(m.group(2)) + 1, int(m.group(3) or 1)))
    out = []
    for tok in (t.strip() for t in raw.split(",") if t.strip()):
        if tok in _DTYPES:
            out.append(_DTYPES[tok])
        elif re.fullmatch(r"-?\d+", tok):
            out.append(int(tok))
        elif re.fullmatch(r"-?\d*\.\d+(e-?\d+)?", tok):
            out.append(float(tok))
        elif tok.lower() in ("true", "false"):
            out.append(tok.lower() == "true")
        else:
            out.append(tok)
    if not out:
        raise ValueError(f"axis {axis_name}: no values in {raw!r}")
    return out


def format_console(results: list) -> str:
    lines = []
    by_bench: dict[str, list] = {}
    for r in results:
        by_bench.setdefault(r.benchmark_name, []).append(r)
    for name, rs in by_bench.items():
        keys = list(rs[0].params.keys())
        with_base = any(r.nccl_baseline_us is not None for r in rs)
        header = keys + ["time_us(max/ranks)", "GB/s", "TFLOPS", "roofline%"] + (["baseline_us", "speedup"] if with_base else [])
        rows = []
        for r in rs:
            if r.skipped:
                rows.append([dtype_str(r.params[k]) for k in keys] + [f"skipped: {r.skip_reason}", "", "", ""] + (["", ""] if with_base else []))
                continue
            rows.append([dtype_str(r.params[k]) for k in keys] + [
                f"{r.gpu_time_ms * 1e3:.2f}",
                f"{r.bandwidth_gbps:.1f}" if r.bandwidth_gbps is not None else "",
                f"{r.tflops:.1f}" if r.tflops is not None else "",
                f"{100 * r.roofline_frac:.0f}" if r.roofline_frac is not None else "",
            ] + ([f"{r.nccl_baseline_us:.2f}" if r.nccl_baseline_us is not None else "",
                  f"{r.speedup_vs_baseline:.2f}" if r.speedup_vs_baseline is not None else ""] if with_base else []))
        widths = [max(len(str(x)) for x in col) for col in zip(header, *rows)]
        lines.append(f"== {name} ==")
        lines.append("  ".join(str(h).ljust(w) for h, w in zip(header, widths)))
        for row in rows:
            lines.append("  ".join(str(c).ljust(w) for c, w in zip(row, widths)))
        lines.append("")
    return "\n".join(lines)


def _result_dict(r: Result) -> dict:
    return {
        "benchmark": r.benchmark_name, "params": {k: dtype_str(v) for k, v in r.params.items()}, "world_size": r.world_size,
        "gpu_time_ms": r.gpu_time_ms, "device_time_us_max_over_ranks": r.device_time_us_max_over_ranks,
        "bandwidth_gbps": r.bandwidth_gbps, "tflops": r.tflops, "roofline_us": r.roofline_us,
        "roofline_frac": r.roofline_frac, "nccl_baseline_us": r.nccl_baseline_us, "speedup_vs_baseline": r.speedup_vs_baseline,
        "counters": r.counters, "skipped": r.skipped, "skip_reason": r.skip_reason,
    }


def format_json(results: list) -> str:
    return json.dumps({"results": [_result_dict(r) for r in results]}, indent=2)


def format_csv(results: list) -> str:
    buf = io.StringIO()
    keys = sorted({k for r in results for k in r.params})
    w = csv.writer(buf)
    w.writerow(["benchmark", "world_size"] + keys + ["gpu_time_ms", "bandwidth_gbps", "tflops", "roofline_frac", "skipped",
                                                       "nccl_baseline_us", "speedup_vs_baseline"])
    for r in results:
        w.writerow([r.benchmark_name, r.world_size] + [dtype_str(r.params.get(k, "")) for k in keys] +
                   [r.gpu_time_ms, r.bandwidth_gbps or "", r.tflops or "", r.roofline_frac or "", int(r.skipped),
                    r.nccl_baseline_us or "", r.speedup_vs_baseline or ""])
    return buf.getvalue()


def run_benchmarks(ctx, benchmarks, overrides, skips, n_warmup, n_repeat) -> list:
    """Run every combination on the already-initialised ranks; every rank returns the same list."""
    import torch.distributed as dist

    from ..host.platform import do_bench

    def timed(state, fn, preamble):
        """Milliseconds per call on this rank, as a list (one entry per timed call, or one mean)."""
        if state.timing == "back_to_back" and not ctx.is_cpu:
            pre = preamble or (lambda: None)
            pre()
            for _ in range(max(state.n_warmup, 1)):
                fn()
            ctx.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(state.n_repeat):
                fn()
            e.record()
            torch.cuda.synchronize()
            return [s.elapsed_time(e) / state.n_repeat]
        return do_bench(fn, barrier_fn=ctx.barrier, preamble_fn=preamble or (lambda: None), n_warmup=state.n_warmup,
                        n_repeat=state.n_repeat, return_mode="all")

    results = []
    world = ctx.get_num_ranks()
    # the heap is a bump allocator: take what outlives a point (the collectives' sync block) first,
    # then rewind to this mark after every point
    ctx.device_barrier()
    ctx.sync_block(("ccl", None))
    mark = ctx.heap_mark()
    for bdef in benchmarks:
        for params in combinations(bdef.axes, overrides, skips):
            if params.get("num_ranks", world) != world:
                continue
            ctx.heap_release(mark)
            state = State(params, n_warmup, n_repeat)
            try:
                bdef.fn(state, ctx)
            except SkipCombination as s:
                results.append(Result(bdef.name, params, 0.0, [], skipped=True, skip_reason=s.reason, world_size=world))
                continue
            except MemoryError as e:
                # the symmetric heap is too small for this point: every rank runs the same allocation sequence
                # and fails alike, so the sweep goes on with the next point (--heap_size raises the limit)
                results.append(Result(bdef.name, params, 0.0, [], skipped=True, skip_reason=f"heap too small ({e})"[:120], world_size=world))
                continue
            if state._exec_fn is None:
                results.append(Result(bdef.name, params, 0.0, [], skipped=True, skip_reason="no exec() registered", world_size=world))
                continue
            if "timing" in params:
                state.set_timing(params["timing"])
            times = timed(state, state._exec_fn, state._preamble_fn)
            mean_ms = sum(times) / len(times)
            t = torch.tensor([mean_ms], dtype=torch.float64, device=ctx.device if not ctx.is_cpu else "cpu")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            r = Result(bdef.name, params, ms, times, world_size=world, counters=dict(state._counters))
            r.device_time_us_max_over_ranks = ms * 1e3
            if state._bytes is not None and ms > 0:
                r.bandwidth_gbps = state._bytes / 1e9 / (ms / 1e3)
            if state._flops is not None and ms > 0:
                r.tflops = state._flops / 1e12 / (ms / 1e3)
            if state._roofline_us is not None and ms > 0:
                r.roofline_us = state._roofline_us
                r.roofline_frac = state._roofline_us / (ms * 1e3)
            if state._baseline_fn is not None:
                base = timed(state, state._baseline_fn, state._baseline_preamble_fn)
                tb = torch.tensor([sum(base) / len(base)], dtype=torch.float64, device=ctx.device if not ctx.is_cpu else "cpu")
                if world > 1:
                    dist.all_reduce(tb, op=dist.ReduceOp.MAX)
                r.nccl_baseline_us = float(tb.item()) * 1e3
                r.speedup_vs_baseline = r.nccl_baseline_us / (ms * 1e3) if ms > 0 else None
            results.append(r)
    return results


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, script, names, overrides, skips, n_warmup, n_repeat, heap_size, queue):
    import runpy

    import torch.distributed as dist

    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(rank % torch.cuda.device_count())
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank % torch.cuda.device_count()) if cuda else None)
    import iris_b200

    if script and not registry:
        runpy.run_path(script, run_name="__iris_bench__")
    ctx = iris_b200.iris(heap_size)
    benchmarks = [b for b in registry if b.name in names]
    res = run_benchmarks(ctx, benchmarks, overrides, skips, n_warmup, n_repeat)
    if rank == 0:
        queue.put([_result_dict(r) for r in res])
    ctx.barrier()
    dist.destroy_process_group()


def _collect(q, procs, grace_s: float = 15.0) -> list:
    """Results of rank 0, or an error as soon as a worker has died: a rank that fails (an oracle that
    does not hold, an exception in a benchmark body) leaves the others waiting in a barrier, so they get
    ``grace_s`` seconds to finish on their own and are then terminated (the processes started here, by
    handle), instead of the launcher waiting for a result that will never come."""
    import queue as _queue
    import time

    failed_at = None
    while True:
        try:
            return q.get(timeout=0.5)
        except _queue.Empty:
            pass
        codes = [p.exitcode for p in procs]
        if any(c not in (None, 0) for c in codes) and failed_at is None:
            failed_at = time.time()
        if all(c is not None for c in codes) or (failed_at is not None and time.time() - failed_at > grace_s):
            try:
                return q.get(timeout=0.5)          # rank 0 may have delivered just before exiting
            except _queue.Empty:
                pass
            for p in procs:
                if p.is_alive():
                    p.terminate()
            for p in procs:
                p.join(10)
            bad = {i: p.exitcode for i, p in enumerate(procs) if p.exitcode != 0}
            raise RuntimeError(f"benchmark workers failed (rank: exit code) {bad}; see their output above")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="iris_b200 benchmark runner", allow_abbrev=False)
    p.add_argument("--benchmark_filter", default=None, help="regular expression on benchmark names")
    p.add_argument("--benchmark_format", default="console", choices=["console", "json", "csv"])
    p.add_argument("--benchmark_out", default=None, help="also write the formatted results to this file")
    p.add_argument("--heap_size", type=int, default=1 << 33)
    p.add_argument("--n_warmup", type=int, default=25)
    p.add_argument("--n_repeat", type=int, default=100)
    p.add_argument("--use_gluon", action="store_true", help="accepted for compatibility; ignored")
    return p


def main(argv: list | None = None) -> list:
    argv = list(sys.argv[1:] if argv is None else argv)
    overrides, skips, rest = {}, {}, []
    for a in argv:
        m = re.fullmatch(r"--(axis|skip)_([A-Za-z0-9_]+)=(.*)", a)
        if m:
            (overrides if m.group(1) == "axis" else skips)[m.group(2)] = parse_axis_values(m.group(3), m.group(2))
        else:
            rest.append(a)
    args = build_parser().parse_args(rest)
    benchmarks = [b for b in registry if args.benchmark_filter is None or re.search(args.benchmark_filter, b.name)]
    if not benchmarks:
        print("no benchmarks registered", file=sys.stderr)
        return []
    names = [b.name for b in benchmarks]
    results: list[dict] = []
    if "WORLD_SIZE" in os.environ and "RANK" in os.environ:
        import torch.distributed as dist

        import iris_b200

        if not dist.is_initialized():
            cuda = torch.cuda.is_available()
            if cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl" if cuda else "gloo")
        ctx = iris_b200.iris(args.heap_size)
        res = run_benchmarks(ctx, benchmarks, overrides, skips, args.n_warmup, args.n_repeat)
        results = [_result_dict(r) for r in res]
        rank0 = dist.get_rank() == 0
    else:
        import torch.multiprocessing as mp

        rank_counts = set()
        for b in benchmarks:
            ax = {a.name: a.values for a in b.axes}
            for v in overrides.get("num_ranks", ax.get("num_ranks", [8])):
                rank_counts.add(int(v))
        avail = torch.cuda.device_count() if torch.cuda.is_available() else 8
        script = os.path.abspath(sys.argv[0]) if sys.argv and sys.argv[0].endswith(".py") else None
        for n in sorted(rank_counts):
            if n > avail:
                print(f"skipping num_ranks={n}: only {avail} devices", file=sys.stderr)
                continue
            ctxmp = mp.get_context("spawn")
            q = ctxmp.Queue()
            port = _free_port()
            procs = [ctxmp.Process(target=_worker, args=(r, n, port, script, names, overrides, skips, args.n_warmup,
                                                         args.n_repeat, args.heap_size, q)) for r in range(n)]
            for p in procs:
                p.start()
            results += _collect(q, procs)
            for p in procs:
                p.join()
        rank0 = True
    if rank0:
        rs = [Result(d["benchmark"], d["params"], d["gpu_time_ms"], [], d["bandwidth_gbps"], d["tflops"], d["counters"],
                     d["skipped"], d["skip_reason"], d["world_size"], d["device_time_us_max_over_ranks"], d["roofline_us"],
                     d["roofline_frac"], d.get("nccl_baseline_us"), d.get("speedup_vs_baseline")) for d in results]
        text = {"console": format_console, "json": format_json, "csv": format_csv}[args.benchmark_format](rs)
        print(text)
        if args.benchmark_out:
            with open(args.benchmark_out, "w") as f:
                f.write(text)
    return results
