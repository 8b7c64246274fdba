#!/usr/bin/env python3
"""Performance gate: compare benchmark output with the floors in ``dataset/perf_thresholds.json``.

The reference's CI runs four GEMM + all-scatter examples at 16384^3 on 8 GPUs and fails the job when
the TFLOPS read from the example's JSON (with ``jq``) fall under a per-example threshold
(.github/workflows/iris-performance-regression-test.yml:25-45, .github/scripts/run_perf_benchmark.sh:30-68).
Same gate here, for two kinds of input:

    python bench.py --gpus 1 > line.json
    python benchmark/check_regression.py --bench line.json
    python benchmark/ops/bench_fused_ops.py --axis_num_ranks=8 --benchmark_format=json --benchmark_out=fused.json
    python benchmark/check_regression.py --sweep fused.json

``--bench`` takes files holding the one-line JSON records of ``bench.py`` (several lines and
several files allowed); ``--sweep`` takes the JSON written by the benchmark runner. Entries of the
threshold file that match nothing in the input are reported as "not measured" and do not fail the
gate unless ``--require-all`` is given. Exit code 0 = pass, 1 = regression, 2 = bad input.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def read_bench_lines(paths) -> list[dict]:
    out = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    try:
                        out.append(json.loads(line))
                    except ValueError:
                        pass
    return out


def read_sweeps(paths) -> list[dict]:
    out = []
    for p in paths:
        with open(p) as f:
            doc = json.load(f)
        out.extend(doc["results"] if isinstance(doc, dict) else doc)
    return out


def _verdict(name: str, got: float, rule: dict) -> tuple[bool, str]:
    if "min" in rule:
        ok = got >= rule["min"]
        return ok, f"{name}: {got:.4g} (floor {rule['min']:.4g}, measured {rule.get('measured', '-')})"
    ok = got <= rule["max"]
    return ok, f"{name}: {got:.4g} (ceiling {rule['max']:.4g}, measured {rule.get('measured', '-')})"


def check(thresholds: dict, bench_lines: list[dict], sweeps: list[dict]):
    """Returns ``(failures, passes, missing)`` as lists of messages."""
    failures, passes, missing = [], [], []
    if bench_lines is not None:
        for rule in thresholds.get("bench", []):
            hits = [b for b in bench_lines if b.get("n_gpus") == rule["n_gpus"] and "unavailable" not in b and b.get("impl") != "reference"]
            name = f"bench.py at {rule['n_gpus']} GPU(s) {rule['metric']}"
            if not hits:
                missing.append(name)
                continue
            ok, msg = _verdict(name, float(hits[-1][rule["metric"]]), rule)
            (passes if ok else failures).append(msg)
    if sweeps is not None:
        for rule in thresholds.get("sweeps", []):
            hits = [r for r in sweeps if r.get("benchmark") == rule["benchmark"] and not r.get("skipped")
                    and all(str(r.get("params", {}).get(k)) == str(v) for k, v in rule.get("where", {}).items())]
            name = f"{rule['benchmark']} {rule.get('where', {})} {rule['metric']}"
            if not hits:
                missing.append(name)
                continue
            # several points may match (other axes): the gate is on the best of them
            vals = [float(r[rule["metric"]]) for r in hits if r.get(rule["metric"]) is not None]
            got = max(vals) if "min" in rule else min(vals)
            ok, msg = _verdict(name, got, rule)
            (passes if ok else failures).append(msg)
    return failures, passes, missing


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--thresholds", default=os.path.join(HERE, "dataset", "perf_thresholds.json"))
    p.add_argument("--bench", nargs="*", default=None, help="files with bench.py JSON lines")
    p.add_argument("--sweep", nargs="*", default=None, help="JSON files written by the benchmark runner")
    p.add_argument("--require-all", action="store_true", help="fail when a threshold has no matching measurement")
    a = p.parse_args(argv)
    if a.bench is None and a.sweep is None:
        print("nothing to check: give --bench and / or --sweep", file=sys.stderr)
        return 2
    try:
        with open(a.thresholds) as f:
            thresholds = json.load(f)
        lines = read_bench_lines(a.bench) if a.bench is not None else None
        sweeps = read_sweeps(a.sweep) if a.sweep is not None else None
    except (OSError, ValueError, KeyError) as e:
        print(f"bad input: {e}", file=sys.stderr)
        return 2
    failures, passes, missing = check(thresholds, lines, sweeps)
    for m in passes:
        print("ok    " + m)
    for m in missing:
        print("skip  " + m + ": not measured")
    for m in failures:
        print("FAIL  " + m)
    if failures or (a.require_all and missing):
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
