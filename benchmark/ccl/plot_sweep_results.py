#!/usr/bin/env python3
"""Turn a benchmark CSV into a comparison table (and a figure when matplotlib is installed).

The reference's benchmark/ccl/plot_sweep_results.py plots Iris-vs-RCCL sweeps from the runner's CSV.
This one reads the same kind of file (``--benchmark_format=csv`` of any script in ``benchmark/``),
pivots it into one row per x value and one column per series, prints the table, optionally the
ratio of every series to a baseline series, and draws the curves if it can:

    python benchmark/ccl/plot_sweep_results.py ccl.csv --x bytes --series benchmark,impl --y bandwidth_gbps \
        --baseline "all_reduce/nccl" --out ccl.png

Columns named in ``--where col=value`` filter the rows first. Skipped points are left out.
"""
from __future__ import annotations

import argparse
import csv
import sys
from collections import OrderedDict


def _num(text: str):
    try:
        return float(text)
    except (TypeError, ValueError):
        return None


def load(path: str, where: dict[str, str]) -> list[dict]:
    with open(path, newline="") as f:
        rows = [r for r in csv.DictReader(f)]
    keep = []
    for r in rows:
        if r.get("skipped", "0") not in ("0", "", "False", "false"):
            continue
        if all(r.get(k) == v for k, v in where.items()):
            keep.append(r)
    return keep


def pivot(rows: list[dict], x: str, series: list[str], y: str):
    """``(xs, names, table)`` with ``table[name][x_value] = y``; xs sorted numerically when possible."""
    table: "OrderedDict[str, dict]" = OrderedDict()
    xs: list[str] = []
    for r in rows:
        name = "/".join(r.get(c, "") or "-" for c in series) if series else y
        val = _num(r.get(y))
        if val is None:
            continue
        if r[x] not in xs:
            xs.append(r[x])
        table.setdefault(name, {})[r[x]] = val
    if all(_num(v) is not None for v in xs):
        xs.sort(key=float)
    return xs, list(table), table


def _fmt(v) -> str:
    if v is None:
        return "-"
    if v == 0:
        return "0"
    a = abs(v)
    if a >= 1000:
        return f"{v:.0f}"
    if a >= 10:
        return f"{v:.1f}"
    if a >= 0.1:
        return f"{v:.3f}"
    return f"{v:.3g}"


def render(xs, names, table, x_label: str, y_label: str, baseline: str | None) -> str:
    cols = list(names)
    ratio_cols = []
    if baseline is not None:
        if baseline not in table:
            raise SystemExit(f"baseline series {baseline!r} not found; series are: {', '.join(names)}")
        ratio_cols = [n for n in names if n != baseline]
    head = [x_label] + cols + [f"{n} / {baseline}" for n in ratio_cols]
    lines = [head]
    for xv in xs:
        row = [xv] + [_fmt(table[n].get(xv)) for n in cols]
        for n in ratio_cols:
            a, b = table[n].get(xv), table[baseline].get(xv)
            row.append(_fmt(a / b) if a is not None and b else "-")
        lines.append(row)
    widths = [max(len(str(line[i])) for line in lines) for i in range(len(head))]
    out = [f"# {y_label}"]
    for i, line in enumerate(lines):
        out.append("  ".join(str(c).rjust(w) for c, w in zip(line, widths)))
        if i == 0:
            out.append("  ".join("-" * w for w in widths))
    return "\n".join(out)


def draw(xs, names, table, x_label, y_label, out, logx, logy) -> bool:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return False
    numeric = all(_num(v) is not None for v in xs)
    fig, ax = plt.subplots(figsize=(8, 5))
    for n in names:
        pts = [(float(v) if numeric else i, table[n][v]) for i, v in enumerate(xs) if v in table[n]]
        ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=n)
    if not numeric:
        ax.set_xticks(range(len(xs)), xs, rotation=45)
    if logx and numeric:
        ax.set_xscale("log", base=2)
    if logy:
        ax.set_yscale("log")
    ax.set_xlabel(x_label)
    ax.set_ylabel(y_label)
    ax.grid(True, alpha=0.3)
    ax.legend(fontsize=8)
    fig.tight_layout()
    fig.savefig(out, dpi=130)
    return True


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("csv")
    p.add_argument("--x", default="bytes", help="column of the x axis")
    p.add_argument("--y", default="gpu_time_ms", help="column to compare (gpu_time_ms, bandwidth_gbps, tflops, roofline_frac)")
    p.add_argument("--series", default="benchmark", help="comma-separated columns whose values name a curve")
    p.add_argument("--where", action="append", default=[], help="col=value filter, repeatable")
    p.add_argument("--baseline", default=None, help="series name to divide the others by")
    p.add_argument("--out", default=None, help="figure file (needs matplotlib); the table is always printed")
    p.add_argument("--logx", action="store_true")
    p.add_argument("--logy", action="store_true")
    a = p.parse_args(argv)
    where = dict(w.split("=", 1) for w in a.where)
    rows = load(a.csv, where)
    if not rows:
        print("no rows left after filtering", file=sys.stderr)
        return 1
    for col in [a.x, a.y] + [c for c in a.series.split(",") if c]:
        if col not in rows[0]:
            print(f"column {col!r} is not in {a.csv}; columns: {', '.join(rows[0])}", file=sys.stderr)
            return 2
    xs, names, table = pivot(rows, a.x, [c for c in a.series.split(",") if c], a.y)
    print(render(xs, names, table, a.x, a.y, a.baseline))
    if a.out:
        if draw(xs, names, table, a.x, a.y, a.out, a.logx, a.logy):
            print(f"figure written to {a.out}")
        else:
            print("matplotlib is not installed: no figure written", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
