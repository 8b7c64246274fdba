#!/usr/bin/env python3
"""Local GEMM over the shape list of `benchmark/dataset/gemm_shapes.json` (reference:
examples/benchmark/bench_all_shapes.py sweeps a shape list through its GEMM examples).

    python benchmark/ops/bench_all_shapes.py [--shapes benchmark/dataset/gemm_shapes.json] [--json out.json]

One GPU; CUDA events around 20 back-to-back launches after 3 warm-up launches; columns: this
package's tcgen05 kernel (the plan picks tile width and CTA pairs) and torch.matmul (cuBLAS)."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from iris_b200.ops.gemm import matmul  # noqa: E402


def timed(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=os.path.join(ROOT, "benchmark", "dataset", "gemm_shapes.json"))
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    shapes = json.load(open(args.shapes))["shapes"]
    rows = []
    for sh in shapes:
        M, N, K = sh["M"], sh["N"], sh["K"]
        A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16).t() if sh.get("b_transposed") else torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ours = timed(lambda: matmul(A, B, out=C))
        lib = timed(lambda: torch.matmul(A, B, out=C))
        fl = 2.0 * M * N * K
        rows.append({"name": sh["name"], "M": M, "N": N, "K": K, "iris_ms": ours, "iris_tflops": fl / ours / 1e9,
                     "cublas_ms": lib, "cublas_tflops": fl / lib / 1e9})
        print(f"{sh['name']:18s} {M:6d} {N:6d} {K:6d}  iris {ours:.3f} ms {fl / ours / 1e9:7.0f} TF | cuBLAS {lib:.3f} ms {fl / lib / 1e9:7.0f} TF", flush=True)
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
