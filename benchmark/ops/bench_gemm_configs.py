#!/usr/bin/env python3
"""Local GEMM configurations against the libraries under ONE power state.

A B200 under its 1 kW cap clocks down while a dense GEMM loop runs, so a configuration timed first
reads 5 to 15 % higher than the same one timed after a minute of load. Here every configuration of a
shape (single-CTA and CTA-pair tiles, 256- and 224-wide, bf16 and block-scaled e4m3, the plan's own
choice, cuBLAS bf16, cuBLASLt e4m3 with one scale per tensor) is timed in turn, five launches at a time,
for eight rounds; the median of a configuration's eight timings is reported. Operands exceed L2.

    python benchmark/ops/bench_gemm_configs.py [MxNxK ...]
"""
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from iris_b200.ops import matmul, quantize_activation, quantize_weight  # noqa: E402

SHAPES = [(8192, 8192, 7168), (8192, 3584, 8192), (8192, 8192, 3584), (16384, 8192, 16384), (4096, 7168, 2048)]


def burst(fn, iters=5):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    shapes = [tuple(int(v) for v in a.split("x")) for a in sys.argv[1:]] or SHAPES
    one = torch.ones((), device="cuda")
    for (M, N, K) in shapes:
        x = torch.randn(M, K, device="cuda")
        w = torch.randn(N, K, device="cuda") * 0.05
        a, b = quantize_activation(x), quantize_weight(w)
        xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
        del x, w
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        cfgs = {}
        for pair in (False, True):
            cfgs[f"e4m3 pair={int(pair)}"] = lambda pair=pair: matmul(a, b, out=out, two_sm=pair)
            for bn in (256, 224):
                cfgs[f"bf16 pair={int(pair)} bn={bn}"] = lambda pair=pair, bn=bn: matmul(xb, wb.t(), out=out, two_sm=pair, bn=bn)
        cfgs["bf16 plan"] = lambda: matmul(xb, wb.t(), out=out)
        cfgs["e4m3 plan"] = lambda: matmul(a, b, out=out)
        cfgs["cuBLAS bf16"] = lambda: torch.matmul(xb, wb.t(), out=out)
        cfgs["cuBLASLt e4m3 per-tensor"] = lambda: torch._scaled_mm(a.q, b.q.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for f in cfgs.values():
            f()
        torch.cuda.synchronize()
        times = {k: [] for k in cfgs}
        for _ in range(8):
            for k, f in cfgs.items():
                times[k].append(burst(f))
        flops = 2.0 * M * N * K
        print(f"{M}x{N}x{K} TFLOP/s: " + " | ".join(f"{k} {flops / statistics.median(v) / 1e9:.0f}" for k, v in times.items()), flush=True)
        del a, b, xb, wb, out


if __name__ == "__main__":
    main()
