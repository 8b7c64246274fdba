#!/usr/bin/env python3
"""Block-scaled fp8 GEMM on one GPU: numerics against the fp32 product of the dequantised operands,
then throughput next to the bf16 kernel of this package, torch.matmul (cuBLAS bf16) and
torch._scaled_mm (cuBLASLt fp8 with ONE scale per tensor: a library upper bound, it does less work).

    python benchmark/ops/bench_fp8_gemm.py [--iters 20]

Timing: CUDA events around `iters` back-to-back launches after 3 warm-up launches; fp8 operands plus
the bf16 output of the timed shapes exceed L2 (8192 x 8192 x 7168: 59 + 59 + 134 MB).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from iris_b200.ops.gemm import matmul  # noqa: E402
from iris_b200.ops.gemm_fp8 import dequant_matmul, matmul_fp8, quantize_1x128, quantize_128x128  # noqa: E402


def check(M, N, K):
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    aq, asc = quantize_1x128(x)
    bq, bsc = quantize_128x128(w)
    out = matmul_fp8(aq, asc, bq, bsc)
    torch.cuda.synchronize()
    ref = dequant_matmul(aq, asc, bq, bsc)
    rel = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    ok = rel < 1e-2
    print(f"check M={M} N={N} K={K}: rel={rel:.2e} {'OK' if ok else 'FAIL'}", flush=True)
    return ok


def timed(fn, iters):
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


def bench(M, N, K, iters):
    x = torch.randn(M, K, device="cuda")
    w = torch.randn(N, K, device="cuda") * 0.05
    aq, asc = quantize_1x128(x)
    bq, bsc = quantize_128x128(w)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    del x, w
    cols = []
    fl = 2.0 * M * N * K
    ms = timed(lambda: matmul_fp8(aq, asc, bq, bsc, out=out), iters)
    cols.append(f"fp8 block-scaled {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    ms = timed(lambda: matmul(xb, wb.t(), out=out), iters)
    cols.append(f"bf16 (this package) {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    ms = timed(lambda: torch.matmul(xb, wb.t(), out=out), iters)
    cols.append(f"cuBLAS bf16 {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    try:
        one = torch.ones((), device="cuda")
        ms = timed(lambda: torch._scaled_mm(aq, bq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), iters)
        cols.append(f"cuBLASLt fp8 per-tensor {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    except Exception as e:  # the library path is only a yardstick
        cols.append(f"cuBLASLt fp8 unavailable ({type(e).__name__})")
    print(f"M={M} N={N} K={K}: " + " | ".join(cols), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    torch.manual_seed(0)
    if not check(128, 256, 128):
        print("first case failed; stopping")
        return 1
    ok = True
    for shape in ((128, 256, 512), (256, 512, 1024), (200, 520, 336), (384, 1000, 2048), (4096, 4096, 7168)):
        ok = check(*shape) and ok
    if ok:
        bench(8192, 8192, 7168, args.iters)
        bench(8192, 4096, 7168, args.iters)
        bench(4096, 7168, 2048, args.iters)
        bench(8192, 7168, 8192, args.iters)
    print("ALL OK" if ok else "SOME FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
