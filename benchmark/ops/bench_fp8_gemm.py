#!/usr/bin/env python3
"""Block-scaled fp8 GEMM on one GPU: numerics against the fp32 product of the dequantised operands,
then throughput of the two kernels of this package (scales applied by the tensor core from UE8M0 bytes
in TMEM, for power-of-two scales; promotion of every K block in registers, for arbitrary fp32 scales)
next to the bf16 kernel, torch.matmul (cuBLAS bf16) and torch._scaled_mm (cuBLASLt fp8: with the same
1 x 128 / 128 x 128 block scales when this PyTorch accepts them, and with ONE scale per tensor, a library
upper bound that does less work).

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
from iris_b200.ops.gemm_fp8 import (blockscaled_tile_n, dequant_matmul, matmul_fp8, matmul_fp8_blockscaled, pack_scales_a,  # noqa: E402
                                    pack_scales_b, quantize_1x128, quantize_128x128)


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
    ap, asp = quantize_1x128(xq_src := xb.float(), pow2=True)
    bp, bsp = quantize_128x128(wb.float(), pow2=True)
    del xq_src
    sfa, sfb = pack_scales_a(asp), pack_scales_b(bsp, N, blockscaled_tile_n(M, N))
    for two_sm, name in ((False, "fp8 tensor-core scaling"), (True, "same, CTA pairs")):
        ms = timed(lambda: matmul_fp8_blockscaled(ap, sfa, bp, sfb, out=out, two_sm=two_sm), iters)
        cols.append(f"{name} {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    ms = timed(lambda: matmul_fp8(aq, asc, bq, bsc, out=out), iters)
    cols.append(f"fp8 register promotion {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    try:   # cuBLASLt with the same block scales (scale_a [M, K/128], scale_b [K/128, N/128] as PyTorch lays them out)
        sa_lt = asc.t().contiguous().t()
        sb_lt = bsc.t().contiguous()
        ms = timed(lambda: torch._scaled_mm(aq, bq.t(), scale_a=sa_lt, scale_b=sb_lt, out_dtype=torch.bfloat16), iters)
        cols.append(f"cuBLASLt fp8 block scales {ms:.3f} ms {fl / ms / 1e9:.0f} TF")
    except Exception as e:
        cols.append(f"cuBLASLt fp8 block scales unavailable ({type(e).__name__})")
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
