#!/usr/bin/env python3
"""Local GEMM on one GPU: numerics against an fp32 PyTorch product, then throughput of the CTA-pair
(tcgen05 cta_group::2) and single-CTA kernels next to torch.matmul (cuBLAS) on the shapes of the
tensor-parallel MLP benchmark.

    python benchmark/ops/bench_local_gemm.py [--iters 20]

Timing: all configurations and cuBLAS take turns (`iters` back-to-back launches each, eight rounds, medians), so
that they run under the same power state; the SM clock is read through NVML while each burst runs and
time x clock is printed next to the time. Operands (A + B + C >= 170 MB) are larger than L2.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from iris_b200.ops.gemm import matmul  # noqa: E402


def check(M, N, K, dtype, kmajor, two_sm, bias=False, bn=0):
    A = torch.randn(M, K, device="cuda", dtype=dtype)
    B = (torch.randn(N, K, device="cuda", dtype=dtype) * 0.05).t() if kmajor else torch.randn(K, N, device="cuda", dtype=dtype) * 0.05
    b = torch.randn(N, device="cuda", dtype=dtype) if bias else None
    C = matmul(A, B, bias=b, two_sm=two_sm, bn=bn)
    torch.cuda.synchronize()
    ref = A.float() @ B.float()
    if bias:
        ref = ref + b.float()
    rel = (C.float() - ref).abs().max().item() / ref.abs().max().item()
    ok = rel < 2e-2
    print(f"check two_sm={two_sm} bn={bn} M={M} N={N} K={K} {str(dtype)[6:]} B{'^T' if kmajor else ''} bias={bias}: rel={rel:.2e} {'OK' if ok else 'FAIL'}", flush=True)
    return ok


class _Clock:
    """SM clock through NVML, read while the GPU works (None when NVML is not there)."""

    def __init__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
            self.nv = pynvml
        except Exception:
            self.h = None

    def mhz(self):
        return self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM) if self.h is not None else None


def bench(M, N, K, kmajor, iters, rounds=8):
    """Every configuration and cuBLAS in turn (A, B, C, ..., A, B, C, ...), `iters` launches at a time, `rounds`
    times: under the power cap all of them then see the same clocks. Reported: median time, TFLOP/s and
    time x SM MHz (thousands of SM cycles per GEMM, which takes the clock out of the comparison)."""
    import statistics

    dt = torch.bfloat16
    A = torch.randn(M, K, device="cuda", dtype=dt)
    B = torch.randn(N, K, device="cuda", dtype=dt).t() if kmajor else torch.randn(K, N, device="cuda", dtype=dt)
    C = torch.empty(M, N, device="cuda", dtype=dt)
    cfgs = (("pair bn256", lambda: matmul(A, B, out=C, two_sm=True, bn=256)),
            ("pair bn224", lambda: matmul(A, B, out=C, two_sm=True, bn=224)),
            ("plan", lambda: matmul(A, B, out=C)),
            ("single CTA", lambda: matmul(A, B, out=C, two_sm=False)),
            ("cuBLAS", lambda: torch.matmul(A, B, out=C)))
    clock = _Clock()
    for _, fn in cfgs:
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    times = {n: [] for n, _ in cfgs}
    clocks = {n: [] for n, _ in cfgs}
    for _ in range(rounds):
        for name, fn in cfgs:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record()
            mhz = clock.mhz()           # read while the launches above are still running
            torch.cuda.synchronize()
            times[name].append(s.elapsed_time(e) / iters)
            if mhz:
                clocks[name].append(mhz)
    cols = []
    for name, _ in cfgs:
        ms = statistics.median(times[name])
        mhz = statistics.median(clocks[name]) if clocks[name] else None
        cyc = f", {mhz:.0f} MHz, {ms * mhz:.0f} kcycles" if mhz else ""
        cols.append(f"{name} {ms:.3f} ms {2 * M * N * K / ms / 1e9:.0f} TF{cyc}")
    print(f"M={M} N={N} K={K} B{'^T' if kmajor else ''}: " + " | ".join(cols), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    torch.manual_seed(0)
    ok = check(256, 256, 64, torch.bfloat16, True, True)
    if not ok:
        print("first case failed; stopping")
        return 1
    cases = [(256, 256, 64, torch.bfloat16, False, True, False, 0), (256, 448, 512, torch.bfloat16, True, True, False, 224),
             (384, 896, 1024, torch.float16, False, True, False, 224), (1024, 1024, 1024, torch.bfloat16, True, True, True, 0),
             (200, 520, 328, torch.bfloat16, False, True, False, 0), (200, 264, 328, torch.bfloat16, False, False, True, 128),
             (4096, 3584, 4096, torch.bfloat16, False, None, False, 0), (4096, 3584, 4096, torch.bfloat16, True, None, False, 0)]
    for c in cases:
        ok = check(*c[:6], bias=c[6], bn=c[7]) and ok
    if ok:
        for km in (True, False):
            bench(8192, 3584, 8192, km, args.iters)
            bench(8192, 8192, 3584, km, args.iters)
        bench(8192, 8192, 8192, True, args.iters)
    print("ALL OK" if ok else "SOME FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
