#!/usr/bin/env python3
"""GEMM + all-reduce taken apart: the GEMM alone, the all-reduce alone, both back to back, the fused
kernel, and the library pair, at serving shapes (reference: benchmark/ops/bench_matmul_all_reduce_stages.py,
``M in {32, 896, 2048}, N = 2880, K = 4096``, with torch.mm + dist.all_reduce as the unfused form).

    python benchmark/ops/bench_matmul_all_reduce_stages.py --axis_num_ranks=8 --benchmark_format=csv --benchmark_out=stages.csv
    python benchmark/ccl/plot_sweep_results.py stages.csv --x M --series stage --baseline library_pair

What the rows say: ``gemm`` + ``all_reduce`` is the cost with no overlap at all; ``sequential`` adds
the launch gap between the two kernels; ``fused`` is one kernel that reduces tiles while later tiles
are still being multiplied; ``library_pair`` is cuBLAS followed by NCCL. On the CPU backend the same
script runs with torch GEMMs and host collectives (plumbing check only).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.ops import _local_matmul  # noqa: E402
from iris_b200.utils import fused_target_seconds  # noqa: E402


@bench.register
@bench.axis("num_ranks", [8])
@bench.axis("stage", ["gemm", "all_reduce", "sequential", "fused", "library_pair"])
@bench.axis("M", [32, 896, 2048])
@bench.axis("N", [2880])
@bench.axis("K", [4096])
@bench.axis("dtype", [torch.bfloat16])
def matmul_all_reduce_stages(state, ctx):
    W, M, N, K, dt, stage = ctx.get_num_ranks(), state["M"], state["N"], state["K"], state["dtype"], state["stage"]
    if ctx.is_cpu and dt != torch.float32:
        dt = torch.float32
    dev = ctx.get_device()
    g = torch.Generator(device="cpu").manual_seed(17 + ctx.get_rank())
    A = (torch.randn(M, K, generator=g) * 0.5).to(dt).to(dev)
    B = (torch.randn(K, N, generator=g) * 0.05).to(dt).to(dev)
    esize = A.element_size()
    flops, link = 2.0 * M * N * K, 2.0 * (W - 1) / W * M * N * esize
    state.set_flops(flops if stage != "all_reduce" else 0)
    state.set_bytes(int(link) if stage != "gemm" else 0)
    state.set_roofline_us(fused_target_seconds(flops if stage != "all_reduce" else 0.0, link if stage != "gemm" else 0.0) * 1e6)
    part = ctx.zeros((M, N), dtype=dt)
    out = ctx.zeros((M, N), dtype=dt)
    P = torch.empty(M, N, dtype=dt, device=dev)

    def lib():       # library pair: torch.matmul (cuBLAS) + torch.distributed all_reduce (NCCL; gloo without GPUs)
        torch.matmul(A, B, out=P)
        if W > 1:
            dist.all_reduce(P)

    if stage == "gemm":
        state.exec(lambda: part.copy_(_local_matmul(A, B)) if ctx.is_cpu else _local_matmul(A, B))
        return
    if stage == "all_reduce":
        part.copy_(_local_matmul(A, B))
        ws = ctx.ccl.all_reduce(out, part)
        state.exec(lambda: ctx.ccl.all_reduce(out, part, workspace=ws, async_op=True))
        return
    if stage == "sequential":
        ws = ctx.ccl.all_reduce(out, part)

        def run():
            part.copy_(_local_matmul(A, B))
            ctx.ccl.all_reduce(out, part, workspace=ws, async_op=True)

        state.exec(run)
        return
    if stage == "fused":
        ws = ctx.ops.matmul_all_reduce(out, A, B)
        # the oracle before the clock: the fp32 partial products summed by the process group
        want = A.float() @ B.float()
        if W > 1:
            dist.all_reduce(want)
        tol = (2e-2 if dt != torch.float32 else 1e-4) * max(want.abs().max().item(), 1.0)
        assert (out.float() - want).abs().max().item() <= tol, "fused matmul_all_reduce disagrees with the fp32 sum"
        state.add_counter("fused_kernel", 0 if ws.variant == "unfused" else 1)
        state.exec(lambda: ctx.ops.matmul_all_reduce(out, A, B, workspace=ws, async_op=True))
        state.exec_baseline(lib)          # the same point gets the library pair's time and the ratio
        return
    state.exec(lib)


if __name__ == "__main__":
    bench.main()
