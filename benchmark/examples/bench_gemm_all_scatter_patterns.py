#!/usr/bin/env python3
"""GEMM + all-scatter, one problem under every overlap pattern, side by side.

The reference ships one example per pattern and quotes their throughput at 16384 x 16384 x 16384 fp16 on
eight GPUs (.github/workflows/iris-performance-regression-test.yml:25-45; docs/conceptual/taxonomy.md):

    bulk_synchronous   examples/12_gemm_all_scatter_bulk_synchronous   GEMM kernel, then the all-scatter
    fused              examples/07_gemm_all_scatter                    epilogue of every tile stores to all ranks
    wg_specialized     examples/10_gemm_all_scatter_wg_specialization  communication CTAs forward finished tiles
    producer_consumer  examples/11_gemm_all_scatter_producer_consumer  (here: the same kernel as wg_specialized;
                       two kernels that spin on one another's flags are not launched on one GPU)
    nccl               torch.matmul (cuBLAS) + dist.all_gather_into_tensor

Every rank multiplies A [M, K] by its column block B_r [K, N / W] and all ranks end with C [M, N].
Reported: aggregate TFLOP/s = 2 M N K / time (the reference's convention), device time, maximum over ranks.

    python benchmark/examples/bench_gemm_all_scatter_patterns.py --axis_num_ranks=8
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.ops import FusedConfig  # noqa: E402

PEAK_TFLOPS = 1383.6
LINK_GBPS = 770.0


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("pattern", ["bulk_synchronous", "fused", "wg_specialized", "nccl"])
@bench.axis("M", [16384])
@bench.axis("N", [16384])
@bench.axis("K", [16384])
@bench.axis("dtype", ["float16"])
@bench.axis("comm_sms", [16])
def gemm_all_scatter(state, ctx):
    W, M, N, K = ctx.get_num_ranks(), state["M"], state["N"], state["K"]
    dt = getattr(torch, state["dtype"]) if isinstance(state["dtype"], str) else state["dtype"]
    dev = ctx.get_device()
    if dev.type != "cuda":
        dt = torch.float32                                                # gloo ranks: the host fallbacks
    Nl = N // W
    A = torch.randn(M, K, device=dev, dtype=dt)
    B = (torch.randn(Nl, K, device=dev, dtype=dt) * 0.02).t()             # weight stored (out, in)
    C = ctx.zeros((M, N), dtype=dt)
    flops_rank = 2.0 * M * Nl * K
    link = (W - 1) * M * Nl * 2
    state.set_flops(flops_rank * W)                                      # aggregate over ranks: every rank does flops_rank in the same time
    state.set_bytes(link)
    state.set_roofline_us(max(flops_rank / (PEAK_TFLOPS * 1e6), link / (LINK_GBPS * 1e3)))
    state.set_repeat(min(state.n_repeat, 20))            # long kernels: fewer repeats than the default, never more than asked for
    state.set_warmup(min(state.n_warmup, 5))
    pattern = state["pattern"]
    if pattern == "nccl":
        loc = torch.empty(M, Nl, device=dev, dtype=dt)
        parts = torch.empty(W, M, Nl, device=dev, dtype=dt)

        def base():
            torch.matmul(A, B, out=loc)
            if W > 1:
                dist.all_gather_into_tensor(parts, loc)
                C.view(M, W, Nl).copy_(parts.permute(1, 0, 2))
            else:
                C.copy_(loc)

        state.exec(base)
        return
    cfg = FusedConfig(overlap=pattern, comm_sms=state["comm_sms"] if pattern == "wg_specialized" else 0)
    ws = ctx.ops.matmul_all_gather(C, A, B, scatter_cols=True, config=cfg)
    try:   # deviation of a row sample of this rank's column block from an fp32 product (a counter: benchmarks report, tests assert)
        n, r = min(64, M), ctx.get_rank()
        ref = A[:n].float() @ B.float()
        if dev.type == "cuda":
            torch.cuda.synchronize()
        state.add_counter("max_rel_err", round((C[:n, r * Nl:(r + 1) * Nl].float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12), 6))
    except Exception:  # noqa: BLE001
        state.add_counter("max_rel_err", -1.0)
    state.exec(lambda: ctx.ops.matmul_all_gather(C, A, B, scatter_cols=True, config=cfg, workspace=ws, async_op=True))


if __name__ == "__main__":
    bench.main()
