#!/usr/bin/env python3
"""All-gather + GEMM over the small-M sweep of ``benchmark/dataset/ag_gemm.json``
(``m in {1 .. 1024}, k = 8192, n = 3584``): the decode-time shapes where the gather is latency and
the GEMM is a sliver. The reference times a pull kernel and a push kernel + consumer GEMM on these
shapes (benchmark/examples/bench_all_gather_gemm_pull.py, bench_all_gather_gemm_push.py, A sharded
along K: each rank holds ``(m, k / W)``). Here:

    layout=k   ``ops.all_gather_matmul`` in the reference layout (A sharded along K)
    layout=m   the same op with rows sharded (needs m divisible by the ranks)
    impl=nccl  all_gather (NCCL) + torch.matmul (cuBLAS)

    python benchmark/examples/bench_all_gather_gemm.py --axis_num_ranks=8 --benchmark_format=csv --benchmark_out=ag_gemm.csv

Shapes the fused kernel does not take (rows per rank below its tile) run as collective + GEMM inside
the op; the ``fused_kernel`` counter says which path a point took.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import iris_b200.bench as bench  # noqa: E402
from iris_b200.utils import fused_target_seconds  # noqa: E402

SHAPES = json.load(open(os.path.join(ROOT, "benchmark", "dataset", "ag_gemm.json")))["shapes"]


@bench.register
@bench.axis("num_ranks", [8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("layout", ["k", "m"])
@bench.axis("m", [s["m"] for s in SHAPES])
@bench.axis("n", [SHAPES[0]["n"]])
@bench.axis("k", [SHAPES[0]["k"]])
def all_gather_gemm(state, ctx):
    W, m, n, k, layout = ctx.get_num_ranks(), state["m"], state["n"], state["k"], state["layout"]
    dt = torch.float32 if ctx.is_cpu else torch.bfloat16
    dev = ctx.get_device()
    if layout == "m" and m % W:
        state.skip(f"{m} rows do not split over {W} ranks")
    if layout == "k" and k % W:
        state.skip(f"k = {k} does not split over {W} ranks")
    g = torch.Generator(device="cpu").manual_seed(5 + ctx.get_rank())
    shard = (m, k // W) if layout == "k" else (m // W, k)
    A = (torch.randn(*shard, generator=g) * 0.5).to(dt).to(dev)
    B = (torch.randn(k, n, generator=torch.Generator(device="cpu").manual_seed(1)) * 0.02).to(dt).to(dev)
    esize = A.element_size()
    flops, link = 2.0 * m * n * k, (W - 1) * A.numel() * esize
    state.set_flops(flops)
    state.set_bytes(int(link))
    state.set_roofline_us(fused_target_seconds(flops, link) * 1e6)
    C = ctx.zeros((m, n), dtype=dt)
    if state["impl"] == "nccl":
        gathered = [torch.empty_like(A) for _ in range(W)]
        Cr = torch.empty(m, n, dtype=dt, device=dev)

        def base():
            if W > 1:
                dist.all_gather(gathered, A)
                torch.matmul(torch.cat(gathered, dim=1 if layout == "k" else 0), B, out=Cr)
            else:
                torch.matmul(A, B, out=Cr)

        state.exec(base)
        return
    sd = 1 if layout == "k" else 0
    ws = ctx.ops.all_gather_matmul(C, A, B, shard_dim=sd)
    parts = [torch.empty_like(A) for _ in range(W)]
    dist.all_gather(parts, A)
    want = torch.cat(parts, dim=sd).float() @ B.float()
    tol = (3e-2 if dt != torch.float32 else 1e-4) * max(want.abs().max().item(), 1.0)
    assert (C.float() - want).abs().max().item() <= tol, "all_gather_matmul disagrees with gather + fp32 matmul"
    state.add_counter("fused_kernel", 0 if ws.variant == "unfused" else 1)
    state.exec(lambda: ctx.ops.all_gather_matmul(C, A, B, shard_dim=sd, workspace=ws, async_op=True))


if __name__ == "__main__":
    bench.main()
