#!/usr/bin/env python3
"""Fused GEMM + collective ops next to cuBLAS + NCCL (reference: benchmark/ops/bench_all_gather_matmul.py,
bench_matmul_all_gather.py, bench_matmul_all_reduce.py and the stage profiler
bench_matmul_all_reduce_stages.py).

    python benchmark/ops/bench_fused_ops.py --axis_num_ranks=8 --benchmark_format=json

Shapes are the tensor-parallel ones: all_gather_matmul gathers A [M/W, K] by rows and multiplies
by B [K, F/W']; matmul_reduce_scatter / matmul_all_reduce multiply A [M, F'] by B [F', K].
The roofline is the slower of FLOPs / measured cuBLAS peak and NVLink bytes / measured link rate.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402

PEAK_TFLOPS = 1383.6   # measured sustained cuBLAS bf16 on this pool
LINK_GBPS = 770.0


def _roof(flops, link_bytes):
    return max(flops / (PEAK_TFLOPS * 1e6), link_bytes / (LINK_GBPS * 1e3))


def _record_error(state, got, ref):
    """Counter `max_rel_err` of a benchmark point: largest deviation of a sample of the fused result from an fp32
    PyTorch product, over the reference's largest magnitude (bf16 rounding gives a few 1e-3). Never raises:
    a benchmark reports, the tests assert."""
    try:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        err = (got.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12)
        state.add_counter("max_rel_err", round(err, 6))
    except Exception:  # noqa: BLE001
        state.add_counter("max_rel_err", -1.0)


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("M", [8192])
@bench.axis("N", [3584])
@bench.axis("K", [8192])
def all_gather_matmul(state, ctx):
    W, M, N, K = ctx.get_num_ranks(), state["M"], state["N"], state["K"]
    dt = torch.bfloat16 if ctx.get_device().type == "cuda" else torch.float32          # gloo ranks: the host fallbacks, fp32
    A = torch.randn(M // W, K, device=ctx.get_device(), dtype=dt)
    B = torch.randn(K, N, device=ctx.get_device(), dtype=dt) * 0.02
    C = ctx.zeros((M, N), dtype=dt)
    state.set_flops(2 * M * N * K)
    state.set_bytes((W - 1) * (M // W) * K * 2)
    state.set_roofline_us(_roof(2 * M * N * K, (W - 1) * (M // W) * K * 2))
    if state["impl"] == "nccl":
        Aall = torch.empty(M, K, device=ctx.get_device(), dtype=dt)
        Cr = torch.empty(M, N, device=ctx.get_device(), dtype=dt)

        def base():
            if W > 1:
                dist.all_gather_into_tensor(Aall, A)
                torch.matmul(Aall, B, out=Cr)
            else:
                torch.matmul(A, B, out=Cr)

        state.exec(base)
        return
    ws = ctx.ops.all_gather_matmul(C, A, B, shard_dim=0)
    r, n = ctx.get_rank(), min(64, M // W)
    _record_error(state, C[r * (M // W):r * (M // W) + n], A[:n].float() @ B.float())       # this rank's own rows of the gathered product
    state.exec(lambda: ctx.ops.all_gather_matmul(C, A, B, shard_dim=0, workspace=ws, async_op=True))


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("op", ["reduce_scatter", "all_reduce"])
@bench.axis("M", [128, 1024, 8192])
@bench.axis("N", [8192])
@bench.axis("K", [3584])
def matmul_reduce(state, ctx):
    W, M, N, K = ctx.get_num_ranks(), state["M"], state["N"], state["K"]
    rs = state["op"] == "reduce_scatter"
    if rs and M % (128 * W):
        state.skip("row reduce-scatter needs M to be a multiple of 128 * ranks")
    dt = torch.bfloat16 if ctx.get_device().type == "cuda" else torch.float32          # gloo ranks: the host fallbacks, fp32
    A = torch.randn(M, K, device=ctx.get_device(), dtype=dt)
    B = torch.randn(K, N, device=ctx.get_device(), dtype=dt) * 0.02
    link = (W - 1) / W * M * N * 2 * (1 if rs else 2)
    state.set_flops(2 * M * N * K)
    state.set_bytes(int(link))
    state.set_roofline_us(_roof(2 * M * N * K, link))
    if state["impl"] == "nccl":
        P = torch.empty(M, N, device=ctx.get_device(), dtype=dt)
        R = torch.empty(M // W, N, device=ctx.get_device(), dtype=dt) if rs else None

        def base():
            torch.matmul(A, B, out=P)
            if W > 1:
                dist.reduce_scatter_tensor(R, P) if rs else dist.all_reduce(P)

        state.exec(base)
        return
    if rs:
        C = ctx.zeros((M // W, N), dtype=dt)
        ws = ctx.ops.matmul_reduce_scatter(C, A, B, scatter_rows=True)
        r, n = ctx.get_rank(), min(64, M // W)
        ref = torch.zeros(W, n, N, device=ctx.get_device())                # row sample of every rank's block, summed over ranks
        for o in range(W):
            ref[o] = A[o * (M // W):o * (M // W) + n].float() @ B.float()
        if W > 1:
            dist.all_reduce(ref)
        _record_error(state, C[:n], ref[r])
        state.exec(lambda: ctx.ops.matmul_reduce_scatter(C, A, B, scatter_rows=True, workspace=ws, async_op=True))
    else:
        C = ctx.zeros((M, N), dtype=dt)
        ws = ctx.ops.matmul_all_reduce(C, A, B)
        n = min(64, M)
        ref = A[:n].float() @ B.float()
        if W > 1:
            dist.all_reduce(ref)
        _record_error(state, C[:n], ref)
        state.exec(lambda: ctx.ops.matmul_all_reduce(C, A, B, workspace=ws, async_op=True))


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("M", [1024, 4096])
@bench.axis("N", [3584])
@bench.axis("K", [8192])
def matmul_all_gather(state, ctx):
    W, M, N, K = ctx.get_num_ranks(), state["M"], state["N"], state["K"]
    dt = torch.bfloat16 if ctx.get_device().type == "cuda" else torch.float32          # gloo ranks: the host fallbacks, fp32
    A = torch.randn(M, K, device=ctx.get_device(), dtype=dt)
    B = torch.randn(K, N, device=ctx.get_device(), dtype=dt) * 0.02
    C = ctx.zeros((W * M, N), dtype=dt)
    state.set_flops(2 * M * N * K)
    state.set_bytes((W - 1) * M * N * 2)
    state.set_roofline_us(_roof(2 * M * N * K, (W - 1) * M * N * 2))
    if state["impl"] == "nccl":
        loc = torch.empty(M, N, device=ctx.get_device(), dtype=dt)
        full = torch.empty(W * M, N, device=ctx.get_device(), dtype=dt)

        def base():
            torch.matmul(A, B, out=loc)
            if W > 1:
                dist.all_gather_into_tensor(full, loc)

        state.exec(base)
        return
    ws = ctx.ops.matmul_all_gather(C, A, B)
    r, n = ctx.get_rank(), min(64, M)
    _record_error(state, C[r * M:r * M + n], A[:n].float() @ B.float())
    state.exec(lambda: ctx.ops.matmul_all_gather(C, A, B, workspace=ws, async_op=True))


if __name__ == "__main__":
    bench.main()
