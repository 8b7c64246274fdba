#!/usr/bin/env python3
"""Sweep of the collectives next to NCCL (reference: benchmark/ccl/bench_all_reduce.py,
bench_all_gather.py, bench_all_to_all.py, bench_reduce_scatter.py and the RCCL comparison of
bench_all_reduce_vllm.py).

    python benchmark/ccl/bench_collectives.py --axis_num_ranks=8 --axis_bytes=pow2:10:30 \
        --benchmark_format=csv --benchmark_out=ccl.csv

Sizes are bytes per rank; bus bandwidth follows the NCCL convention
(all_reduce 2(W-1)/W, all_gather / reduce_scatter / all_to_all (W-1)/W of the full payload).
Each point checks the result against a float64 host reduction before it is timed.
``--axis_timing=back_to_back`` times a run of calls issued without a gap (one event pair around all of them)
instead of one call at a time behind a barrier and an L2 flush: below about 1 MB the per-call protocol
measures the launch skew between the ranks rather than the collective.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.ccl import Config  # noqa: E402

LINK_GBPS = 770.0   # measured peer-copy bandwidth per direction per GPU on this pool


def _shape(nbytes, dtype, world):
    n = max(nbytes // torch.empty((), dtype=dtype).element_size(), world * 8)
    cols = min(n, 8192)
    cols -= cols % (world * 8)
    cols = max(cols, world * 8)
    return max(n // cols, 1), cols


def _inputs(ctx, M, N, dtype):
    g = torch.Generator(device=ctx.get_device())
    g.manual_seed(1234 + ctx.get_rank())
    inp = ctx.empty((M, N), dtype=dtype)
    inp.copy_((torch.rand(M, N, device=ctx.get_device(), generator=g) * 2 - 1).to(dtype))
    return inp


def _host_sum(inp, world):
    parts = [torch.empty_like(inp) for _ in range(world)]
    dist.all_gather(parts, inp)
    return torch.stack([p.double().cpu() for p in parts]).sum(0)


@bench.register
@bench.axis("num_ranks", [2, 4, 8])
@bench.axis("dtype", [torch.bfloat16, torch.float32])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("variant", ["auto"])
@bench.axis("timing", ["per_call"])
@bench.axis("bytes", bench.power_of_two(10, 30))
def all_reduce(state, ctx):
    W, dtype = ctx.get_num_ranks(), state["dtype"]
    M, N = _shape(state["bytes"], dtype, W)
    inp = _inputs(ctx, M, N, dtype)
    out = ctx.zeros((M, N), dtype=dtype)
    nbytes = M * N * inp.element_size()
    state.set_bytes(int(2 * (W - 1) / W * nbytes))
    state.set_roofline_us(2 * (W - 1) / W * nbytes / (LINK_GBPS * 1e3))
    if state["impl"] == "nccl":
        buf = inp.clone()
        state.exec(lambda: dist.all_reduce(buf), preamble_fn=lambda: buf.copy_(inp))
        return
    cfg = Config(all_reduce_variant=state["variant"])
    ws = ctx.ccl.all_reduce(out, inp, config=cfg)
    if nbytes <= 1 << 24:
        ref = _host_sum(inp, W)
        tol = 1e-5 * W if dtype == torch.float32 else 0.03 * W
        assert (out.double().cpu() - ref).abs().max().item() <= tol, "all_reduce mismatch"
    state.add_counter("variant_code", {"one_shot": 2, "two_shot": 3, "nvls": 5}.get(ws.variant, -1))
    state.exec(lambda: ctx.ccl.all_reduce(out, inp, config=cfg, workspace=ws, async_op=True))


@bench.register
@bench.axis("num_ranks", [2, 4, 8])
@bench.axis("dtype", [torch.bfloat16])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("timing", ["per_call"])
@bench.axis("bytes", bench.power_of_two(10, 30))
def all_gather(state, ctx):
    W, dtype = ctx.get_num_ranks(), state["dtype"]
    M, N = _shape(state["bytes"], dtype, W)
    inp = _inputs(ctx, M, N, dtype)
    out = ctx.zeros((W * M, N), dtype=dtype)
    nbytes = M * N * inp.element_size()
    state.set_bytes((W - 1) * nbytes)
    state.set_roofline_us((W - 1) * nbytes / (LINK_GBPS * 1e3))
    if state["impl"] == "nccl":
        ref = torch.empty(W * M, N, dtype=dtype, device=ctx.get_device())
        state.exec(lambda: dist.all_gather_into_tensor(ref, inp))
        return
    ctx.ccl.all_gather(out, inp)
    ref = torch.empty(W * M, N, dtype=dtype, device=ctx.get_device())
    dist.all_gather_into_tensor(ref, inp)
    assert torch.equal(out, ref), "all_gather mismatch"
    state.exec(lambda: ctx.ccl.all_gather(out, inp, async_op=True))


@bench.register
@bench.axis("num_ranks", [2, 4, 8])
@bench.axis("dtype", [torch.bfloat16])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("timing", ["per_call"])
@bench.axis("bytes", bench.power_of_two(10, 30))
def reduce_scatter(state, ctx):
    W, dtype = ctx.get_num_ranks(), state["dtype"]
    M, N = _shape(state["bytes"], dtype, W)
    M = max(M - M % W, W)
    inp = _inputs(ctx, M, N, dtype)
    out = ctx.zeros((M // W, N), dtype=dtype)
    nbytes = M * N * inp.element_size()
    state.set_bytes(int((W - 1) / W * nbytes))
    state.set_roofline_us((W - 1) / W * nbytes / (LINK_GBPS * 1e3))
    if state["impl"] == "nccl":
        o = torch.empty(M // W, N, dtype=dtype, device=ctx.get_device())
        state.exec(lambda: dist.reduce_scatter_tensor(o, inp))
        return
    cfg = Config(reduce_scatter_rows=True)
    ctx.ccl.reduce_scatter(out, inp, config=cfg)
    if nbytes <= 1 << 24:
        ref = _host_sum(inp, W)[ctx.get_rank() * (M // W):(ctx.get_rank() + 1) * (M // W)]
        assert (out.double().cpu() - ref).abs().max().item() <= 0.03 * W, "reduce_scatter mismatch"
    state.exec(lambda: ctx.ccl.reduce_scatter(out, inp, config=cfg, async_op=True))


@bench.register
@bench.axis("num_ranks", [2, 4, 8])
@bench.axis("dtype", [torch.bfloat16])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("timing", ["per_call"])
@bench.axis("bytes", bench.power_of_two(10, 30))
def all_to_all(state, ctx):
    W, dtype = ctx.get_num_ranks(), state["dtype"]
    M, N = _shape(state["bytes"], dtype, W)
    inp = _inputs(ctx, M, N, dtype)
    out = ctx.zeros((M, N), dtype=dtype)
    nbytes = M * N * inp.element_size()
    state.set_bytes(int((W - 1) / W * nbytes))
    state.set_roofline_us((W - 1) / W * nbytes / (LINK_GBPS * 1e3))
    if state["impl"] == "nccl":
        src = inp.view(M, W, N // W).permute(1, 0, 2).contiguous()
        dst = torch.empty_like(src)
        state.exec(lambda: dist.all_to_all_single(dst, src))
        return
    ctx.ccl.all_to_all(out, inp)
    state.exec(lambda: ctx.ccl.all_to_all(out, inp, async_op=True))


if __name__ == "__main__":
    bench.main()
