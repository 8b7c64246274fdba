#!/usr/bin/env python3
"""All-reduce at the shapes a tensor-parallel serving engine issues, next to NCCL.

The reference's benchmark/ccl/bench_all_reduce_vllm.py times its all-reduce variants and RCCL on
``(M tokens, N = 2880 hidden)`` bf16 tensors: decode-like M of 1 to 512 tokens, prefill-like M of
2048 to 8192. Same table here, one benchmark per implementation so that each keeps its own axes:

    python benchmark/ccl/bench_all_reduce_serving_shapes.py --axis_num_ranks=8 \
        --benchmark_format=csv --benchmark_out=serving_all_reduce.csv
    python benchmark/ccl/plot_sweep_results.py serving_all_reduce.csv --x M --series benchmark,variant

Every point is checked against the closed-form sum (rank r contributes r + 1 everywhere) before it
is timed; the reported bytes follow the bus-bandwidth convention 2 (W - 1) / W x payload.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.ccl import Config  # noqa: E402

DECODE_MS = [1, 32, 64, 128, 512]
PREFILL_MS = [2048, 4096, 8192]
ALL_MS = DECODE_MS + PREFILL_MS
LINK_GBPS = 770.0   # measured peer-copy bandwidth per direction per GPU


def _account(state, M, N, dtype, world):
    nbytes = M * N * torch.empty((), dtype=dtype).element_size()
    state.set_bytes(int(2 * (world - 1) / world * nbytes))
    state.set_roofline_us(2 * (world - 1) / world * nbytes / (LINK_GBPS * 1e3))


@bench.register
@bench.axis("num_ranks", [8])
@bench.axis("M", ALL_MS)
@bench.axis("N", [2880])
@bench.axis("dtype", [torch.bfloat16])
def nccl_all_reduce(state, ctx):
    M, N, dtype = state["M"], state["N"], state["dtype"]
    W, rank = ctx.get_num_ranks(), ctx.get_rank()
    _account(state, M, N, dtype, W)
    if ctx.is_cpu:
        state.skip("the library baseline needs the nccl backend")
        return
    t = torch.full((M, N), float(rank + 1), dtype=dtype, device=ctx.get_device())
    state.exec(lambda: dist.all_reduce(t), preamble_fn=lambda: t.fill_(float(rank + 1)))


@bench.register
@bench.axis("num_ranks", [8])
@bench.axis("M", ALL_MS)
@bench.axis("N", [2880])
@bench.axis("dtype", [torch.bfloat16])
@bench.axis("variant", ["auto", "one_shot", "two_shot", "nvls", "push"])
def iris_all_reduce(state, ctx):
    M, N, dtype, variant = state["M"], state["N"], state["dtype"], state["variant"]
    W, rank = ctx.get_num_ranks(), ctx.get_rank()
    _account(state, M, N, dtype, W)
    if variant == "nvls" and not ctx.has_multicast():
        state.skip("no NVLS multicast window on this heap")
        return
    inp = ctx.full((M, N), float(rank + 1), dtype=dtype)
    out = ctx.zeros((M, N), dtype=dtype)
    cfg = Config(all_reduce_variant=variant)
    try:
        ws = ctx.ccl.all_reduce(out, inp, config=cfg)
    except ValueError as e:   # a variant that does not take this size (push is capped)
        state.skip(str(e))
        return
    want = float(W * (W + 1) // 2)
    assert torch.all(out.float() == want), f"all_reduce({variant}) gave {out.flatten()[:4].tolist()}, expected {want}"
    state.add_counter("variant_code", {"one_shot": 2, "two_shot": 3, "nvls": 5, "push": 6}.get(getattr(ws, "variant", None), -1))
    state.exec(lambda: ctx.ccl.all_reduce(out, inp, config=cfg, workspace=ws, async_op=True))


if __name__ == "__main__":
    bench.main()
