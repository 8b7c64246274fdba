#!/usr/bin/env python3
"""All-reduce at the shapes a tensor-parallel serving engine issues, next to NCCL.

The reference's benchmark/ccl/bench_all_reduce_vllm.py times its all-reduce variants and RCCL on
``(M tokens, N = 2880 hidden)`` bf16 tensors: decode-like M of 1 to 512 tokens, prefill-like M of
2048 to 8192. Same table here as one benchmark with an ``impl`` axis (the library is timed once per
size):

    python benchmark/ccl/bench_all_reduce_serving_shapes.py --axis_num_ranks=8 \
        --benchmark_format=csv --benchmark_out=serving_all_reduce.csv
    python benchmark/ccl/plot_sweep_results.py serving_all_reduce.csv --x tokens --series impl,variant \
        --baseline nccl/auto

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

TOKENS = [1, 32, 64, 128, 512] + [2048, 4096, 8192]      # decode-like, then prefill-like
HIDDEN = 2880
LINK_GBPS = 770.0   # measured peer-copy bandwidth per direction per GPU


@bench.register
@bench.axis("num_ranks", [8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("variant", ["auto", "one_shot", "two_shot", "nvls", "push"])
@bench.axis("hidden", [HIDDEN])
@bench.axis("tokens", TOKENS)
@bench.axis("dtype", [torch.bfloat16])
def all_reduce_serving(state, ctx):
    tokens, hidden, dtype, variant, impl = state["tokens"], state["hidden"], state["dtype"], state["variant"], state["impl"]
    world, rank = ctx.get_num_ranks(), ctx.get_rank()
    payload = tokens * hidden * torch.empty((), dtype=dtype).element_size()
    wire = 2 * (world - 1) / world * payload
    state.set_bytes(int(wire))
    state.set_roofline_us(wire / (LINK_GBPS * 1e3))
    if impl == "nccl":
        if variant != "auto":
            state.skip("the library has one entry point: timed once, under variant=auto")
        if ctx.is_cpu:
            state.skip("the library baseline needs the nccl backend")
        t = torch.full((tokens, hidden), float(rank + 1), dtype=dtype, device=ctx.get_device())
        state.exec(lambda: dist.all_reduce(t), preamble_fn=lambda: t.fill_(float(rank + 1)))
        return
    if variant == "nvls" and not ctx.has_multicast():
        state.skip("no NVLS multicast window on this heap")
    src = ctx.full((tokens, hidden), float(rank + 1), dtype=dtype)
    dst = ctx.zeros((tokens, hidden), dtype=dtype)
    cfg = Config(all_reduce_variant=variant)
    ws = ctx.ccl.all_reduce(dst, src, config=cfg)
    expected = float(world * (world + 1) // 2)                 # rank r contributes r + 1 everywhere
    assert torch.all(dst.float() == expected), f"all_reduce({variant}) gave {dst.flatten()[:4].tolist()}, expected {expected}"
    state.add_counter("variant_code", {"one_shot": 2, "two_shot": 3, "nvls": 5, "push": 6}.get(getattr(ws, "variant", None), -1))
    state.exec(lambda: ctx.ccl.all_reduce(dst, src, config=cfg, workspace=ws, async_op=True))


if __name__ == "__main__":
    bench.main()
