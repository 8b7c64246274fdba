#!/usr/bin/env python3
"""Expert-sharded MoE layer throughput (reference: benchmark/examples/bench_moe.py).

Default point: 4096 tokens per rank, hidden 7168, 32 experts per rank, top-8, SwiGLU FFN 2048,
bf16 weights. FLOPs counted: 2 * pairs * (hidden * 2 * ffn + ffn * hidden) per rank."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import MoELayer  # noqa: E402

PEAK_TFLOPS = 1383.6


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("tokens", [4096])
@bench.axis("hidden", [7168])
@bench.axis("ffn", [2048])
@bench.axis("experts_per_rank", [32])
@bench.axis("top_k", [8])
def moe_layer(state, ctx):
    W = ctx.get_num_ranks()
    T, D, F, El, K = state["tokens"], state["hidden"], state["ffn"], state["experts_per_rank"], state["top_k"]
    E = El * W
    dt = torch.bfloat16
    wg = (torch.randn(El, D, F, device="cuda") * 0.02).to(dt)
    wu = (torch.randn(El, D, F, device="cuda") * 0.02).to(dt)
    wd = (torch.randn(El, F, D, device="cuda") * 0.02).to(dt)
    layer = MoELayer(ctx, D, F, E, K, max_tokens=T, w_gate=wg, w_up=wu, w_down=wd, capacity_factor=2.0)
    x = torch.randn(T, D, device="cuda", dtype=dt)
    logits = torch.randn(T, E, device="cuda")
    out = torch.empty_like(x)
    flops = 2 * T * K * (D * 2 * F + F * D)
    state.set_flops(flops)
    state.set_roofline_us(flops / (PEAK_TFLOPS * 1e6))
    state.set_repeat(20)
    state.set_warmup(5)
    state.exec(lambda: layer(x, logits, out=out))


if __name__ == "__main__":
    bench.main()
