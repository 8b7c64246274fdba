#!/usr/bin/env python3
"""Ring attention (context parallelism) throughput; the reference has no counterpart.

Every rank holds `seq_per_rank` tokens (32 query heads, 8 KV heads, head_dim 128, bf16) and attends
over the whole sequence of `num_ranks * seq_per_rank` tokens. FLOPs counted per rank:
4 * S * (W * S) * Hq * D (halved when causal). Roofline: those FLOPs at the measured sustained
bf16 tensor throughput; the K/V bytes that must cross NVLink ((W - 1) * S * Hkv * D * 2 * 2 per
rank at 770 GB/s) are far below it at these sizes."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import RingAttention  # noqa: E402

PEAK_TFLOPS = 1383.6


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("seq_per_rank", [2048, 8192])
@bench.axis("causal", [0, 1])
@bench.axis("layout", ["contiguous", "zigzag"])
def ring_attention(state, ctx):
    W, S, causal = ctx.get_num_ranks(), state["seq_per_rank"], bool(state["causal"])
    if state["layout"] == "zigzag" and not causal:
        state.skip("the layouts only differ under a causal mask")
    Hq, Hkv, D = 32, 8, 128
    dt = torch.bfloat16
    q = torch.randn(S, Hq, D, device="cuda", dtype=dt)
    k = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
    v = torch.randn(S, Hkv, D, device="cuda", dtype=dt)
    layer = RingAttention(ctx, S, Hq, Hkv, D, layout=state["layout"])
    out = torch.empty_like(q)
    flops = 4.0 * S * (W * S) * Hq * D * (0.5 if causal else 1.0)
    state.set_flops(flops)
    state.set_roofline_us(flops / (PEAK_TFLOPS * 1e6))
    state.set_repeat(20)
    state.set_warmup(5)
    state.exec(lambda: layer(q, k, v, causal=causal, out=out))


if __name__ == "__main__":
    bench.main()
