#!/usr/bin/env python3
"""Ring attention (context parallelism) throughput; the reference has no counterpart.

Every rank holds `seq_per_rank` tokens (32 query heads, 8 KV heads, head_dim 128, bf16) and attends
over the whole sequence of `num_ranks * seq_per_rank` tokens. FLOPs counted per rank:
4 * S * (W * S) * Hq * D (halved when causal). Roofline: those FLOPs at the measured sustained
bf16 tensor throughput; the K/V bytes that must cross NVLink ((W - 1) * S * Hkv * D * 2 * 2 per
rank at 770 GB/s) are far below it at these sizes.

``impl=nccl`` is the unfused form: NCCL ``all_gather_into_tensor`` of K and V, then one library attention
call over the gathered keys (flash_attn, whose causal mask is aligned to the end of the key sequence, so
rank r attends to keys [0, (r + 1) * S); contiguous layout only)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import RingAttention, reference_attention, zigzag_positions  # noqa: E402

PEAK_TFLOPS = 1383.6


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("seq_per_rank", [2048, 8192])
@bench.axis("causal", [0, 1])
@bench.axis("layout", ["contiguous", "zigzag"])
def ring_attention(state, ctx):
    W, S, causal = ctx.get_num_ranks(), state["seq_per_rank"], bool(state["causal"])
    if state["layout"] == "zigzag" and not causal:
        state.skip("the layouts only differ under a causal mask")
    Hq, Hkv, D = 32, 8, 128
    dev = ctx.get_device()
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32          # gloo ranks: the layer's host path, fp32
    q = torch.randn(S, Hq, D, device=dev, dtype=dt)
    k = torch.randn(S, Hkv, D, device=dev, dtype=dt)
    v = torch.randn(S, Hkv, D, device=dev, dtype=dt)
    layer = RingAttention(ctx, S, Hq, Hkv, D, layout=state["layout"])
    out = torch.empty_like(q)
    flops = 4.0 * S * (W * S) * Hq * D * (0.5 if causal else 1.0)
    state.set_flops(flops)
    state.set_roofline_us(flops / (PEAK_TFLOPS * 1e6))
    state.set_repeat(min(state.n_repeat, 20))            # long kernels: fewer repeats than the default, never more than asked for
    state.set_warmup(min(state.n_warmup, 5))
    if state["impl"] == "nccl":
        if state["layout"] != "contiguous":
            state.skip("the NCCL baseline gathers a contiguous sequence")
        try:
            from flash_attn import flash_attn_func
        except Exception:
            state.skip("flash_attn is not importable")
        kall = torch.empty(W * S, Hkv, D, device=dev, dtype=dt)
        vall = torch.empty(W * S, Hkv, D, device=dev, dtype=dt)
        rank = ctx.get_rank()

        def base():
            if W > 1:
                dist.all_gather_into_tensor(kall, k)
                dist.all_gather_into_tensor(vall, v)
            else:
                kall.copy_(k)
                vall.copy_(v)
            n = (rank + 1) * S if causal else W * S
            out.copy_(flash_attn_func(q[None], kall[None, :n], vall[None, :n], causal=causal)[0])

        state.exec(base)
        return
    # deviation of the last 64 query rows of this rank from fp32 attention over the gathered sequence (a counter:
    # benchmarks report, tests assert; bf16 gives a few 1e-3). Every rank runs the same collectives here.
    got = layer(q, k, v, causal=causal, out=out)
    ks, vs = [torch.empty_like(k) for _ in range(W)], [torch.empty_like(v) for _ in range(W)]
    if W > 1:
        dist.all_gather(ks, k)
        dist.all_gather(vs, v)
    else:
        ks, vs = [k], [v]
    pos = [zigzag_positions(r, W, S, device=dev) if state["layout"] == "zigzag" else r * S + torch.arange(S, device=dev) for r in range(W)]
    rows = slice(S - min(64, S), S)
    ref = reference_attention(q[rows], torch.cat(ks), torch.cat(vs), causal=causal, q_pos=pos[ctx.get_rank()][rows], k_pos=torch.cat(pos))
    state.add_counter("max_rel_err", round((got[rows].float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12), 6))
    del ks, vs, ref
    state.exec(lambda: layer(q, k, v, causal=causal, out=out))


if __name__ == "__main__":
    bench.main()
