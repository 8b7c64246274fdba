#!/usr/bin/env python3
"""Distributed flash-decode throughput (reference: benchmark/examples/bench_flash_decode.py).

64 query heads, 8 KV heads, head_dim 128, bf16; the total KV length is split evenly over the ranks.
Bytes counted are the K and V bytes each rank must read (the roofline is those bytes over the
measured HBM bandwidth).

``impl=nccl`` is the reference's baseline (examples/benchmark/reference/flash_decode_rccl/
flash_decode_layer_rccl.py:100-130): the same local split-K decode, then ``all_gather_into_tensor`` of
the partial (o, lse) over NCCL and a log-sum-exp merge, instead of the in-kernel exchange."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import iris_b200.bench as bench  # noqa: E402
from iris_b200.models import FlashDecodeLayer  # noqa: E402

HBM_GBPS = 6553.0


@bench.register
@bench.axis("num_ranks", [1, 2, 4, 8])
@bench.axis("impl", ["iris", "nccl"])
@bench.axis("batch", [1, 8, 32, 64])
@bench.axis("total_kv", [32768, 131072, 524288])
def flash_decode(state, ctx):
    W, B, total = ctx.get_num_ranks(), state["batch"], state["total_kv"]
    Hq, Hkv, D, page = 64, 8, 128, 64
    L = total // max(W, 8) if W < 8 else total // W     # per-rank shard of the 8-way split
    nb = -(-L // page)
    need = 2 * B * nb * page * Hkv * D * 2
    if need > 60 << 30:
        state.skip("KV shard does not fit the benchmark's memory budget")
    dt = torch.bfloat16
    kc = torch.randn(B * nb, page, Hkv, D, device="cuda", dtype=dt)
    vc = torch.randn(B * nb, page, Hkv, D, device="cuda", dtype=dt)
    table = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
    lens = torch.full((W, B), L, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=dt)
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=B)
    out = torch.empty(B, Hq, D, device="cuda", dtype=dt)
    kv_bytes = 2 * B * L * Hkv * D * 2
    state.set_bytes(kv_bytes)
    state.set_roofline_us(kv_bytes / (HBM_GBPS * 1e3))
    state.set_repeat(30)
    if state["impl"] == "nccl":
        po = torch.empty(B, Hq, D, device="cuda", dtype=dt)
        g_o = torch.empty(W, B, Hq, D, device="cuda", dtype=dt)
        g_l = torch.empty(W, B, Hq, device="cuda", dtype=torch.float32)

        def base():
            _, pl = layer(q, kc, vc, lens, table, out=po, local_only=True)
            if W > 1:
                dist.all_gather_into_tensor(g_o, po)
                dist.all_gather_into_tensor(g_l, pl)
                out.copy_(FlashDecodeLayer.merge_partials(g_o, g_l))
            else:
                out.copy_(po)

        state.exec(base)
        return
    state.exec(lambda: layer(q, kc, vc, lens, table, out=out))


if __name__ == "__main__":
    bench.main()
