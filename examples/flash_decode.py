#!/usr/bin/env python3
"""Distributed flash decode: the KV cache of every sequence is split over the ranks, each rank
attends to its shard and the partial results are merged across ranks inside the layer (reference:
examples/13_flash_decode). Validated against attention over the concatenated cache.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/flash_decode.py
"""
import torch
import torch.distributed as dist

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.models import FlashDecodeLayer, merge_partials, reference_decode

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    B, Hq, Hkv, D, page = 4, 16, 2, 128, 64
    lens = torch.tensor([300, 1000, 64, 777])            # keys of every sequence on THIS rank's shard
    nb = int(-(-lens.max() // page))
    torch.manual_seed(100 + r)
    kc = torch.randn(B * nb, page, Hkv, D, device=dev, dtype=dt)
    vc = torch.randn(B * nb, page, Hkv, D, device=dev, dtype=dt)
    table = torch.arange(B * nb, device=dev, dtype=torch.int32).view(B, nb)
    torch.manual_seed(7)                                   # the query is the same on every rank
    q = torch.randn(B, Hq, D, device=dev, dtype=dt)
    kv_lens = lens.to(dev).to(torch.int32).repeat(W, 1)    # [W, B]: every shard has the same lengths here
    layer = FlashDecodeLayer(ctx, Hq, Hkv, D, max_batch=B)
    out = layer(q, kc, vc, kv_lens, table)
    # reference: merge the per-shard fp32 results of all ranks
    o, lse = reference_decode(q, kc, vc, kv_lens[r], table)
    os_, ls_ = [torch.empty_like(o) for _ in range(W)], [torch.empty_like(lse) for _ in range(W)]
    dist.all_gather(os_, o)
    dist.all_gather(ls_, lse)
    ref = merge_partials(torch.stack(os_), torch.stack(ls_))
    assert (out.float() - ref).abs().max().item() < 3e-2
    ctx.check()
    ctx.info("distributed flash decode validated")
    finish(ctx)
