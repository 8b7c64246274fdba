#!/usr/bin/env python3
"""Ring attention (context parallelism): every rank holds a slice of the sequence; K/V blocks go
round the ring inside the kernel while attention consumes them (no counterpart in the reference).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/ring_attention.py
"""
import torch
import torch.distributed as dist

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.models import RingAttention, reference_attention

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    S, Hq, Hkv, D = 256, 8, 2, 128
    torch.manual_seed(20 + r)
    q = torch.randn(S, Hq, D, device=dev, dtype=dt)
    k = torch.randn(S, Hkv, D, device=dev, dtype=dt)
    v = torch.randn(S, Hkv, D, device=dev, dtype=dt)
    layer = RingAttention(ctx, S, Hq, Hkv, D)
    ks, vs = [torch.empty_like(k) for _ in range(W)], [torch.empty_like(v) for _ in range(W)]
    dist.all_gather(ks, k)
    dist.all_gather(vs, v)
    for causal in (False, True):
        out = layer(q, k, v, causal=causal)
        ref = reference_attention(q, torch.cat(ks), torch.cat(vs), causal, q_offset=r * S)
        assert (out.float() - ref.float()).abs().max().item() < 3e-2, causal
    ctx.check()
    ctx.info("ring attention validated (full and causal)")
    finish(ctx)
