#!/usr/bin/env python3
"""The parallelism package end to end: a layout, tensor-parallel linears, a Ulysses attention
exchange, data-parallel gradient buckets and a point-to-point hand-over between neighbours. No
counterpart in the reference, which stops at the collectives and leaves their composition to the
caller.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/parallel_layouts.py

Every stage is checked against the same computation done unsharded in fp32.
"""
import torch
import torch.distributed as dist

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.models import reference_attention
    from iris_b200.parallel import (ColumnParallelLinear, GradientBuckets, ParallelLayout, RowParallelLinear, UlyssesExchange,
                                    shard_sequence)
    from iris_b200.utils import validate_all_reduce

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    tol = 0.06 if dt == torch.bfloat16 else 1e-3

    # ---- layout: all ranks form one tensor-parallel group here; with more ranks add "dp"
    layout = ParallelLayout({"tp": W}).build_groups()
    assert layout.group("tp") is None and layout.ranks("tp") == list(range(W))

    # ---- tensor-parallel MLP from the two linear layers, sequence-parallel activations
    S, hidden, ffn_local = 128 * W, 256, 256
    g = torch.Generator().manual_seed(0)
    X = (torch.randn(S, hidden, generator=g) * 0.5)
    W1 = torch.randn(hidden, ffn_local * W, generator=g) * 0.05
    W2 = torch.randn(ffn_local * W, hidden, generator=g) * 0.05
    up = ColumnParallelLinear(ctx, hidden, ffn_local, dtype=dt, weight=W1[:, r * ffn_local:(r + 1) * ffn_local].to(dt))
    down = RowParallelLinear(ctx, ffn_local, hidden, dtype=dt, weight=W2[r * ffn_local:(r + 1) * ffn_local].to(dt))
    x_mine = shard_sequence(X, r, W).to(dev, dt)
    y = down(torch.nn.functional.silu(up(x_mine)))
    ref = (torch.nn.functional.silu(X.to(dt).float() @ W1.to(dt).float()) @ W2.to(dt).float())[r * (S // W):(r + 1) * (S // W)]
    err = (y.float().cpu() - ref).abs().max().item()
    assert err < tol * max(ref.abs().max().item(), 1.0), err

    # ---- Ulysses: tokens sharded -> heads sharded, attention on full sequences, and back
    H, D = 2 * W, 64
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    ex = UlyssesExchange(ctx)
    heads = [ex.to_heads(shard_sequence(t, r, W).to(dev, dt)).clone() for t in (q, k, v)]
    o_heads = reference_attention(*heads, causal=True).to(dt)
    o_mine = ex.to_sequence(o_heads)
    want = reference_attention(q.to(dt), k.to(dt), v.to(dt), causal=True)[r * (S // W):(r + 1) * (S // W)]
    assert (o_mine.float().cpu() - want.float().cpu()).abs().max().item() < tol

    # ---- data parallel: every rank a replica, gradients averaged through heap buckets
    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 8)).to(dev)
    buckets = GradientBuckets(ctx, model.parameters(), bucket_bytes=16 << 10).attach()
    data = torch.randn(16, 64, generator=torch.Generator().manual_seed(10 + r)).to(dev)
    model(data).square().mean().backward()
    local = [p.grad.detach().clone() for p in model.parameters()]
    buckets.finish()
    for p, gl in zip(model.parameters(), local):
        mine = ctx.as_symmetric(gl.reshape(1, -1).contiguous())
        assert validate_all_reduce(mine, p.grad.reshape(1, -1) * W, ctx, atol=1e-4)
    # ---- pipeline-style hand-over: every rank passes micro-batches to its successor through mailboxes
    if W > 1:
        from iris_b200.parallel import P2PChannel

        ch = P2PChannel(ctx, (32, 64), dtype=torch.float32, depth=2)
        for step in range(4):
            ch.send(torch.full((32, 64), float(10 * r + step), device=dev), (r + 1) % W)
            got = ch.recv((r - 1) % W)
            assert torch.all(got == 10 * ((r - 1) % W) + step)
    ctx.check()
    ctx.info(f"parallel layouts validated ({len(buckets.buckets)} gradient buckets, MLP error {err:.3g} of {ref.abs().max().item():.3g})")
    dist.barrier()
    finish(ctx)
