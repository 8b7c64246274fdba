#!/usr/bin/env python3
"""The fused GEMM + collective ops with validation (reference: examples/28_ops_matmul_all_reduce,
29_ops_all_gather_matmul, 30_ops_matmul_all_gather).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/ops_fused.py
"""
import torch
import torch.distributed as dist

from _common import finish, init

if __name__ == "__main__":
    ctx = init(4 << 30)
    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev, dt = ctx.get_device(), (torch.bfloat16 if torch.cuda.is_available() else torch.float32)
    torch.manual_seed(r)
    M_local, K, N = 512, 1024, 768
    A = torch.randn(M_local, K, device=dev, dtype=dt)
    B = torch.randn(K, N, device=dev, dtype=dt) * 0.05
    # all_gather_matmul: every rank contributes its rows of A
    C = ctx.zeros((W * M_local, N), dtype=dt)
    ctx.ops.all_gather_matmul(C, A, B, shard_dim=0)
    Aall = [torch.empty_like(A) for _ in range(W)]
    dist.all_gather(Aall, A)
    ref = torch.cat(Aall).float() @ B.float()
    assert (C.float() - ref).abs().max() < 0.05 * ref.abs().max()
    # matmul_all_reduce: every rank contributes a partial product
    C2 = ctx.zeros((M_local, N), dtype=dt)
    ctx.ops.matmul_all_reduce(C2, A, B)
    tot = A.float() @ B.float()
    dist.all_reduce(tot)
    assert (C2.float() - tot).abs().max() < 0.05 * tot.abs().max()
    # matmul_all_gather (30): every rank's row block of the product lands on all ranks
    C3 = ctx.zeros((W * M_local, N), dtype=dt)
    ctx.ops.matmul_all_gather(C3, A, B)
    mine = A.float() @ B.float()
    blocks = [torch.empty_like(mine) for _ in range(W)]
    dist.all_gather(blocks, mine)
    assert (C3.float() - torch.cat(blocks)).abs().max() < 0.05 * mine.abs().max()
    # the same all_gather_matmul on block-scaled e4m3 operands (1 x 128 activation scales, 128 x 128 weight
    # scales, powers of two): the oracle is the product of the dequantised operands
    from iris_b200.ops import quantize_activation, quantize_weight

    Aq, Bq = quantize_activation(A), quantize_weight(B.t().contiguous())       # weight stored (out, in)
    C4 = ctx.zeros((W * M_local, N), dtype=torch.bfloat16)
    ctx.ops.all_gather_matmul(C4, Aq, Bq, shard_dim=0)
    Adq = Aq.dequantize().float()
    Adq_all = [torch.empty_like(Adq) for _ in range(W)]
    dist.all_gather(Adq_all, Adq)
    ref8 = torch.cat(Adq_all) @ Bq.dequantize().float()          # the quantised weight presents itself as [K, N]
    assert (C4.float() - ref8).abs().max() < 0.05 * ref8.abs().max()
    ctx.check()
    ctx.info("all_gather_matmul (bf16 and e4m3), matmul_all_reduce and matmul_all_gather validated")
    finish(ctx)
