#!/usr/bin/env python3
"""One training step of a tensor-parallel MLP: forward and backward run on the fused GEMM +
collective kernels (`iris_b200.models.TensorParallelMLP`), the optimizer is plain torch.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/tp_mlp_training_step.py
"""
import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.models import TensorParallelMLP

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dev = ctx.get_device()
    gpu = torch.cuda.is_available()
    dt = torch.bfloat16 if gpu else torch.float32
    rows, hidden, ffn_local = (256, 512, 384) if gpu else (16, 32, 24)
    torch.manual_seed(r)
    mlp = TensorParallelMLP(ctx, hidden, ffn_local, activation="silu", dtype=dt)
    opt = torch.optim.SGD(mlp.parameters(), lr=0.05)
    x = torch.randn(rows, hidden, device=dev, dtype=dt)
    target = torch.randn(rows, hidden, device=dev, dtype=dt)
    losses = []
    for step in range(5):
        opt.zero_grad()
        loss = (mlp(x).float() - target.float()).square().mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
        ctx.barrier()
    assert losses[-1] < losses[0], losses
    ctx.check()
    ctx.info(f"loss {losses[0]:.4f} -> {losses[-1]:.4f}")
    finish(ctx)
