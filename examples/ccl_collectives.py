#!/usr/bin/env python3
"""The four collectives with validation (reference: examples/24_ccl_all_reduce .. 27_ccl_reduce_scatter).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/ccl_collectives.py
"""
import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init()
    from iris_b200.ccl import Config

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    M, N = 1024, 512 * W
    inp = ctx.full((M, N), float(r + 1), dtype=torch.float32)
    out = ctx.zeros((M, N), dtype=torch.float32)
    ctx.ccl.all_reduce(out, inp)
    assert torch.all(out == W * (W + 1) / 2)
    gathered = ctx.zeros((W * M, N), dtype=torch.float32)
    ctx.ccl.all_gather(gathered, inp)
    assert all(torch.all(gathered[s * M:(s + 1) * M] == s + 1) for s in range(W))
    a2a = ctx.zeros((M, N), dtype=torch.float32)
    ctx.ccl.all_to_all(a2a, inp)
    assert all(torch.all(a2a[:, s * (N // W):(s + 1) * (N // W)] == s + 1) for s in range(W))
    rs = ctx.zeros((M // W, N), dtype=torch.float32)
    ctx.ccl.reduce_scatter(rs, inp, config=Config(reduce_scatter_rows=True))
    assert torch.all(rs == W * (W + 1) / 2)
    ctx.check()
    ctx.info("all_reduce, all_gather, all_to_all, reduce_scatter validated")
    finish(ctx)
