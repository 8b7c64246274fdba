#!/usr/bin/env python3
"""Every all-reduce algorithm on the same tensor (reference: examples/16_all_reduce_ring_based and the
variants of iris/ccl/all_reduce.py: atomic, ring, one_shot, two_shot, spinlock), plus the ones
added here: push (small messages), nvls (multimem through the switch) and auto (chosen by size).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/all_reduce_variants.py
"""
import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init(1 << 30)
    from iris_b200.ccl import Config

    W, r = ctx.get_num_ranks(), ctx.get_rank()
    dt = torch.bfloat16 if torch.cuda.is_available() else torch.float32
    M, N = 512, 1024
    inp = ctx.full((M, N), float(r + 1), dtype=dt)
    want = float(sum(range(1, W + 1)))
    variants = ["atomic", "ring", "one_shot", "two_shot", "spinlock", "push", "auto"]
    if ctx.has_multicast():
        variants.append("nvls")
    for v in variants:
        out = ctx.zeros((M, N), dtype=dt)
        ctx.ccl.all_reduce(out, inp, config=Config(all_reduce_variant=v))
        assert torch.all(out.float() == want), v
    ctx.check()
    ctx.info("all-reduce variants validated: " + ", ".join(variants))
    finish(ctx)
