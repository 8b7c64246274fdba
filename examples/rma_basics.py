#!/usr/bin/env python3
"""One-sided operations from the host: load, store, get, put and atomics between ranks (reference:
examples/00_load, 01_store, 02_all_load, 03_all_store, 04_atomic_add, 05_atomic_xchg). Works on the
GPU backend (small kernels built on include/iris/rma.cuh) and on the CPU backend (gloo).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/rma_basics.py
"""
import torch

from _common import finish, init

if __name__ == "__main__":
    ctx = init(256 << 20)
    W, r = ctx.get_num_ranks(), ctx.get_rank()
    peer = (r + 1) % W
    n = 4096
    src = ctx.arange(0, n, dtype=torch.float32)
    src += 1000.0 * r
    dst = ctx.zeros(n, dtype=torch.float32)
    counter = ctx.zeros(1, dtype=torch.int32)
    slot = ctx.zeros(1, dtype=torch.int32)
    ctx.barrier()

    # load: read the neighbour's copy of `src`                                   (00_load, 02_all_load)
    got = ctx.rma.load(src, from_rank=peer)
    assert torch.equal(got.cpu(), torch.arange(n, dtype=torch.float32) + 1000.0 * peer)
    # store / put: write into the neighbour's `dst`                              (01_store, 03_all_store)
    ctx.rma.put(src, dst, to_rank=peer)
    ctx.barrier()
    left = (r - 1) % W
    assert torch.equal(dst.cpu(), torch.arange(n, dtype=torch.float32) + 1000.0 * left)
    # get: pull the neighbour's `src` into local memory
    mine = ctx.zeros(n, dtype=torch.float32)
    ctx.rma.get(src, mine, from_rank=peer)
    assert torch.equal(mine.cpu(), got.cpu())
    # atomics: every rank adds 1 to every rank's counter, then swaps its rank into rank 0's slot (04, 05)
    for p in range(W):
        ctx.rma.atomic_add(counter, 1, to_rank=p)
    ctx.rma.atomic_xchg(slot, r + 1, to_rank=0)
    ctx.barrier()
    assert int(counter.item()) == W
    if r == 0:
        assert 1 <= int(slot.item()) <= W
    ctx.check()
    ctx.info("load / store / get / put / atomics validated")
    finish(ctx)
