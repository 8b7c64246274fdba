"""RMA plumbing on the CPU backend, gloo, world_size 2 (no GPU).

Scenario: a 1 GiB symmetric heap per rank; a 4096-element fp32 buffer, zero-initialised; rank 0
stores 1.0 into rank 1's buffer in 1024-element blocks; every rank atomically adds int32 1 to
every peer's counter (and its own); barrier; rank 1's buffer is all ones and every counter equals
world_size.
"""
import torch

from helpers import run_ranks


def _scenario(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 30)
    assert ctx.get_rank() == rank and ctx.get_num_ranks() == world
    buf = ctx.zeros(4096, dtype=torch.float32)
    counter = ctx.zeros(1, dtype=torch.int32)
    assert ctx.is_symmetric(buf) and ctx.is_symmetric(counter)
    bases = ctx.get_heap_bases()
    assert bases.dtype == torch.int64 and bases.numel() == world
    assert int(bases[rank]) == ctx.heap.base
    ctx.barrier()
    if rank == 0:
        for blk in range(4):
            ctx.rma.store(buf[blk * 1024:(blk + 1) * 1024], 1.0, to_rank=1)
    for peer in range(world):
        old = ctx.rma.atomic_add(counter, 1, to_rank=peer, sem="acq_rel", scope="sys")
        assert 0 <= int(old.item()) < world
    ctx.barrier()
    expected = 1.0 if rank == 1 else 0.0
    assert torch.all(buf == expected), f"rank {rank}: {buf[:8]}"
    assert int(counter.item()) == world
    # the remote view of the same buffer shows what the other rank holds
    other = ctx.heap.peer_view(buf, 1 - rank)
    assert torch.all(other == (1.0 if (1 - rank) == 1 else 0.0))
    ctx.barrier()


def test_rma_plumbing_world2():
    run_ranks(_scenario, 2)


def _ops(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    a = ctx.arange(0, 64, dtype=torch.int32)
    a += rank * 1000
    b = ctx.zeros(64, dtype=torch.int32)
    ctx.barrier()
    peer = (rank + 1) % world
    # load / get read the peer's copy
    got = ctx.rma.load(a, from_rank=peer)
    assert torch.equal(got, torch.arange(64, dtype=torch.int32) + peer * 1000)
    ctx.rma.get(a, b, from_rank=peer)
    assert torch.equal(b, got)
    ctx.barrier()
    # put / copy write the peer's copy
    b.zero_()
    ctx.barrier()
    ctx.rma.put(a, b, to_rank=peer)
    ctx.barrier()
    src = (rank - 1) % world
    assert torch.equal(b, torch.arange(64, dtype=torch.int32) + src * 1000)
    ctx.barrier()
    c = ctx.zeros(64, dtype=torch.int32)
    ctx.barrier()
    ctx.rma.copy(a, c, from_rank=rank, to_rank=peer)
    ctx.barrier()
    assert torch.equal(c, torch.arange(64, dtype=torch.int32) + src * 1000)
    # atomics on the peer
    f = ctx.full((8,), 5, dtype=torch.int32)
    ctx.barrier()
    ctx.rma.atomic_max(f, 9 + rank, to_rank=peer)
    ctx.barrier()
    assert torch.all(f == 9 + src)
    ctx.barrier()                 # everybody has looked before anybody changes the cells again
    # the peer's cells now hold 9 + (its predecessor) = 9 + my rank: the swap goes through
    old = ctx.rma.atomic_cas(f, 9 + rank, 42, to_rank=peer)
    assert torch.all(old == 9 + rank)
    ctx.barrier()
    assert torch.all(f == 42)
    x = ctx.rma.atomic_xchg(f, 7, to_rank=rank)
    assert torch.all(x == 42) and torch.all(f == 7)
    ctx.barrier()


def test_rma_ops_world2():
    run_ranks(_ops, 2)


def test_rma_ops_world3():
    run_ranks(_ops, 3)
