"""Every one-sided operation x dtype x memory order, exact compare, on gloo ranks (no GPU).

The reference tests each device op in a file of its own (tests/unittests/test_load_triton.py,
test_store_triton.py, test_get_*, test_put_*, test_copy_*, test_atomic_{add,and,cas,max,min,or,xchg,
xor}_triton.py: a tiny kernel, a sweep over dtype x sem x scope x BLOCK_SIZE, rtol = atol = 0).
Here one pair of ranks walks the whole table through ``ctx.rma``, which runs the device header's
functions over a range of elements; the expected values are written out with plain torch.
"""
import itertools

import pytest
import torch

from helpers import run_ranks

MOVE_DTYPES = ["float16", "bfloat16", "float32", "float64", "int8", "uint8", "int16", "int32", "int64"]
ATOMIC_INT = ["int32", "int64"]
ATOMIC_FLOAT = ["float32", "float64"]
SEMS = ["relaxed", "acquire", "release", "acq_rel"]
SCOPES = ["cta", "gpu", "sys"]
SIZES = [1, 8, 33, 512]


def _pattern(n, dtype, rank):
    """Distinct per rank, exactly representable in every dtype of the sweep."""
    return ((torch.arange(n, dtype=torch.int64) % 50) + 10 * (rank + 1)).to(dtype)


def _movement(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    peer = (rank + 1) % world
    prev = (rank - 1) % world
    for name, n in itertools.product(MOVE_DTYPES, SIZES):
        dt = getattr(torch, name)
        src = ctx.zeros(n, dtype=dt)
        dst = ctx.zeros(n, dtype=dt)
        src.copy_(_pattern(n, dt, rank))
        ctx.barrier()
        # load: what the peer holds, returned locally; the peer's memory is untouched
        got = ctx.rma.load(src, from_rank=peer)
        assert got.dtype == dt and torch.equal(got, _pattern(n, dt, peer)), (name, n, "load")
        assert torch.equal(ctx.rma.load(src, from_rank=rank), _pattern(n, dt, rank)), (name, n, "load self")
        # get: peer's src -> my dst
        ctx.rma.get(src, dst, from_rank=peer)
        assert torch.equal(dst, _pattern(n, dt, peer)), (name, n, "get")
        ctx.barrier()
        dst.zero_()
        ctx.barrier()
        # put: my src -> peer's dst, so my dst receives prev's pattern
        ctx.rma.put(src, dst, to_rank=peer)
        ctx.barrier()
        assert torch.equal(dst, _pattern(n, dt, prev)), (name, n, "put")
        ctx.barrier()
        dst.zero_()
        ctx.barrier()
        # copy, caller is the source
        ctx.rma.copy(src, dst, from_rank=rank, to_rank=peer)
        ctx.barrier()
        assert torch.equal(dst, _pattern(n, dt, prev)), (name, n, "copy push")
        ctx.barrier()
        dst.zero_()
        ctx.barrier()
        # copy, caller is the destination
        ctx.rma.copy(src, dst, from_rank=peer, to_rank=rank)
        assert torch.equal(dst, _pattern(n, dt, peer)), (name, n, "copy pull")
        ctx.barrier()
        # store: scalar and tensor values
        dst.zero_()
        ctx.barrier()
        ctx.rma.store(dst, 3, to_rank=peer)
        ctx.barrier()
        assert torch.all(dst == 3), (name, n, "store scalar")
        ctx.barrier()
        ctx.rma.store(dst, _pattern(n, dt, rank) + 1, to_rank=peer)
        ctx.barrier()
        assert torch.equal(dst, _pattern(n, dt, prev) + 1), (name, n, "store tensor")
        # the source never changed
        assert torch.equal(src, _pattern(n, dt, rank)), (name, n, "source intact")
        ctx.barrier()
    # cache modifiers and the volatile flag are accepted for every op that takes them
    t = ctx.zeros(16, dtype=torch.float32)
    t.fill_(float(rank + 1))
    ctx.barrier()
    for cm in (None, "", ".ca", ".cg", ".cs", ".cv"):
        for vol in (False, True):
            assert torch.all(ctx.rma.load(t, from_rank=peer, cache_modifier=cm, volatile=vol) == peer + 1)
    ctx.barrier()
    for i, cm in enumerate((None, "", ".wb", ".cg", ".cs", ".wt")):
        ctx.rma.store(t, 100 + i, to_rank=peer, cache_modifier=cm)
        ctx.barrier()
        assert torch.all(t == 100 + i)
        ctx.barrier()
    with pytest.raises(ValueError):
        ctx.rma.load(t, from_rank=peer, cache_modifier=".zz")
    with pytest.raises(ValueError):
        ctx.rma.load(t, from_rank=world)
    with pytest.raises(ValueError):
        ctx.rma.copy(t, t, from_rank=peer, to_rank=peer) if world > 2 else ctx.rma.load(t, from_rank=-1)
    ctx.barrier()


def test_data_movement_every_dtype_world2():
    run_ranks(_movement, 2)


def _atomics(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    peer = (rank + 1) % world
    prev = (rank - 1) % world
    n = 33
    for name, sem, scope in itertools.product(ATOMIC_INT + ATOMIC_FLOAT, SEMS, SCOPES):
        dt = getattr(torch, name)
        is_int = not dt.is_floating_point
        t = ctx.zeros(n, dtype=dt)
        base = _pattern(n, dt, 0)

        def reset():
            ctx.barrier()
            t.copy_(base)
            ctx.barrier()

        kw = dict(sem=sem, scope=scope)
        # add: every rank adds (rank + 1) to everyone (itself included); old values are in range
        reset()
        total = sum(r + 1 for r in range(world))
        for dest in range(world):
            old = ctx.rma.atomic_add(t, rank + 1, to_rank=dest, **kw)
            assert torch.all(old >= base) and torch.all(old <= base + total), (name, sem, scope, "add old")
        ctx.barrier()
        assert torch.equal(t, base + total), (name, sem, scope, "add")
        # sub
        reset()
        old = ctx.rma.atomic_sub(t, 2, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, base - 2), (name, sem, scope, "sub")
        # min / max against a per-element tensor
        reset()
        lim = torch.full((n,), 30, dtype=dt)
        old = ctx.rma.atomic_min(t, lim, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, torch.minimum(base, lim)), (name, sem, scope, "min")
        reset()
        old = ctx.rma.atomic_max(t, lim, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, torch.maximum(base, lim)), (name, sem, scope, "max")
        # xchg: my value lands on the peer, I get what was there
        reset()
        old = ctx.rma.atomic_xchg(t, 1000 + rank, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.all(t == 1000 + prev), (name, sem, scope, "xchg")
        if not is_int:
            with pytest.raises(TypeError):
                ctx.rma.atomic_cas(t, 0, 1, to_rank=peer)
            with pytest.raises(RuntimeError):
                ctx.rma.atomic_and(t, 1, to_rank=peer)
            continue
        # bitwise
        reset()
        old = ctx.rma.atomic_and(t, 0x0F, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, base & 0x0F), (name, sem, scope, "and")
        reset()
        old = ctx.rma.atomic_or(t, 0x100, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, base | 0x100), (name, sem, scope, "or")
        reset()
        old = ctx.rma.atomic_xor(t, 0x55, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base) and torch.equal(t, base ^ 0x55), (name, sem, scope, "xor")
        # cas: only elements equal to `cmp` are swapped
        reset()
        old = ctx.rma.atomic_cas(t, 12, 77, to_rank=peer, **kw)
        ctx.barrier()
        assert torch.equal(old, base), (name, sem, scope, "cas old")
        assert torch.equal(t, torch.where(base == 12, torch.full_like(base, 77), base)), (name, sem, scope, "cas")
    # lock built from cas / xchg: increments under the lock are never lost
    lock = ctx.zeros(1, dtype=torch.int32)
    cell = ctx.zeros(1, dtype=torch.int64)
    ctx.barrier()
    for _ in range(50):
        while int(ctx.rma.atomic_cas(lock, 0, 1, to_rank=0, sem="acquire", scope="sys").item()) != 0:
            pass
        v = ctx.rma.load(cell, from_rank=0)
        ctx.rma.store(cell, int(v.item()) + 1, to_rank=0)
        ctx.rma.atomic_xchg(lock, 0, to_rank=0, sem="release", scope="sys")
    ctx.barrier()
    if rank == 0:
        assert int(cell.item()) == 50 * world
    with pytest.raises(ValueError):
        ctx.rma.atomic_add(lock, 1, to_rank=0, sem="seq_cst")
    with pytest.raises(ValueError):
        ctx.rma.atomic_add(lock, 1, to_rank=0, scope="cluster")
    ctx.barrier()


def test_atomics_every_order_and_scope_world2():
    run_ranks(_atomics, 2)


def test_atomics_world3():
    run_ranks(_atomics, 3, timeout=600.0)
