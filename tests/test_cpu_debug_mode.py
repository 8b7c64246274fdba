"""Debug aids on gloo ranks (no GPU): ``IRIS_DEBUG=1``, heap checks of host RMA, simulation dump.

The reference has no sanitizer or debug build (it relies on ``tl.debug_barrier`` and hand-placed
acquire / release atomics); its only run-time aid is the heap-bases JSON of simulation runs
(iris/host/iris.py:119-134). Checked here: poisoned fresh memory, divergence reported at the first
barrier after it happens, one-sided operations on a tensor that is not on the heap refused before
any address is formed, and the JSON file.
"""
import json
import os

import pytest
import torch

from helpers import run_ranks


def _poison(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    assert ctx.debug_checks and ctx.heap.poison
    for dt in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        assert torch.isnan(ctx.empty(257, dtype=dt)).all(), dt
    for dt in (torch.int8, torch.int16, torch.int32, torch.int64):
        assert torch.all(ctx.empty(65, dtype=dt) == -1), dt
    assert torch.all(ctx.empty(9, dtype=torch.uint8) == 255)
    # initialising factories are unaffected
    assert torch.all(ctx.zeros(33) == 0) and torch.all(ctx.ones(33, dtype=torch.int32) == 1)
    assert torch.equal(ctx.arange(5), torch.arange(5))
    # collectives still work, and end with the debug checks
    inp = ctx.full((4, 4 * world), float(rank + 1))
    out = ctx.empty((4, 4 * world))
    ctx.ccl.all_reduce(out, inp)
    assert torch.all(out == sum(range(1, world + 1)))
    # memory handed out again after a release is poisoned again
    mark = ctx.heap_mark()
    a = ctx.zeros(128)
    del a
    ctx.heap_release(mark)
    assert torch.isnan(ctx.empty(128)).all()
    ctx.barrier()


def test_debug_mode_poisons_fresh_memory():
    run_ranks(_poison, 2, env={"IRIS_DEBUG": "1"})


def _divergence(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    ctx.barrier()                       # heaps agree: passes
    if rank == 1:
        ctx.heap.allocate(100, torch.float32)   # one rank allocates behind the others' back
    with pytest.raises(RuntimeError, match="offsets differ"):
        ctx.barrier()


def test_debug_mode_reports_divergent_heaps_at_the_next_barrier():
    run_ranks(_divergence, 2, env={"IRIS_DEBUG": "1"})


def _status_at_barrier(rank, world):
    import iris_b200 as iris
    from iris_b200.host.iris import IrisTimeoutError

    ctx = iris.iris(1 << 24)
    ctx._status.fill_(2)                # what a kernel leaves behind when a flag wait runs out
    with pytest.raises(IrisTimeoutError) as e:
        ctx.barrier()
    assert e.value.code == 2 and e.value.rank == rank and "flag" in str(e.value)
    assert int(ctx._status.item()) == 0     # reading the status clears it; the context stays usable
    import torch.distributed as dist

    dist.barrier()
    ctx.barrier()


def test_debug_mode_raises_a_recorded_status_at_the_barrier():
    run_ranks(_status_at_barrier, 2, env={"IRIS_DEBUG": "1"})


def _off_by_default(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    assert not ctx.debug_checks and not ctx.heap.poison
    ctx._status.fill_(2)
    ctx.barrier()                       # no check without the debug flag
    assert int(ctx._status.item()) == 2
    ctx._status.zero_()
    ctx.barrier()


def test_debug_checks_are_off_by_default():
    run_ranks(_off_by_default, 2)


def _rma_heap_check(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    peer = 1 - rank
    on_heap = ctx.zeros(16)
    private = torch.zeros(16)
    ctx.barrier()
    for call in (lambda: ctx.rma.load(private, from_rank=peer),
                 lambda: ctx.rma.store(private, 1.0, to_rank=peer),
                 lambda: ctx.rma.get(private, on_heap, from_rank=peer),
                 lambda: ctx.rma.put(on_heap, private, to_rank=peer),
                 lambda: ctx.rma.copy(private, on_heap, from_rank=peer, to_rank=rank),
                 lambda: ctx.rma.copy(on_heap, private, from_rank=rank, to_rank=peer),
                 lambda: ctx.rma.atomic_add(private, 1.0, to_rank=peer),
                 lambda: ctx.rma.atomic_xchg(private, 1.0, to_rank=peer)):
        with pytest.raises(ValueError, match="symmetric heap"):
            call()
    # the local end of a get / put may be any tensor, and so may a target on the calling rank
    on_heap.fill_(float(rank + 1))
    ctx.barrier()
    ctx.rma.get(on_heap, private, from_rank=peer)
    assert torch.all(private == peer + 1)
    private.fill_(7.0)
    ctx.rma.put(private, on_heap, to_rank=peer)
    ctx.barrier()
    assert torch.all(on_heap == 7.0)
    ctx.rma.store(private, 3.0, to_rank=rank)
    assert torch.all(private == 3.0)
    assert torch.all(ctx.rma.load(private, from_rank=rank) == 3.0)
    ctx.barrier()


def test_host_rma_refuses_tensors_outside_the_heap():
    run_ranks(_rma_heap_check, 2)


def _simulation(rank, world, prefix):
    import iris_b200 as iris

    assert iris.is_simulation_env()
    ctx = iris.iris(1 << 22)
    path = f"{prefix}_rank_{rank}_heap_bases.json"
    with open(path) as f:
        rec = json.load(f)
    assert rec["rank"] == rank and rec["num_ranks"] == world and len(rec["heap_bases"]) == world
    assert [int(b, 16) for b in rec["heap_bases"]] == [int(b) & (2**64 - 1) for b in ctx.get_heap_bases().tolist()]
    assert int(rec["heap_bases"][rank], 16) == ctx.heap.base
    ctx.barrier()


def test_simulation_mode_writes_the_heap_bases(tmp_path):
    prefix = str(tmp_path / "sim")
    run_ranks(_simulation, 2, args=(prefix,), env={"IRIS_SIMULATION": "1", "IRIS_HEAP_BASES_PREFIX": prefix})
    assert sorted(os.listdir(tmp_path)) == ["sim_rank_0_heap_bases.json", "sim_rank_1_heap_bases.json"]
