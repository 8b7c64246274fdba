"""Failure detection without a GPU fault: failures are produced on the host (a rank that skips a
barrier, a message nobody sends, a flag nothing sets, a heap that is too small, ranks that
allocate differently) among gloo ranks on the CPU backend; every wait is bounded and surfaces as
an exception or a status, never as a hang."""
import time

import pytest
import torch

from helpers import run_ranks


def _missing_rank(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    ctx.timeout_ms = 300
    ctx.device_barrier()          # everybody takes part: fine
    if rank == 0:
        # rank 0 skips the second barrier: the others' bounded wait must run out and raise
        time.sleep(1.0)
        return
    t0 = time.time()
    with pytest.raises(iris.IrisTimeoutError) as ei:
        ctx.device_barrier()
    assert ei.value.rank == rank and ei.value.code == 1
    assert time.time() - t0 < 5.0
    # the context is still usable afterwards
    t = ctx.zeros(4, dtype=torch.int32)
    ctx.rma.atomic_add(t, 2, to_rank=rank)
    assert torch.all(t == 2)


def test_barrier_times_out_when_a_rank_never_arrives():
    codes, errors = run_ranks(_missing_rank, 3, expect_failures=True, timeout=120)
    assert not errors, errors
    assert all(c == 0 for c in codes)


def _unset_flag(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    flag = ctx.zeros(1, dtype=torch.int32)
    ctx.barrier()
    t0 = time.time()
    assert ctx.wait_flag(flag, 1, timeout_ms=100) is False
    assert 0.09 < time.time() - t0 < 3.0
    ctx.barrier()
    # now a peer sets it: producer/consumer across processes through the shared heap
    peer = (rank + 1) % world
    ctx.rma.atomic_xchg(flag, 1, to_rank=peer, sem="release", scope="sys")
    assert ctx.wait_flag(flag, 1, timeout_ms=5000) is True
    ctx.barrier()


def test_wait_on_a_flag_nothing_sets_returns_false():
    run_ranks(_unset_flag, 2)


def _fd_timeout(rank, world):
    from iris_b200.host.heap import FdMesh

    mesh = FdMesh(rank, world)
    with pytest.raises(TimeoutError):
        mesh.recv(timeout_ms=200)        # nobody sent anything
    mesh.close()


def test_fd_mesh_receive_is_bounded():
    run_ranks(_fd_timeout, 2)


def _asymmetric(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    ctx.verify_symmetry()
    ctx.zeros(100 if rank == 0 else 5000, dtype=torch.float32)   # ranks diverge
    with pytest.raises(RuntimeError, match="offsets differ"):
        ctx.verify_symmetry()
    ctx.barrier()


def test_divergent_allocation_is_detected():
    run_ranks(_asymmetric, 2)


def _raising_rank(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 24)
    ctx.device_barrier()          # allocates the barrier's sync block while everybody is alive
    ctx.barrier()
    if rank == 1:
        raise ValueError("injected failure on rank 1")
    ctx.timeout_ms = 300
    with pytest.raises(iris.IrisTimeoutError):
        ctx.device_barrier()


def test_a_rank_that_raises_is_reported_and_the_rest_time_out():
    codes, errors = run_ranks(_raising_rank, 2, expect_failures=True, timeout=120)
    assert codes[0] == 0 and codes[1] != 0
    assert len(errors) == 1 and errors[0][0] == 1 and "injected failure" in errors[0][1]


def _host_barrier_names_missing_ranks(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 22)
    for _ in range(4):                                   # rounds are counted, old keys are dropped
        ctx.barrier(timeout_s=20.0)
    if rank in (1, 3):
        time.sleep(2.5)                                  # these two are late for the next round
        return
    t0 = time.time()
    with pytest.raises(iris.BarrierTimeoutError) as ei:
        ctx.barrier(timeout_s=0.5)
    assert ei.value.missing == [1, 3] and ei.value.rank == rank and ei.value.round == 5
    assert "did not arrive: [1, 3]" in str(ei.value) and time.time() - t0 < 2.0
    # the context is still usable: memory operations do not depend on the lost ranks
    t = ctx.zeros(4, dtype=torch.int32)
    ctx.rma.atomic_add(t, 1, to_rank=rank)
    assert torch.all(t == 1)


def test_host_barrier_with_a_limit_names_the_missing_ranks():
    codes, errors = run_ranks(_host_barrier_names_missing_ranks, 4, expect_failures=True, timeout=120)
    assert not errors, errors
    assert all(c == 0 for c in codes)


def _group_barrier_and_env(rank, world):
    import torch.distributed as dist

    import iris_b200 as iris

    ctx = iris.iris(1 << 22)
    assert ctx._barrier_timeout_s == 15.0                # from the environment: every host barrier is bounded
    pairs = [[0, 1], [2, 3]]
    groups = [dist.new_group(p) for p in pairs]
    mine = groups[0] if rank < 2 else groups[1]
    if rank < 2:
        for _ in range(3):
            ctx.barrier(group=mine)                      # only the pair takes part; the other pair does nothing meanwhile
    ctx.barrier()
    # collectives end with the same bounded barrier
    inp, out = ctx.full((4, 8), float(rank + 1)), ctx.zeros((4, 8))
    ctx.ccl.all_reduce(out, inp)
    assert torch.all(out == 10)
    ctx.barrier()


def test_bounded_host_barrier_from_the_environment_and_in_groups():
    run_ranks(_group_barrier_and_env, 4, env={"IRIS_BARRIER_TIMEOUT_S": "15"})


def _heartbeats(rank, world):
    import iris_b200 as iris

    ctx = iris.iris(1 << 22)
    assert sorted(ctx.stale_ranks(60.0)) == [r for r in range(world) if r != rank]      # nobody has beaten yet
    ctx.barrier()
    ctx.heartbeat()
    ctx.barrier()
    assert ctx.stale_ranks(60.0) == []
    ctx.barrier()
    # rank 2 leaves between steps; the others keep beating and find out on the host
    if rank == 2:
        return
    for _ in range(3):
        time.sleep(0.4)
        ctx.heartbeat()
    assert ctx.stale_ranks(1.0) == [2]
    assert ctx.stale_ranks(60.0) == []                   # a generous limit still accepts its last beat


def test_heartbeats_reveal_a_rank_that_left_between_steps():
    codes, errors = run_ranks(_heartbeats, 3, expect_failures=True, timeout=120)
    assert not errors, errors
    assert all(c == 0 for c in codes)


def test_store_protocols_against_a_plain_dictionary_store():
    """The two protocols only need set / get / check / wait / delete_key: a dictionary stands in."""
    from iris_b200.host.watchdog import BarrierTimeoutError, Heartbeat, StoreBarrier

    class DictStore:
        def __init__(self):
            self.d = {}

        def set(self, k, v):
            self.d[k] = v.encode() if isinstance(v, str) else v

        def get(self, k):
            return self.d[k]

        def check(self, keys):
            return all(k in self.d for k in keys)

        def wait(self, keys, timeout):
            if not self.check(keys):
                raise RuntimeError("timeout")

        def delete_key(self, k):
            return self.d.pop(k, None) is not None

    store = DictStore()
    b0, b1 = StoreBarrier(0, store), StoreBarrier(1, store)
    with pytest.raises(BarrierTimeoutError) as ei:
        b0.wait([0, 1], 0.01)                            # rank 1 has not arrived
    assert ei.value.missing == [1]
    assert b1.wait([0, 1], 0.01) == 1                    # rank 0's key of round 1 is there: passes
    for n in range(2, 6):
        store.set(f"iris/barrier/0-1/{n}/1", "1")        # rank 1 arrives first in the later rounds
        assert b0.wait([0, 1], 0.01) == n
    assert "iris/barrier/0-1/1/0" not in store.d and "iris/barrier/0-1/5/0" in store.d       # old rounds are cleaned up
    with pytest.raises(ValueError):
        b0.wait([1, 2], 0.01)
    hb0, hb1 = Heartbeat(0, 3, store), Heartbeat(1, 3, store)
    hb1.beat(now=100.0)
    assert hb0.last(1) == 100.0 and hb0.last(2) is None
    assert hb0.stale(5.0, now=103.0) == [2] and hb0.stale(5.0, now=106.0) == [1, 2] and hb0.stale(5.0, ranks=[1], now=103.0) == []


def test_heap_creation_cleans_up_after_an_injected_driver_failure():
    """Fault injection on the host: the driver stand-in is told to fail its k-th memory call. Whatever
    step of the VMM heap's construction that hits (reserve, create, map, set access), the constructor
    raises with the driver's message, nothing stays allocated, reserved or mapped, and the next
    attempt succeeds. (No GPU: the stand-in keeps allocations in host memory.)"""
    import torch.distributed as dist

    from helpers import free_port
    from iris_b200.host.heap import KIND_VMM, SymmetricHeap, _rt

    import os

    rt = _rt()
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(free_port()), "IRIS_FAKE_DRIVER_DEVICES": "2"})
    created_pg = not dist.is_initialized()
    if created_pg:
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        rt.iris_rt_install_fake_driver(2)
        baseline = rt.iris_rt_fake_live_objects()
        failed_steps = 0
        for k in range(1, 8):
            rt.iris_rt_fake_fail_after(k)
            try:
                heap = SymmetricHeap(4 << 20, 0, 0, 1, allocator_type="vmem", enable_multicast=False)
            except RuntimeError as e:
                failed_steps += 1
                assert "out of memory" in str(e) or "fake driver error" in str(e) or "cuMem" in str(e), str(e)
                assert rt.iris_rt_fake_live_objects() == baseline, f"step {k} leaked driver objects"
                continue
            finally:
                rt.iris_rt_fake_fail_after(0)
            # the failure point lies beyond the calls a construction makes: it went through
            assert heap.kind == KIND_VMM
            t = heap.allocate(16, torch.int32)
            t.fill_(k)
            assert int(t.sum()) == 16 * k
            del t
            heap.close()
            assert rt.iris_rt_fake_live_objects() == baseline
        assert failed_steps >= 3          # reserve, create, map and set-access were each hit at least once in total
        # a clean run after all the failures
        heap = SymmetricHeap(4 << 20, 0, 0, 1, allocator_type="vmem", enable_multicast=False)
        assert rt.iris_rt_fake_live_objects() > baseline
        heap.close()
        assert rt.iris_rt_fake_live_objects() == baseline
    finally:
        rt.iris_rt_fake_fail_after(0)
        rt.iris_rt_install_fake_driver(0)
        os.environ.pop("IRIS_FAKE_DRIVER_DEVICES", None)
        if created_pg:
            dist.destroy_process_group()


def _peer_import_fails(rank, world, fail_at=6):
    from iris_b200.host.heap import KIND_VMM, SymmetricHeap, _rt

    rt = _rt()
    rt.iris_rt_install_fake_driver(2)
    baseline = rt.iris_rt_fake_live_objects()
    if rank == 1:
        rt.iris_rt_fake_fail_after(fail_at)      # 6: its own region comes up (5 calls), importing the peer's handle fails; 1: its own region fails
    with pytest.raises(RuntimeError, match="could not create a symmetric heap on every rank"):
        SymmetricHeap(4 << 20, 0, rank, world, allocator_type="vmem", enable_multicast=False)
    rt.iris_rt_fake_fail_after(0)
    # the rank whose calls all succeeded gives its region up as well: nobody keeps half a heap
    assert rt.iris_rt_fake_live_objects() == baseline
    heap = SymmetricHeap(4 << 20, 0, rank, world, allocator_type="vmem", enable_multicast=False)
    assert heap.kind == KIND_VMM
    t = heap.allocate(8, torch.int32)
    t.fill_(rank + 1)
    import torch.distributed as dist

    dist.barrier()
    assert torch.all(heap.peer_view(t, 1 - rank) == 2 - rank)
    dist.barrier()
    del t
    heap.close()


def test_a_failed_peer_import_fails_the_heap_on_every_rank():
    run_ranks(_peer_import_fails, 2, env={"IRIS_FAKE_DRIVER_DEVICES": "2"}, timeout=120)


def test_a_rank_that_cannot_create_its_region_fails_the_heap_on_every_rank():
    """The ranks vote after creating and exporting, before any handle is exchanged: the rank whose region came
    up does not wait for a descriptor that will never arrive, and every rank leaves the backend together."""
    run_ranks(_peer_import_fails, 2, args=(1,), env={"IRIS_FAKE_DRIVER_DEVICES": "2"}, timeout=120)
