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
