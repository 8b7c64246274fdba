"""Launch helpers for multi-process tests.

CPU tests run `world` gloo ranks as child processes of the test (spawn); GPU tests run one child
per GPU with the nccl backend. The child entry point is a module-level function
``fn(rank, world, *args)``; an exception in any rank fails the test with that rank's traceback.
"""
from __future__ import annotations

import datetime
import os
import socket
import sys
import time
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, backend, fn, args, errq, env):
    reported = False
    try:
        os.environ.update(env)
        os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                           "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
        if ROOT not in sys.path:
            sys.path.insert(0, ROOT)
        import torch.distributed as dist

        if backend == "nccl":
            torch.cuda.set_device(rank)
            # a collective that a failed peer never joins ends with an error after this long, not after NCCL's ten minutes
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                    timeout=datetime.timedelta(seconds=float(os.environ.get("IRIS_TEST_PG_TIMEOUT_S", "180"))))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
        try:
            fn(rank, world, *args)
        except BaseException:
            # report first: the clean-up below can block when the peers are in a different state
            errq.put((rank, traceback.format_exc()))
            reported = True
            raise
        finally:
            # Leave in order: unbind and unmap every heap this process created (a heap may be bound
            # to an NVLink multicast object, which must not outlive an abrupt exit), then the group.
            try:
                from iris_b200.host.iris import close_all

                close_all()
            except Exception:
                pass
            if not reported:
                try:
                    dist.destroy_process_group()
                except Exception:
                    pass
    except BaseException:
        if not reported:
            errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world: int, args=(), backend: str = "gloo", timeout: float = 300.0, env: dict | None = None,
              expect_failures: bool = False):
    """Run ``fn(rank, world, *args)`` on ``world`` ranks; raise with the first failing traceback."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    env = dict(env or {})
    if backend == "gloo":
        env.setdefault("IRIS_BACKEND", "cpu")
    else:
        # GPU ranks leave on their own: a host barrier that a failed peer never joins raises
        # BarrierTimeoutError instead of blocking (device-side waits are bounded already).
        env.setdefault("IRIS_BARRIER_TIMEOUT_S", os.environ.get("IRIS_BARRIER_TIMEOUT_S", "60"))
    # A GPU rank whose heap may be bound to a multicast object is never killed from here: ending it
    # in the middle of a kernel has left NVLink faults on its peers' GPUs. Only CPU ranks, or GPU
    # ranks started with NVLS off, get the last-resort stop.
    nvls_off = env.get("IRIS_NVLS", os.environ.get("IRIS_NVLS", "1")) == "0"
    may_kill = backend == "gloo" or nvls_off
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, errq, env)) for r in range(world)]
    for p in procs:
        p.start()
    # Wait for all ranks, but not for ever for the peers of a rank that has failed: they are usually
    # stuck in a barrier with it, so they get a short grace period and are then stopped.
    deadline, failed_at, grace = time.time() + timeout, None, 20.0
    while any(p.is_alive() for p in procs):
        now = time.time()
        if failed_at is None and any(p.exitcode not in (None, 0) for p in procs):
            failed_at = now
        if may_kill and (now > deadline or (failed_at is not None and now - failed_at > grace and not expect_failures)):
            break
        if not may_kill and now > deadline + 180.0:      # their own barrier / process-group limits have long passed
            break
        time.sleep(0.05)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        if may_kill:
            p.kill()  # the exact child processes started above
            p.join()
    if failed_at is not None and not expect_failures:
        hung = []           # their peer failed first: the failure below is the one to report
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    codes = [p.exitcode for p in procs]
    if expect_failures:
        return codes, errors
    if hung:
        raise AssertionError(f"{len(hung)} rank(s) still running after {timeout}s")
    if errors:
        # a rank whose collective broke because a peer went away is a consequence: report the cause first
        errors.sort(key=lambda e: any(w in e[1] for w in ("Connection closed", "Connection reset", "ProcessGroup", "NCCL error")))
        rank, tb = errors[0]
        raise AssertionError(f"rank {rank} failed:\n{tb}")
    if any(c != 0 for c in codes):
        raise AssertionError(f"rank exit codes {codes}")
    return codes, errors
