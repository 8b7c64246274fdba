"""Host-side liveness: a barrier that names the ranks that did not arrive, and heartbeats.

``torch.distributed.barrier`` waits for as long as the process group's timeout (minutes) and then
fails without saying who was missing. The reference has nothing beyond it (its device barrier traps
after 1e9 spins, iris/host/distributed/helpers.py:342-381; its socket mesh has a 10 s connect
deadline, fd_passing.py:108-120). Here the rendezvous store that every process group already has
carries two small protocols:

``StoreBarrier``   each member writes ``barrier/<members>/<round>/<rank>`` and waits, with a limit, for
                   the keys of all members; when the limit passes it looks which keys exist and raises
                   ``BarrierTimeoutError`` listing the missing ranks. Rounds are counted per member
                   set, old keys are deleted two rounds later.
``Heartbeat``      ``beat()`` stores the wall-clock time under ``heartbeat/<rank>``; ``stale(max_age)``
                   returns the ranks whose last beat is older (or absent). A training or serving loop
                   beats once per step and asks before it launches kernels that wait for peers, so a
                   rank that left between steps is noticed on the host instead of in a device-side
                   timeout.

Both only use ``set`` / ``get`` / ``check`` / ``wait`` / ``delete_key`` of the c10d store, so they work
the same under gloo and nccl and touch no GPU.
"""
from __future__ import annotations

import time
from datetime import timedelta

import torch.distributed as dist


class BarrierTimeoutError(RuntimeError):
    """Some ranks did not reach a host barrier in time; ``missing`` lists them (global ranks)."""

    def __init__(self, rank: int, missing: list, timeout_s: float, round_no: int):
        self.rank, self.missing, self.timeout_s, self.round = rank, list(missing), timeout_s, round_no
        super().__init__(f"rank {rank}: host barrier round {round_no} timed out after {timeout_s:g} s; "
                         f"ranks that did not arrive: {self.missing}")


def _default_store():
    store = dist.distributed_c10d._get_default_store()
    if store is None:
        raise RuntimeError("the default process group has no store")
    return store


class StoreBarrier:
    def __init__(self, rank: int, store=None, prefix: str = "iris"):
        self.rank = rank
        self.store = store if store is not None else _default_store()
        self.prefix = prefix
        self._rounds: dict = {}

    def _key(self, tag: str, round_no: int, rank: int) -> str:
        return f"{self.prefix}/barrier/{tag}/{round_no}/{rank}"

    def wait(self, members, timeout_s: float) -> int:
        """Barrier among ``members`` (global ranks, this rank included). Returns the round number."""
        members = sorted(int(m) for m in members)
        if self.rank not in members:
            raise ValueError(f"rank {self.rank} is not one of {members}")
        tag = "-".join(map(str, members))
        n = self._rounds.get(tag, 0) + 1
        self._rounds[tag] = n
        self.store.set(self._key(tag, n, self.rank), "1")
        keys = [self._key(tag, n, m) for m in members]
        try:
            self.store.wait(keys, timedelta(seconds=float(timeout_s)))
        except Exception:
            missing = [m for m, k in zip(members, keys) if not self.store.check([k])]
            if missing:
                raise BarrierTimeoutError(self.rank, missing, timeout_s, n) from None
            # everybody arrived between the timeout and the check: the barrier holds
        if n > 2:
            try:
                self.store.delete_key(self._key(tag, n - 2, self.rank))
            except Exception:
                pass              # a store without delete support only grows by a few bytes per round
        return n


class Heartbeat:
    def __init__(self, rank: int, world: int, store=None, prefix: str = "iris"):
        self.rank, self.world = rank, world
        self.store = store if store is not None else _default_store()
        self.prefix = prefix

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/heartbeat/{rank}"

    def beat(self, now: float | None = None) -> None:
        self.store.set(self._key(self.rank), repr(time.time() if now is None else float(now)))

    def last(self, rank: int) -> float | None:
        """Wall-clock time of ``rank``'s last beat, ``None`` if it never beat."""
        key = self._key(rank)
        if not self.store.check([key]):
            return None
        try:
            return float(self.store.get(key).decode())
        except (ValueError, RuntimeError):
            return None

    def stale(self, max_age_s: float, ranks=None, now: float | None = None) -> list:
        """Ranks (default: all others) with no beat during the last ``max_age_s`` seconds."""
        now = time.time() if now is None else float(now)
        out = []
        for r in (range(self.world) if ranks is None else ranks):
            if r == self.rank:
                continue
            t = self.last(r)
            if t is None or now - t > max_age_s:
                out.append(r)
        return out
