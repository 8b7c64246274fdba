"""The Iris context: one symmetric heap per rank plus everything that hangs off it.

``iris(heap_size)`` must be called collectively by every rank of an initialised
``torch.distributed`` process group (``nccl`` for GPU ranks, ``gloo`` for the CPU backend). The
public surface follows the reference class (iris/host/iris.py:74-1342): tensor factories on the
heap, ``get_heap_bases`` / ``get_device_context``, host and device barriers, ``broadcast``,
logging helpers, and the ``ccl`` / ``ops`` / ``tracing`` namespaces. Added here: ``rma`` (one-sided
operations on tensors from the host, which also run on the CPU backend), ``check()`` (raises when a
kernel recorded a timed-out wait) and process-group sub-contexts.
"""
from __future__ import annotations

import ctypes as C
import os
import weakref

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib
from . import distributed as D
from . import tensors as T
from .heap import SymmetricHeap, _rt
from .logging import DEBUG, ERROR, INFO, WARNING, log_rank
from .platform import get_cu_count, get_device_id_for_rank, is_simulation_env

SYNC_BLOCK_BYTES = (8 + _lib.MAX_RANKS) * 4
_LIVE_CONTEXTS: "weakref.WeakSet" = weakref.WeakSet()


def close_all() -> None:
    """Close every context this process still holds (heaps unbound from their multicast object,
    peer mappings released). For a process that is about to leave after an error: its peers may
    never reach a barrier, so nothing collective happens here."""
    for ctx in list(_LIVE_CONTEXTS):
        try:
            ctx.close()
        except Exception:
            pass


_STATUS_NAMES = {
    1: "a cross-rank barrier wait ran out (a peer never arrived)",
    2: "a wait on a producer flag ran out",
    3: "a wait inside a GEMM pipeline ran out",
    4: "a pointer outside the symmetric heap was translated",
    5: "a spin-lock could not be taken in time",
}


class IrisTimeoutError(RuntimeError):
    """A device-side wait ran out of time; carries the rank and the status code."""

    def __init__(self, rank: int, code: int):
        self.rank, self.code = rank, code
        super().__init__(f"rank {rank}: {_STATUS_NAMES.get(code, 'device status ' + str(code))}")


class Iris:
    """Symmetric-heap context of one rank (see module docstring)."""

    def __init__(self, heap_size: int = 1 << 30, allocator_type: str = "torch"):
        _, self.cur_rank, self.num_ranks = D.init_distributed()
        if self.num_ranks > _lib.MAX_RANKS:
            raise RuntimeError(f"at most {_lib.MAX_RANKS} ranks share a heap")
        use_cuda = torch.cuda.is_available() and os.environ.get("IRIS_BACKEND", "") != "cpu" and allocator_type != "cpu"
        if use_cuda:
            self.gpu_id = get_device_id_for_rank(self.cur_rank, torch.cuda.device_count())
            torch.cuda.set_device(self.gpu_id)
        else:
            self.gpu_id = -1
        self.heap = SymmetricHeap(heap_size, max(self.gpu_id, 0), self.cur_rank, self.num_ranks, allocator_type)
        self.device = self.heap.device
        self.heap_size = heap_size
        if is_simulation_env():
            self._dump_heap_bases()
        # host backend: the shared-memory heap, or (tests) the VMM heap on the host-memory driver stand-in
        self.is_cpu = self.heap.device.type == "cpu"
        self.timeout_ms = int(os.environ.get("IRIS_TIMEOUT_MS", "5000"))
        # IRIS_DEBUG=1: fresh heap memory is poisoned, every host barrier compares the ranks'
        # allocation offsets, and every synchronous collective ends with check()
        self.debug_checks = os.environ.get("IRIS_DEBUG", "0") not in ("", "0")
        env_limit = os.environ.get("IRIS_BARRIER_TIMEOUT_S", "")
        self._barrier_timeout_s = float(env_limit) if env_limit else None
        self._watchdog = None
        # status word + sync block of the context itself (barrier) + per-purpose sync blocks
        self._status = self.heap.allocate(1, torch.int32)
        self._status.zero_()
        self._sync_blocks: dict = {}
        self._group_ctx_cache: dict = {}
        self._ctx_struct = None
        from .tracing import Tracing

        self.tracing = Tracing(self)
        self._device_context = None
        self._build_device_context()
        from ..ccl import CCL
        from .rma import HostRMA

        self.ccl = CCL(self)
        self.rma = HostRMA(self)
        self._ops = None
        self._closed = False
        _LIVE_CONTEXTS.add(self)
        D.distributed_barrier()

    def _dump_heap_bases(self) -> None:
        """Simulation runs (``IRIS_SIMULATION=1``) leave ``<prefix>_rank_<r>_heap_bases.json`` behind
        for tools that replay a captured kernel and need the addresses it saw (prefix from
        ``IRIS_HEAP_BASES_PREFIX``, default ``iris``; reference: iris/host/iris.py:119-134)."""
        import json

        prefix = os.environ.get("IRIS_HEAP_BASES_PREFIX", "iris")
        record = {"rank": self.cur_rank, "num_ranks": self.num_ranks,
                  "heap_bases": [hex(int(b)) for b in self.heap.bases_host()]}
        with open(f"{prefix}_rank_{self.cur_rank}_heap_bases.json", "w") as f:
            json.dump(record, f, indent=2)

    # ------------------------------------------------------------------ logging helpers
    def _log(self, level, message):
        log_rank(level, message, self.cur_rank, self.num_ranks)

    def debug(self, message):
        self._log(DEBUG, message)

    def info(self, message):
        self._log(INFO, message)

    def warning(self, message):
        self._log(WARNING, message)

    def error(self, message):
        self._log(ERROR, message)

    # ------------------------------------------------------------------ namespaces
    @property
    def ops(self):
        """Fused GEMM + collective operations (created on first use)."""
        if self._ops is None:
            from ..ops import OpsNamespace

            self._ops = OpsNamespace(self)
        return self._ops

    # ------------------------------------------------------------------ collective host helpers
    def broadcast(self, value, src: int = 0):
        """Broadcast a scalar, numpy array or tensor from rank ``src`` to all ranks. What the other
        ranks pass as ``value`` is ignored (``None`` is fine): the source's value decides the kind."""
        is_array = isinstance(value, (torch.Tensor, np.ndarray))
        # one object broadcast carries the kind and, for scalars, the value itself
        kind, payload = D.distributed_broadcast_scalar(("tensor", None) if is_array else ("scalar", value), src)
        if kind == "tensor":
            return D.distributed_broadcast_tensor(value, src)
        return payload

    def barrier(self, stream=None, group=None, timeout_s: float | None = None):
        """Host barrier: wait for this rank's GPU work (one stream or the device), then for all ranks.

        With ``timeout_s`` (or ``IRIS_BARRIER_TIMEOUT_S`` in the environment) the ranks meet through
        the rendezvous store instead of a collective, and a rank that does not arrive in time makes
        the others raise ``BarrierTimeoutError`` naming it, instead of waiting for the process
        group's own timeout."""
        if not self.is_cpu:
            if stream is None:
                torch.cuda.synchronize(self.device)
            else:
                stream.synchronize()
        if timeout_s is None:
            timeout_s = self._barrier_timeout_s
        if timeout_s is None:
            D.distributed_barrier(group)
        else:
            members = range(self.num_ranks) if group is None else dist.get_process_group_ranks(group)
            self._store_barrier().wait(members, timeout_s)
        if self.debug_checks:
            self.debug_verify(group)

    def debug_verify(self, group=None) -> None:
        """What ``IRIS_DEBUG=1`` runs after every host barrier and synchronous collective: a failed
        device-side wait raises here rather than at some later ``check()``, and (for barriers of all
        ranks) heaps that have diverged are reported at the first barrier after the divergence."""
        self.check()
        if group is None:
            self.verify_symmetry()

    def device_barrier(self, group=None):
        """Barrier across ranks executed on the GPU, on the current stream, without host
        synchronisation; capturable in a CUDA graph. On the CPU backend it runs on the host."""
        sb = self.sync_block(("device_barrier", self._group_key(group)))
        ctx = self.ctx_struct(group)
        if self.is_cpu:
            bases = (C.c_uint64 * self.num_ranks)(*[int(b) for b in ctx.bases[: ctx.world]])
            rc = _rt().iris_cpu_barrier(ctx.rank, ctx.world, bases, sb.data_ptr(), self.timeout_ms * 1_000_000, self._status.data_ptr())
            if rc != 0:
                self.check()
            return
        _lib.check(self._klib().iris_device_barrier(C.byref(ctx), C.c_void_p(sb.data_ptr()), C.c_void_p(_lib.current_stream_ptr())),
                   "device barrier launch")

    def _store_barrier(self):
        if self._watchdog is None:
            from .watchdog import Heartbeat, StoreBarrier

            self._watchdog = (StoreBarrier(self.cur_rank), Heartbeat(self.cur_rank, self.num_ranks))
        return self._watchdog[0]

    def heartbeat(self) -> None:
        """Tell the other ranks that this one is alive (one small write to the rendezvous store);
        call it once per step."""
        self._store_barrier()
        self._watchdog[1].beat()

    def stale_ranks(self, max_age_s: float) -> list:
        """Ranks that have not called ``heartbeat()`` during the last ``max_age_s`` seconds: ask before
        launching kernels that wait for peers, so that a rank that left between steps is found on
        the host and not by a device-side timeout."""
        self._store_barrier()
        return self._watchdog[1].stale(max_age_s)

    def heap_mark(self) -> int:
        """Current bump offset of the heap; pass it to ``heap_release`` to free everything allocated since."""
        return self.heap.get_offset()

    def heap_release(self, mark: int) -> None:
        """Rewind the heap to ``mark`` (collective: every rank must do the same, and no tensor
        allocated after the mark may be used again). Cached kernel descriptors are dropped."""
        self.barrier()
        self.heap.set_offset(mark)
        self._sync_blocks = {k: v for k, v in self._sync_blocks.items() if self.heap.offset_of(v) < mark}
        # descriptors remembered for repeated calls may point into the released range (workspaces,
        # sync blocks): forget them all, and change the epoch that every cache key carries
        self.ccl._desc_cache.clear()
        self.ccl._fast.clear()
        self.ccl._ws_cache = {k: w for k, w in self.ccl._ws_cache.items()
                              if not any(t is not None and self.heap.offset_of(t) >= mark for t in (w.ring_buffer, w.flags, w.sync_block))}
        self._ctx_epoch = object()
        self._group_ctx_cache.clear()
        def before_mark(w):
            held = [w.sync_block] + list(w.extra.get("scratch", {}).values())
            return all(t is None or t.numel() == 0 or self.heap.offset_of(t) < mark for t in held)

        kept = {k: w for k, w in self.__dict__.get("_ops_workspaces", {}).items() if before_mark(w)}
        self.__dict__["_ops_workspaces"] = kept
        if self.ccl._push_ws is not None and self.heap.offset_of(self.ccl._push_ws[0]) >= mark:
            self.ccl._push_ws = None
        self.barrier()

    def verify_symmetry(self) -> None:
        """Raise if the ranks' heaps have diverged (different allocation sequences): symmetric
        addressing is only valid when every rank allocated the same sizes in the same order."""
        offs = D.distributed_allgather(np.array([self.heap.get_offset()], dtype=np.int64)).flatten().tolist()
        if len(set(offs)) != 1:
            raise RuntimeError(f"symmetric heap offsets differ across ranks: {offs}; every rank must allocate the same "
                               f"tensors in the same order")

    def check(self) -> None:
        """Raise IrisTimeoutError if a kernel recorded a failed wait since the last check."""
        if not self.is_cpu:
            torch.cuda.synchronize(self.device)
        code = int(self._status.item())
        if code != 0:
            self._status.zero_()
            raise IrisTimeoutError(self.cur_rank, code)

    # ------------------------------------------------------------------ tensor factories
    def zeros(self, *size, **kw):
        return T.zeros(self.heap, self.device, size, **kw)

    def ones(self, *size, **kw):
        return T.ones(self.heap, self.device, size, **kw)

    def full(self, size, fill_value, **kw):
        return T.full(self.heap, self.device, size, fill_value, **kw)

    def empty(self, *size, **kw):
        return T.empty(self.heap, self.device, size, **kw)

    def zeros_like(self, input, **kw):
        return T.zeros_like(self.heap, self.device, input, **kw)

    def rand(self, *size, **kw):
        return T.rand(self.heap, self.device, size, **kw)

    def randn(self, *size, **kw):
        return T.randn(self.heap, self.device, size, **kw)

    def uniform(self, size, low=0.0, high=1.0, dtype=torch.float):
        return T.uniform(self.heap, self.device, size, low, high, dtype)

    def randint(self, *args, **kw):
        # torch.randint(high, size) | torch.randint(low, high, size)
        if len(args) == 2:
            low, (high, size) = 0, args
        elif len(args) == 3:
            low, high, size = args
        else:
            raise ValueError("randint(low=0, high, size) takes 2 or 3 positional arguments")
        return T.randint(self.heap, self.device, low, high, size, **kw)

    def arange(self, start=0, end=None, step=1, **kw):
        if end is None:
            start, end = 0, start
        return T.arange(self.heap, self.device, start, end, step, **kw)

    def linspace(self, start, end, steps, **kw):
        return T.linspace(self.heap, self.device, start, end, steps, **kw)

    def as_symmetric(self, tensor: torch.Tensor) -> torch.Tensor:
        return self.heap.as_symmetric(tensor)

    def is_symmetric(self, tensor: torch.Tensor) -> bool:
        return self.heap.is_symmetric(tensor)

    # ------------------------------------------------------------------ device-facing state
    def get_heap_bases(self) -> torch.Tensor:
        """int64[num_ranks] on the device: address of every rank's heap in THIS process."""
        return self.heap.get_heap_bases()

    def get_device_context(self) -> torch.Tensor:
        """int64 tensor ``[rank, world, bases..., trace block]`` for ``DeviceContext::initialize``."""
        return self._device_context

    def _build_device_context(self) -> None:
        words = [self.cur_rank, self.num_ranks] + [int(b) for b in self.heap.bases_host().view(np.int64)]
        words += self.tracing.context_words()
        self._device_context = torch.tensor(words, dtype=torch.int64, device=self.device)
        self._ctx_struct = None
        self._group_ctx_cache.clear()
        self._ctx_epoch = object()    # changes whenever cached kernel descriptors become stale

    def _group_key(self, group):
        if group is None:
            return None
        return tuple(dist.get_process_group_ranks(group))

    def ctx_struct(self, group=None) -> _lib.IrisCtx:
        """The kernel-parameter form of the context (``IrisCtx``), optionally restricted to a
        process group: ranks are renumbered 0..n-1 inside the group and only their bases are listed."""
        key = self._group_key(group)
        cached = self._group_ctx_cache.get(key)
        if cached is not None:
            return cached
        rank_in_group, _, world, start, stride = D.extract_group_info(group, self.cur_rank, self.num_ranks)
        c = _lib.IrisCtx()
        c.rank, c.world = rank_in_group, world
        c.heap_size = self.heap_size
        c.mc_base = self.heap.mc_base if group is None else 0
        c.status = self._status.data_ptr()
        c.timeout_ns = self.timeout_ms * 1_000_000
        host_bases = self.heap.bases_host()
        for i in range(world):
            c.bases[i] = int(host_bases[start + i * stride])
        tw = self.tracing.context_words()
        c.trace_enabled, c.trace_max_events = int(tw[0]), int(tw[1])
        for i in range(15):
            c.trace_ptrs[i] = int(tw[2 + i]) or None
        self._group_ctx_cache[key] = c
        return c

    def sync_block(self, key) -> torch.Tensor:
        """A zeroed SyncBlock on the heap, one per purpose; every rank must request the same keys
        in the same order (they are heap allocations)."""
        sb = self._sync_blocks.get(key)
        if sb is None:
            sb = self.heap.allocate(SYNC_BLOCK_BYTES // 4, torch.int32)
            sb.zero_()
            self._sync_blocks[key] = sb
            self.barrier()
        return sb

    def _klib(self):
        lib = _lib.kernels()
        if not getattr(lib, "_iris_misc_typed", False):
            vp, i32 = C.c_void_p, C.c_int
            lib.iris_device_barrier.argtypes = [C.POINTER(_lib.IrisCtx), vp, vp]
            lib.iris_device_barrier.restype = i32
            lib.iris_wait_flag.argtypes = [vp, C.c_int32, C.c_uint64, vp, vp]
            lib.iris_wait_flag.restype = i32
            lib.iris_set_flag.argtypes = [C.POINTER(_lib.IrisCtx), vp, C.c_int32, i32, vp]
            lib.iris_set_flag.restype = i32
            lib._iris_misc_typed = True
        return lib

    # ------------------------------------------------------------------ queries
    def get_device(self) -> torch.device:
        return self.device

    def get_cu_count(self) -> int:
        """Number of SMs of this rank's GPU (0 on the CPU backend)."""
        return 0 if self.is_cpu else get_cu_count(self.gpu_id)

    def get_device_id(self) -> int:
        return self.gpu_id

    def get_rank(self) -> int:
        return self.cur_rank

    def get_num_ranks(self) -> int:
        return self.num_ranks

    def has_multicast(self) -> bool:
        """True when the heap is bound to an NVLS multicast object (multimem paths are usable)."""
        return self.heap.mc_base != 0

    def wait_flag(self, flag: torch.Tensor, target: int, timeout_ms: int = 1000) -> bool:
        """Wait on the device (or on the host for the CPU backend) until ``flag[0] >= target``;
        returns False when ``timeout_ms`` passed first. The context stays usable either way."""
        if self.is_cpu:
            return _rt().iris_cpu_wait_flag(flag.data_ptr(), int(target), int(timeout_ms) * 1_000_000) == 0
        res = torch.zeros(1, dtype=torch.int32, device=self.device)
        _lib.check(self._klib().iris_wait_flag(C.c_void_p(flag.data_ptr()), int(target), int(timeout_ms) * 1_000_000,
                                               C.c_void_p(res.data_ptr()), C.c_void_p(_lib.current_stream_ptr())), "wait_flag launch")
        return int(res.item()) == 0

    def close(self) -> None:
        """Unmap and free this rank's heap and its mappings of the peers' heaps. Heap tensors must not be
        used afterwards; call it on every rank (peers may still be reading until the barrier before it)."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        _LIVE_CONTEXTS.discard(self)
        if not self.is_cpu:
            try:
                torch.cuda.synchronize(self.device)     # none of this rank's kernels may still touch the mappings
            except Exception:
                pass
        self.heap.close()

    def __enter__(self) -> "Iris":
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        # leave together when the block ended normally; after an exception only release local resources,
        # because the other ranks may never reach a barrier
        if exc_type is None:
            self.barrier()
        self.close()
        return False


def iris(heap_size: int = 1 << 30, allocator_type: str = "torch") -> Iris:
    """Create the context (collective). ``heap_size`` is bytes per rank."""
    return Iris(heap_size, allocator_type)
