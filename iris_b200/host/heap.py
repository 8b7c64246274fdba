"""Python face of the native symmetric heap (csrc/runtime/symmetric_heap.cpp).

One region per rank is created, exported and mapped into every peer ONCE, at construction. After
that ``allocate`` is a local bump-pointer operation: because every rank performs the same sequence
of allocations, equal offsets name the same object on every rank, which is all the device-side
translation needs. (The reference re-exchanges handles after every allocation,
iris/host/memory/symmetric_heap.py:95-130.)

Backends (``allocator_type`` / env ``IRIS_ALLOCATOR``):

``"torch"``  the default name of the reference; here: one pool backed by CUDA VMM when the driver
             can export POSIX handles, else by ``cuMemAlloc`` + CUDA IPC.
``"vmem"``   CUDA VMM only (error when unavailable); required for the NVLS multicast window.
``"ipc"``    ``cuMemAlloc`` + CUDA IPC only.
``"cpu"``    memfd shared memory between processes of one host (no GPU); chosen automatically when
             the process group's backend is gloo and CUDA is not available.
"""
from __future__ import annotations

import ctypes as C
import os
import tempfile
import uuid

import numpy as np
import torch
import torch.distributed as dist

from .. import _lib
from . import distributed as D
from .logging import logger
from .tensor_utils import tensor_from_ptr

KIND_VMM, KIND_IPC, KIND_CPU = 0, 1, 2
_ERRLEN = 512
_TAG_HEAP, _TAG_MC = 1, 2


def _rt():
    rt = _lib.runtime()
    if getattr(rt, "_iris_typed", False):
        return rt
    u64, i64, i32, vp, cp = C.c_uint64, C.c_int64, C.c_int, C.c_void_p, C.c_char_p
    sig = {
        "iris_rt_cuda_ok": (i32, [cp, i32]),
        "iris_rt_device_count": (i32, []),
        "iris_rt_device_attribute": (i32, [i32, i32]),
        "iris_rt_device_name": (i32, [i32, cp, i32]),
        "iris_rt_set_device": (i32, [i32]),
        "iris_rt_current_device": (i32, []),
        "iris_rt_can_access_peer": (i32, [i32, i32]),
        "iris_rt_p2p_attribute": (i32, [i32, i32, i32]),
        "iris_rt_address_range": (i32, [u64, C.POINTER(u64), C.POINTER(u64)]),
        "iris_rt_ipc_get_handle": (i32, [u64, cp]),
        "iris_rt_ipc_open_handle": (i32, [cp, C.POINTER(u64)]),
        "iris_rt_ipc_close_handle": (i32, [u64]),
        "iris_heap_create": (vp, [u64, i32, i32, i32, i32, i32, cp, i32]),
        "iris_heap_base": (u64, [vp]),
        "iris_heap_size": (u64, [vp]),
        "iris_heap_mapped_size": (u64, [vp]),
        "iris_heap_offset": (u64, [vp]),
        "iris_heap_set_offset": (None, [vp, u64]),
        "iris_heap_peer_base": (u64, [vp, i32]),
        "iris_heap_mc_base": (u64, [vp]),
        "iris_heap_kind": (i32, [vp]),
        "iris_heap_alloc": (i64, [vp, u64, u64]),
        "iris_heap_export_fd": (i32, [vp, cp, i32]),
        "iris_heap_export_blob": (i32, [vp, cp, cp, i32]),
        "iris_heap_import_fd": (i32, [vp, i32, i32, cp, i32]),
        "iris_heap_import_blob": (i32, [vp, i32, cp, cp, i32]),
        "iris_heap_mc_supported": (i32, [i32]),
        "iris_heap_mc_create": (i32, [vp, cp, i32]),
        "iris_heap_mc_attach": (i32, [vp, i32, i32, cp, i32]),
        "iris_heap_mc_bind": (i32, [vp, cp, i32]),
        "iris_heap_destroy": (i32, [vp]),
        "iris_heap_set_next_reserve": (None, [u64]),
        "iris_heap_grow": (i32, [vp, u64, cp, i32]),
        "iris_heap_import_external": (i32, [vp, u64, C.POINTER(C.c_uint64), cp, i32]),
        "iris_heap_num_segments": (i32, [vp]),
        "iris_heap_segment_offset": (u64, [vp, i32]),
        "iris_heap_segment_size": (u64, [vp, i32]),
        "iris_heap_reserved": (u64, [vp]),
        "iris_heap_segment_export_fd": (i32, [vp, i32, cp, i32]),
        "iris_heap_segment_import_fd": (i32, [vp, i32, i32, u64, u64, cp, i32]),
        "iris_fdmesh_create": (vp, [cp, cp, i32]),
        "iris_fdmesh_send": (i32, [vp, cp, i32, i32, i32, u64, cp, i32]),
        "iris_fdmesh_recv": (i32, [vp, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(u64), cp, i32]),
        "iris_fdmesh_destroy": (None, [vp]),
        "iris_close_fd": (None, [i32]),
        "iris_rt_install_fake_driver": (i32, [i32]),
        "iris_rt_fake_fail_after": (None, [i32]),
        "iris_rt_fake_live_objects": (i32, []),
        "iris_rt_driver_version": (i32, [C.POINTER(i32)]),
        "iris_rt_error_string": (i32, [i32, cp, i32]),
        "iris_rt_malloc": (i32, [i32, u64, C.POINTER(u64)]),
        "iris_rt_free": (i32, [u64]),
        "iris_rt_mem_granularity": (i32, [i32, i32, i32, C.POINTER(u64)]),
        "iris_rt_mem_create": (i32, [u64, i32, i32, C.POINTER(u64)]),
        "iris_rt_mem_release": (i32, [u64]),
        "iris_rt_mem_address_reserve": (i32, [u64, u64, u64, C.POINTER(u64)]),
        "iris_rt_mem_address_free": (i32, [u64, u64]),
        "iris_rt_mem_map": (i32, [u64, u64, u64, u64]),
        "iris_rt_mem_unmap": (i32, [u64, u64]),
        "iris_rt_mem_set_access": (i32, [u64, u64, C.POINTER(i32), i32]),
        "iris_rt_mem_export_fd": (i32, [u64, C.POINTER(i32)]),
        "iris_rt_mem_import_fd": (i32, [i32, C.POINTER(u64)]),
        "iris_rt_mem_retain_handle": (i32, [u64, C.POINTER(u64)]),
        "iris_cpu_rma": (i32, [i32, i32, i32, u64, u64, u64, C.c_double, i64, i64, u64, i32, i32, i32, C.POINTER(u64)]),
        "iris_cpu_wait_flag": (i32, [u64, C.c_int32, u64]),
        "iris_cpu_barrier": (i32, [i32, i32, C.POINTER(u64), u64, u64, u64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(rt, name)
        fn.restype = res
        fn.argtypes = args
    rt._iris_typed = True
    return rt


class FdMesh:
    """AF_UNIX datagram mesh that passes file descriptors between the ranks of one host."""

    def __init__(self, rank: int, world: int, group=None):
        self.rank, self.world = rank, world
        rt = _rt()
        self.path = os.path.join(tempfile.gettempdir(), f"iris-b200-{os.getpid()}-{rank}-{uuid.uuid4().hex[:8]}.sock")
        err = C.create_string_buffer(_ERRLEN)
        self.handle = rt.iris_fdmesh_create(self.path.encode(), err, _ERRLEN)
        if not self.handle:
            raise RuntimeError(f"fd mesh: {err.value.decode()}")
        self.paths = D.distributed_allgather_object(self.path, group)
        dist.barrier(group=group)

    def send(self, peer: int, fd: int, tag: int, payload: int = 0) -> None:
        err = C.create_string_buffer(_ERRLEN)
        if _rt().iris_fdmesh_send(self.handle, self.paths[peer].encode(), fd, self.rank, tag, payload, err, _ERRLEN) != 0:
            raise RuntimeError(f"fd mesh send to rank {peer}: {err.value.decode()}")

    def recv(self, timeout_ms: int = 30000):
        fd, src, tag, payload = C.c_int(-1), C.c_int(-1), C.c_int(0), C.c_uint64(0)
        err = C.create_string_buffer(_ERRLEN)
        rc = _rt().iris_fdmesh_recv(self.handle, timeout_ms, C.byref(fd), C.byref(src), C.byref(tag), C.byref(payload), err, _ERRLEN)
        if rc == -2:
            raise TimeoutError(f"fd mesh: {err.value.decode()}")
        if rc != 0:
            raise RuntimeError(f"fd mesh recv: {err.value.decode()}")
        return fd.value, src.value, tag.value, payload.value

    def close(self) -> None:
        if self.handle:
            _rt().iris_fdmesh_destroy(self.handle)
            self.handle = None


class SymmetricHeap:
    """A symmetric heap of ``heap_size`` bytes per rank mapped into every rank of ``group``."""

    def __init__(self, heap_size: int, device_id: int, cur_rank: int, num_ranks: int, allocator_type: str = "torch",
                 group=None, enable_multicast: bool | None = None):
        self.heap_size = int(heap_size)
        self.device_id = device_id
        self.cur_rank = cur_rank
        self.num_ranks = num_ranks
        self.group = group
        self._handle = None
        self._mesh = None
        self.poison = os.environ.get("IRIS_DEBUG", "0") not in ("", "0")
        rt = _rt()
        allocator_type = os.environ.get("IRIS_ALLOCATOR", allocator_type)
        cuda = torch.cuda.is_available() and os.environ.get("IRIS_BACKEND", "") != "cpu"
        # Tests without a GPU: IRIS_FAKE_DRIVER_DEVICES=n routes the native runtime to a host-memory
        # stand-in for the driver's memory API, so that the VMM path below (create, export, pass the
        # descriptor, import, map) runs for real on shared host memory. Heap only: no kernels.
        fake = int(os.environ.get("IRIS_FAKE_DRIVER_DEVICES", "0") or 0) if not cuda else 0
        if fake and allocator_type in ("torch", "vmem"):
            rt.iris_rt_install_fake_driver(fake)
            self.device_id = device_id = cur_rank % fake
            kinds = [KIND_VMM]
        elif allocator_type == "cpu" or not cuda:
            kinds = [KIND_CPU]
        elif allocator_type == "ipc":
            kinds = [KIND_IPC]
        elif allocator_type == "vmem":
            kinds = [KIND_VMM]
        elif allocator_type == "torch":
            kinds = [KIND_VMM, KIND_IPC]
        else:
            raise ValueError(f"unknown allocator_type {allocator_type!r} (torch, vmem, ipc, cpu)")
        self.allocator_type = allocator_type
        self.device = torch.device("cpu") if (kinds == [KIND_CPU] or fake) else torch.device("cuda", device_id)
        # allocator_type="vmem" (the reference's VMemAllocator, allocators/vmem_allocator.py:37-344): address
        # space for the whole heap is reserved, physical memory is mapped on demand (first IRIS_VMEM_INITIAL
        # bytes, default 64 MiB; later segments as allocations need them) and an external allocation can be
        # mapped in without a copy. Such a heap is not bound to a multicast object.
        self.reserve = 0
        if allocator_type == "vmem" and kinds == [KIND_VMM]:
            self.reserve = self.heap_size
            initial = int(os.environ.get("IRIS_VMEM_INITIAL", str(64 << 20)))
            self._initial_size = max(min(self.heap_size, initial), 1 << 20)
            if enable_multicast is None:
                enable_multicast = False

        last_error = None
        for kind in kinds:
            try:
                self._create(kind)
                last_error = None
                break
            except Exception as e:  # fall through to the next backend, all ranks fail alike
                last_error = e
                logger.warning(f"symmetric heap backend {kind} failed: {e}")
                self._destroy_native()
        # every rank must have ended on the same backend
        kinds_seen = D.distributed_allgather(np.array([self.kind if last_error is None else -1], dtype=np.int64), group)
        if last_error is not None or len(set(int(k) for k in kinds_seen.flatten())) != 1:
            raise RuntimeError(f"could not create a symmetric heap on every rank: {last_error}; backends {kinds_seen.flatten().tolist()}")

        self.mc_base = 0
        if enable_multicast is None:
            enable_multicast = os.environ.get("IRIS_NVLS", "1") != "0"
        if enable_multicast and self.kind == KIND_VMM and num_ranks > 1:
            self._setup_multicast()
        bases = [rt.iris_heap_peer_base(self._handle, r) for r in range(num_ranks)]
        self._bases_host = np.array(bases, dtype=np.uint64)
        # int64 on the device, as in the reference ("for gloo compatibility", symmetric_heap.py:83-91)
        self.heap_bases = torch.from_numpy(self._bases_host.view(np.int64).copy()).to(self.device)
        if self._mesh is not None:
            self._mesh.close()
            self._mesh = None
        dist.barrier(group=group)

    # ------------------------------------------------------------------ construction
    def _create(self, kind: int) -> None:
        rt = _rt()
        err = C.create_string_buffer(_ERRLEN)
        if kind != KIND_CPU and self.device.type == "cuda":
            torch.cuda.set_device(self.device_id)
            torch.zeros(1, device=f"cuda:{self.device_id}")  # make sure the primary context exists
        create_size = self.heap_size
        if self.reserve and kind == KIND_VMM:
            rt.iris_heap_set_next_reserve(self.reserve)
            create_size = self._initial_size
        # Every step that can fail on one rank only is followed by a vote, so that all ranks leave this backend
        # together (a rank that went on alone to the next backend would sit in a different exchange than its peers).
        def agree(ok: bool, what: str, msg: str = "") -> None:
            if self.num_ranks == 1:
                if not ok:
                    raise RuntimeError(msg or what)
                return
            oks = D.distributed_allgather(np.array([1 if ok else 0], dtype=np.int64), self.group).flatten()
            if not all(int(o) for o in oks):
                bad = [r for r, o in enumerate(oks) if not int(o)]
                raise RuntimeError(f"{what} failed on rank(s) {bad}" + (f": {msg}" if msg else ""))

        h = rt.iris_heap_create(create_size, self.device_id, self.cur_rank, self.num_ranks, kind, 0, err, _ERRLEN)
        msg = "" if h else err.value.decode()
        fd, blob = -1, None
        if h:
            self._handle = h
            self.kind = kind
            self.base = rt.iris_heap_base(h)
            if self.num_ranks > 1:
                if kind in (KIND_VMM, KIND_CPU):
                    fd = rt.iris_heap_export_fd(h, err, _ERRLEN)
                    if fd < 0:
                        msg = err.value.decode()
                else:
                    blob = C.create_string_buffer(64)
                    if rt.iris_heap_export_blob(h, blob, err, _ERRLEN) != 0:
                        msg, blob = err.value.decode(), None
        local_ok = bool(h) and (self.num_ranks == 1 or fd >= 0 or blob is not None)
        try:
            agree(local_ok, "creating / exporting the heap", msg)
        except RuntimeError:
            if fd >= 0:
                rt.iris_close_fd(fd)
            raise
        if self.num_ranks == 1:
            return
        msg = ""
        if kind in (KIND_VMM, KIND_CPU):
            if self._mesh is None:
                self._mesh = FdMesh(self.cur_rank, self.num_ranks, self.group)
            try:
                for p in range(self.num_ranks):
                    if p != self.cur_rank:
                        self._mesh.send(p, fd, _TAG_HEAP)
                for _ in range(self.num_ranks - 1):      # every message is taken off the mesh even after a failure
                    pfd, src, tag, _ = self._mesh.recv()
                    if tag != _TAG_HEAP or pfd < 0:
                        msg = msg or f"unexpected message (tag {tag}) while exchanging heap handles"
                        continue
                    rc = rt.iris_heap_import_fd(h, src, pfd, err, _ERRLEN)
                    rt.iris_close_fd(pfd)
                    if rc != 0:
                        msg = msg or f"mapping rank {src}'s heap: {err.value.decode()}"
            except Exception as e:  # a broken mesh: still vote below, the peers must not wait for this rank
                msg = msg or f"{type(e).__name__}: {e}"
            finally:
                rt.iris_close_fd(fd)
        else:
            blobs = D.distributed_allgather(np.frombuffer(blob.raw, dtype=np.uint8).copy(), self.group)
            for p in range(self.num_ranks):
                if p == self.cur_rank:
                    continue
                if rt.iris_heap_import_blob(h, p, blobs[p].tobytes(), err, _ERRLEN) != 0:
                    msg = msg or f"opening rank {p}'s IPC handle: {err.value.decode()}"
        agree(not msg, "mapping the peers' heaps", msg)

    def _setup_multicast(self) -> None:
        """Bind the heap to an NVLS multicast object; on any failure continue without it."""
        rt = _rt()
        err = C.create_string_buffer(_ERRLEN)
        ok = 1 if rt.iris_heap_mc_supported(self.device_id) else 0
        fd = -1
        if ok and self.cur_rank == 0:
            fd = rt.iris_heap_mc_create(self._handle, err, _ERRLEN)
            if fd < 0:
                logger.warning(f"NVLS multicast unavailable: {err.value.decode()}")
                ok = 0
        oks = D.distributed_allgather(np.array([ok], dtype=np.int64), self.group).flatten()
        if not all(int(o) for o in oks):
            if fd >= 0:
                rt.iris_close_fd(fd)
            return
        if self.cur_rank == 0:
            for p in range(1, self.num_ranks):
                self._mesh.send(p, fd, _TAG_MC)
            rc = rt.iris_heap_mc_attach(self._handle, fd, 1, err, _ERRLEN)
            rt.iris_close_fd(fd)
        else:
            pfd, _, tag, _ = self._mesh.recv()
            if tag != _TAG_MC:
                raise RuntimeError("unexpected message while exchanging the multicast handle")
            rc = rt.iris_heap_mc_attach(self._handle, pfd, 0, err, _ERRLEN)
            rt.iris_close_fd(pfd)
        oks = D.distributed_allgather(np.array([1 if rc == 0 else 0], dtype=np.int64), self.group).flatten()
        if not all(int(o) for o in oks):
            logger.warning(f"NVLS multicast attach failed on some rank: {err.value.decode()}")
            return
        rc = rt.iris_heap_mc_bind(self._handle, err, _ERRLEN)
        oks = D.distributed_allgather(np.array([1 if rc == 0 else 0], dtype=np.int64), self.group).flatten()
        if not all(int(o) for o in oks):
            logger.warning(f"NVLS multicast bind failed on some rank: {err.value.decode()}")
            return
        self.mc_base = rt.iris_heap_mc_base(self._handle)

    # ------------------------------------------------------------------ allocation
    def allocate(self, num_elements: int, dtype: torch.dtype, alignment: int = 1024) -> torch.Tensor:
        """Bump-allocate ``num_elements`` of ``dtype`` (flat tensor). Raises MemoryError when full."""
        elem = torch.empty((), dtype=dtype).element_size()
        nbytes = int(num_elements) * elem
        off = _rt().iris_heap_alloc(self._handle, nbytes, alignment)
        if off < 0 and self.reserve:
            # growable heap: map more physical memory behind what is mapped (collective: every rank reaches this
            # point of its allocation sequence with the same request), then allocate again
            used = _rt().iris_heap_offset(self._handle)
            mapped = _rt().iris_heap_mapped_size(self._handle)
            start = -(-used // alignment) * alignment
            need = start + max(nbytes, alignment) - mapped
            chunk = int(os.environ.get("IRIS_VMEM_CHUNK", str(64 << 20)))
            grow = max(need, min(chunk, self.reserve - mapped))
            if mapped + need <= self.reserve and grow > 0:
                self._add_segment(lambda err: _rt().iris_heap_grow(self._handle, int(grow), err, _ERRLEN))
                off = _rt().iris_heap_alloc(self._handle, nbytes, alignment)
        if off < 0:
            used = _rt().iris_heap_offset(self._handle)
            raise MemoryError(f"Heap out of memory: requested {nbytes} bytes, {self.heap_size - used} of {self.heap_size} free")
        t = tensor_from_ptr(self.base + off, int(num_elements), dtype, self.device, keepalive=self)
        if self.poison and nbytes:
            # debug mode: fresh memory reads as NaN (floating point) or -1 (integers), so that a
            # kernel that consumes data nobody wrote shows up in the first comparison
            t.view(torch.uint8).fill_(0xFF)
        return t

    def get_heap_bases(self) -> torch.Tensor:
        return self.heap_bases

    def bases_host(self) -> np.ndarray:
        return self._bases_host

    def get_offset(self) -> int:
        return _rt().iris_heap_offset(self._handle)

    def set_offset(self, offset: int) -> None:
        """Rewind (or advance) the bump pointer; every rank must do the same."""
        _rt().iris_heap_set_offset(self._handle, int(offset))

    def owns_ptr(self, ptr: int, nbytes: int = 0) -> bool:
        return self.base <= ptr and ptr + nbytes <= self.base + self.heap_size

    def is_symmetric(self, tensor: torch.Tensor) -> bool:
        """True when ``tensor``'s storage lies inside this rank's heap (zero-size tensors count)."""
        if not isinstance(tensor, torch.Tensor):
            return False
        if tensor.device.type != self.device.type:
            return False
        if tensor.numel() == 0:
            return True
        return self.owns_ptr(tensor.data_ptr(), tensor.numel() * tensor.element_size() if tensor.is_contiguous() else 0)

    # ------------------------------------------------------------------ segments (growable heaps)
    def _add_segment(self, make) -> int:
        """Create one more segment of this rank's heap with ``make(err) -> index`` and map every peer's new
        segment at the same offset of that peer's window (collective; descriptors travel over the fd mesh)."""
        rt = _rt()
        err = C.create_string_buffer(_ERRLEN)
        seg = make(err)
        ok = seg >= 0
        msg = err.value.decode() if not ok else ""
        off = rt.iris_heap_segment_offset(self._handle, seg) if ok else 0
        size = rt.iris_heap_segment_size(self._handle, seg) if ok else 0
        # every rank must have got the same segment, or the heaps stop being symmetric
        seen = D.distributed_allgather(np.array([1 if ok else 0, off, size], dtype=np.int64), self.group).reshape(-1, 3)
        if not all(int(r[0]) for r in seen):
            raise RuntimeError(f"a rank could not add a heap segment: {msg or 'see the other ranks'}")
        if len({(int(r[1]), int(r[2])) for r in seen}) != 1:
            raise RuntimeError(f"heap segments differ between ranks (offset, size): {[(int(r[1]), int(r[2])) for r in seen]}")
        if self.num_ranks > 1:
            mesh = FdMesh(self.cur_rank, self.num_ranks, self.group)
            fd = rt.iris_heap_segment_export_fd(self._handle, seg, err, _ERRLEN)
            try:
                if fd < 0:
                    raise RuntimeError(err.value.decode())
                for p in range(self.num_ranks):
                    if p != self.cur_rank:
                        mesh.send(p, fd, _TAG_HEAP)
                for _ in range(self.num_ranks - 1):
                    pfd, src, tag, _ = mesh.recv()
                    if tag != _TAG_HEAP or pfd < 0:
                        raise RuntimeError(f"unexpected message (tag {tag}) while exchanging segment handles")
                    rc = rt.iris_heap_segment_import_fd(self._handle, src, pfd, off, size, err, _ERRLEN)
                    rt.iris_close_fd(pfd)
                    if rc != 0:
                        raise RuntimeError(f"mapping rank {src}'s segment: {err.value.decode()}")
            finally:
                if fd >= 0:
                    rt.iris_close_fd(fd)
                mesh.close()
            dist.barrier(group=self.group)
        self.heap_size = max(self.heap_size, rt.iris_heap_mapped_size(self._handle)) if not self.reserve else self.heap_size
        return seg

    def import_external_tensor(self, tensor: torch.Tensor) -> torch.Tensor:
        """Map the allocation behind ``tensor`` into the heap WITHOUT copying (collective) and return the view of
        ``tensor`` at its heap address: peers reach it like any heap tensor, and both views alias the same memory
        (reference: allocators/vmem_allocator.py:241-317). Needs a growable heap (``allocator_type="vmem"``) and
        memory that was created with the driver's virtual-memory API and may be shared through a file descriptor;
        anything else (``cudaMalloc``'d pools) raises ``RuntimeError`` and ``as_symmetric`` falls back to a copy.
        Every rank must import an allocation of the same size."""
        if not self.reserve:
            raise RuntimeError("import_external_tensor needs a growable heap (allocator_type='vmem')")
        rt = _rt()
        inner = C.c_uint64(0)
        seg = self._add_segment(lambda err: rt.iris_heap_import_external(self._handle, tensor.data_ptr(), C.byref(inner), err, _ERRLEN))
        off = rt.iris_heap_segment_offset(self._handle, seg)
        size = rt.iris_heap_segment_size(self._handle, seg)
        rt.iris_heap_set_offset(self._handle, off + size)           # later allocations come after the imported segment
        span = (tensor.untyped_storage().nbytes() - tensor.storage_offset() * tensor.element_size()) // tensor.element_size()
        flat = tensor_from_ptr(self.base + off + inner.value, max(span, tensor.numel()), tensor.dtype, self.device, keepalive=(self, tensor))
        return flat.as_strided(tensor.shape, tensor.stride())

    def as_symmetric(self, tensor: torch.Tensor) -> torch.Tensor:
        """Return a tensor on the heap with ``tensor``'s contents (the tensor itself if already there). On a
        growable heap the tensor's own memory is mapped into the heap when the driver allows it (no copy);
        otherwise the contents are copied into a fresh heap allocation."""
        if self.is_symmetric(tensor):
            return tensor
        if self.reserve and tensor.device.type == self.device.type and os.environ.get("IRIS_VMEM_IMPORT", "1") != "0":
            # all ranks decide together: an import that one rank cannot do must not leave the others in the exchange
            can = 1
            try:
                from .platform import mem_retain_allocation_handle, mem_release
                mem_release(mem_retain_allocation_handle(tensor.data_ptr()))
            except Exception:
                can = 0
            votes = D.distributed_allgather(np.array([can], dtype=np.int64), self.group)
            if int(votes.min()) == 1:
                return self.import_external_tensor(tensor)
        flat = self.allocate(tensor.numel(), tensor.dtype)
        out = flat.view(tensor.shape) if tensor.is_contiguous() else flat.view(tensor.shape)
        out.copy_(tensor)
        return out

    def offset_of(self, tensor: torch.Tensor) -> int:
        return tensor.data_ptr() - self.base

    def peer_view(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        """The same object on ``rank``, addressed through this process's mapping of that heap."""
        if not self.is_symmetric(tensor):
            raise ValueError("tensor is not on the symmetric heap")
        ptr = int(self._bases_host[rank]) + self.offset_of(tensor)
        flat = tensor_from_ptr(ptr, tensor.numel(), tensor.dtype, self.device, keepalive=self)
        return flat.as_strided(tensor.shape, tensor.stride()) if tensor.numel() else flat.view(tensor.shape)

    # ------------------------------------------------------------------ teardown
    def _destroy_native(self) -> None:
        if self._handle:
            _rt().iris_heap_destroy(self._handle)
            self._handle = None

    def close(self) -> None:
        if self._handle and self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._destroy_native()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
