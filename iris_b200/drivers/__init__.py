"""Fabric drivers: export / import of device memory between processes and nodes.

``BaseFabricDriver`` is the abstract surface (reference: iris/drivers/base.py:25-78);
``NvidiaFabricDriver`` implements it on CUDA VMM fabric handles through the native runtime
(reference: iris/drivers/fabric/nvidia.py:265-454, there through ctypes); ``AmdFabricDriver`` raises
``DriverNotSupported``. ``DriverStack`` picks the driver for the platform. Inside one node the
symmetric heap shares POSIX file descriptors instead (iris_b200/host/heap.py); fabric handles are
for multi-node NVLink domains.
"""
from __future__ import annotations

import ctypes as C
from abc import ABC, abstractmethod
from dataclasses import dataclass

FABRIC_HANDLE_BYTES = 64


class DriverNotSupported(RuntimeError):
    pass


class DriverNotInitialized(RuntimeError):
    pass


@dataclass
class LocalAllocation:
    handle: int      # native heap object
    va: int
    size: int


@dataclass
class PeerMapping:
    owner: int       # native heap object holding the mapping
    slot: int
    va: int
    size: int


class BaseFabricDriver(ABC):
    @abstractmethod
    def initialize(self, device_id: int) -> None: ...

    @abstractmethod
    def allocate_exportable(self, size: int) -> LocalAllocation: ...

    @abstractmethod
    def export_handle(self, alloc: LocalAllocation) -> bytes: ...

    @abstractmethod
    def import_and_map(self, handle: bytes, size: int) -> PeerMapping: ...

    @abstractmethod
    def cleanup_import(self, mapping: PeerMapping) -> None: ...

    @abstractmethod
    def cleanup_local(self, alloc: LocalAllocation) -> None: ...


class NvidiaFabricDriver(BaseFabricDriver):
    """CUDA VMM allocations with ``CU_MEM_HANDLE_TYPE_FABRIC`` (64-byte handles)."""

    MAX_IMPORTS = 72

    def __init__(self, runtime=None):
        self._rt = runtime
        self.device_id = None
        self._import_heap = None
        self._next_slot = 1

    def _lib(self):
        if self._rt is None:
            from ..host.heap import _rt

            self._rt = _rt()
        return self._rt

    def _need_init(self):
        if self.device_id is None:
            raise DriverNotInitialized("call initialize(device_id) first")

    def initialize(self, device_id: int) -> None:
        err = C.create_string_buffer(512)
        if not self._lib().iris_rt_cuda_ok(err, 512):
            raise DriverNotSupported(f"CUDA driver unavailable: {err.value.decode()}")
        if self._lib().iris_rt_set_device(device_id) != 0:
            raise DriverNotSupported(f"cannot use device {device_id}")
        self.device_id = device_id

    def allocate_exportable(self, size: int) -> LocalAllocation:
        self._need_init()
        err = C.create_string_buffer(512)
        h = self._lib().iris_heap_create(size, self.device_id, 0, self.MAX_IMPORTS, 0, 1, err, 512)
        if not h:
            raise RuntimeError(f"fabric allocation failed: {err.value.decode()}")
        return LocalAllocation(handle=h, va=self._lib().iris_heap_base(h), size=self._lib().iris_heap_mapped_size(h))

    def export_handle(self, alloc: LocalAllocation) -> bytes:
        self._need_init()
        blob, err = C.create_string_buffer(FABRIC_HANDLE_BYTES), C.create_string_buffer(512)
        if self._lib().iris_heap_export_blob(alloc.handle, blob, err, 512) != 0:
            raise RuntimeError(f"fabric export failed: {err.value.decode()}")
        return blob.raw

    def import_and_map(self, handle: bytes, size: int) -> PeerMapping:
        self._need_init()
        if len(handle) != FABRIC_HANDLE_BYTES:
            raise ValueError(f"a fabric handle is {FABRIC_HANDLE_BYTES} bytes, got {len(handle)}")
        if self._import_heap is None:
            self._import_heap = self.allocate_exportable(size)
        if self._next_slot >= self.MAX_IMPORTS:
            raise RuntimeError("too many imported mappings")
        err = C.create_string_buffer(512)
        slot = self._next_slot
        if self._lib().iris_heap_import_blob(self._import_heap.handle, slot, bytes(handle), err, 512) != 0:
            raise RuntimeError(f"fabric import failed: {err.value.decode()}")
        self._next_slot += 1
        return PeerMapping(owner=self._import_heap.handle, slot=slot, va=self._lib().iris_heap_peer_base(self._import_heap.handle, slot), size=size)

    def cleanup_import(self, mapping: PeerMapping) -> None:
        # mappings are released together with the heap object that holds them (cleanup_local /
        # close): the native destroy attempts every unmap / release step even after a failure
        pass

    def cleanup_local(self, alloc: LocalAllocation) -> int:
        failures = self._lib().iris_heap_destroy(alloc.handle)
        alloc.handle = 0
        return failures

    def close(self) -> int:
        failures = 0
        if self._import_heap is not None:
            failures = self.cleanup_local(self._import_heap)
            self._import_heap = None
        return failures


class AmdFabricDriver(BaseFabricDriver):
    def _no(self, *a, **k):
        raise DriverNotSupported("this framework targets NVIDIA B200; there is no AMD fabric driver")

    initialize = allocate_exportable = export_handle = import_and_map = cleanup_import = cleanup_local = _no


class DriverStack:
    """Select and hold the fabric driver of the platform."""

    def __init__(self, vendor: str | None = None, runtime=None):
        if vendor is None:
            import torch

            vendor = "amd" if getattr(torch.version, "hip", None) else "nvidia"
        self.vendor = vendor
        self.fabric = NvidiaFabricDriver(runtime) if vendor == "nvidia" else AmdFabricDriver()


def fabric_handle_bytes_to_tensor(handle: bytes):
    """A 64-byte handle as a uint8 tensor (for exchange with torch.distributed collectives)."""
    import torch

    if len(handle) != FABRIC_HANDLE_BYTES:
        raise ValueError(f"a fabric handle is {FABRIC_HANDLE_BYTES} bytes")
    return torch.tensor(list(handle), dtype=torch.uint8)
