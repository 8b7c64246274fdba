"""GPU runtime queries and the benchmark loop.

The module is also importable as ``iris_b200.hip`` so that code written against the reference's
``iris.hip`` keeps working: same function names (iris/host/platform/hip.py), answered by the CUDA
driver through the native runtime library. ``get_cu_count`` is the SM count, ``get_num_xcc`` is 1
(a B200 is presented as one device; there are no XCD chiplets to swizzle over).
"""
from __future__ import annotations

import ctypes as C
import os
import statistics

import torch

from .heap import _rt

# CUdevice_attribute values used below
_ATTR_SM_COUNT = 16
_ATTR_CLOCK_RATE = 13
_ATTR_CC_MAJOR = 75
_ATTR_CC_MINOR = 76
_ATTR_MAX_SMEM_OPTIN = 97
_ATTR_MULTICAST = 132


def is_simulation_env() -> bool:
    """True when ``IRIS_SIMULATION`` asks for several ranks on one device (heap only, no kernels)."""
    return os.environ.get("IRIS_SIMULATION", "0") not in ("", "0")


def count_devices() -> int:
    return _rt().iris_rt_device_count()


def set_device(device_id: int) -> None:
    if torch.cuda.is_available():
        torch.cuda.set_device(device_id)
    if _rt().iris_rt_set_device(device_id) != 0 and torch.cuda.is_available():
        raise RuntimeError(f"cannot make device {device_id} current")


def get_device_id() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else -1


def get_cu_count(device_id: int | None = None) -> int:
    """Number of SMs (the reference's compute units)."""
    return _rt().iris_rt_device_attribute(get_device_id() if device_id is None else device_id, _ATTR_SM_COUNT)


def get_wall_clock_rate(device_id: int | None = None) -> int:
    """Rate of the device timestamp used by tracing, in kHz: ``%globaltimer`` counts nanoseconds."""
    return 1_000_000


def get_sm_clock_rate(device_id: int | None = None) -> int:
    return _rt().iris_rt_device_attribute(get_device_id() if device_id is None else device_id, _ATTR_CLOCK_RATE)


def get_arch_string(device_id: int | None = None) -> str:
    d = get_device_id() if device_id is None else device_id
    major = _rt().iris_rt_device_attribute(d, _ATTR_CC_MAJOR)
    minor = _rt().iris_rt_device_attribute(d, _ATTR_CC_MINOR)
    return f"sm_{major}{minor}"


def get_device_name(device_id: int | None = None) -> str:
    buf = C.create_string_buffer(256)
    _rt().iris_rt_device_name(get_device_id() if device_id is None else device_id, buf, 256)
    return buf.value.decode()


def get_num_xcc(device_id: int | None = None) -> int:
    return 1


def multicast_supported(device_id: int | None = None) -> bool:
    return _rt().iris_rt_device_attribute(get_device_id() if device_id is None else device_id, _ATTR_MULTICAST) == 1


def can_access_peer(device_id: int, peer_id: int) -> bool:
    return bool(_rt().iris_rt_can_access_peer(device_id, peer_id))


def get_address_range(ptr: int):
    """``(base, size)`` of the device allocation containing ``ptr``."""
    base, size = C.c_uint64(0), C.c_uint64(0)
    if _rt().iris_rt_address_range(int(ptr), C.byref(base), C.byref(size)) != 0:
        raise RuntimeError(f"address {ptr:#x} is not inside a device allocation")
    return base.value, size.value


def get_ipc_handle(ptr: int) -> bytes:
    buf = C.create_string_buffer(64)
    if _rt().iris_rt_ipc_get_handle(int(ptr), buf) != 0:
        raise RuntimeError("cuIpcGetMemHandle failed")
    return buf.raw


def open_ipc_handle(handle: bytes) -> int:
    ptr = C.c_uint64(0)
    rc = _rt().iris_rt_ipc_open_handle(bytes(handle), C.byref(ptr))
    if rc != 0:
        raise RuntimeError(f"cuIpcOpenMemHandle failed ({-rc})")
    return ptr.value


def close_ipc_handle(ptr: int) -> None:
    _rt().iris_rt_ipc_close_handle(int(ptr))


# ---------------------------------------------------------------------------------------------------
# Driver-level memory primitives under the reference's names (iris/host/platform/hip.py:264-846). The
# symmetric heap does not use them; they are for code that builds its own mappings.
class DriverError(RuntimeError):
    """A driver call failed; ``code`` is the CUresult (1000 = no driver on this machine)."""

    def __init__(self, what: str, code: int):
        self.code = code
        buf = C.create_string_buffer(128)
        if code != 1000:
            _rt().iris_rt_error_string(code, buf, 128)
        detail = buf.value.decode() or "no CUDA driver on this machine"
        super().__init__(f"{what} failed: {detail}")


def gpu_try(rc: int, what: str = "driver call") -> None:
    """Raise ``DriverError`` for a non-zero return code of the native runtime (0 passes)."""
    if rc != 0:
        raise DriverError(what, -rc)


def install_fake_driver(devices: int = 0) -> int:
    """Tests only: route the native runtime to a host-memory stand-in for the driver's memory API with
    ``devices`` devices (0 switches back to the real driver). Touches no GPU."""
    return _rt().iris_rt_install_fake_driver(int(devices))


def get_driver_version() -> int:
    v = C.c_int(0)
    gpu_try(_rt().iris_rt_driver_version(C.byref(v)), "cuDriverGetVersion")
    return v.value


def get_rocm_version():
    """The reference returns ``(major, minor)`` of ROCm; here of the CUDA driver API."""
    v = get_driver_version()
    return v // 1000, (v % 1000) // 10


def get_ipc_handle_size() -> int:
    return 64


def hip_malloc(size: int, device_id: int | None = None) -> int:
    """Plain device allocation; returns the address. (``malloc_fine_grained`` is the same call: device
    memory of an NVLink domain is coherent for peers at system scope, there is no separate pool.)"""
    ptr = C.c_uint64(0)
    gpu_try(_rt().iris_rt_malloc(max(get_device_id(), 0) if device_id is None else device_id, int(size), C.byref(ptr)), "cuMemAlloc")
    return ptr.value


malloc_fine_grained = hip_malloc


def hip_free(ptr: int) -> None:
    gpu_try(_rt().iris_rt_free(int(ptr)), "cuMemFree")


def get_allocation_granularity(device_id: int = 0, recommended: bool = True, fabric: bool = False) -> int:
    g = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_granularity(device_id, int(fabric), int(recommended), C.byref(g)), "cuMemGetAllocationGranularity")
    return g.value


def mem_create(size: int, device_id: int = 0, fabric: bool = False) -> int:
    """Physical allocation of ``size`` bytes (a multiple of the granularity); returns its handle."""
    h = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_create(int(size), device_id, int(fabric), C.byref(h)), "cuMemCreate")
    return h.value


def mem_release(handle: int) -> None:
    gpu_try(_rt().iris_rt_mem_release(int(handle)), "cuMemRelease")


def mem_address_reserve(size: int, alignment: int = 0, hint: int = 0) -> int:
    p = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_address_reserve(int(size), int(alignment), int(hint), C.byref(p)), "cuMemAddressReserve")
    return p.value


def mem_address_free(ptr: int, size: int) -> None:
    gpu_try(_rt().iris_rt_mem_address_free(int(ptr), int(size)), "cuMemAddressFree")


def mem_map(ptr: int, size: int, offset: int, handle: int) -> None:
    gpu_try(_rt().iris_rt_mem_map(int(ptr), int(size), int(offset), int(handle)), "cuMemMap")


def mem_unmap(ptr: int, size: int) -> None:
    gpu_try(_rt().iris_rt_mem_unmap(int(ptr), int(size)), "cuMemUnmap")


def mem_set_access(ptr: int, size: int, device_ids) -> None:
    """Read-write access to the mapped range for the listed devices (an int or a sequence)."""
    ids = [device_ids] if isinstance(device_ids, int) else list(device_ids)
    arr = (C.c_int * len(ids))(*ids)
    gpu_try(_rt().iris_rt_mem_set_access(int(ptr), int(size), arr, len(ids)), "cuMemSetAccess")


def mem_export_to_shareable_handle(handle: int) -> int:
    """POSIX file descriptor of an allocation (pass it to another process over the fd mesh)."""
    fd = C.c_int(-1)
    gpu_try(_rt().iris_rt_mem_export_fd(int(handle), C.byref(fd)), "cuMemExportToShareableHandle")
    return fd.value


def mem_import_from_shareable_handle(fd: int) -> int:
    h = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_import_fd(int(fd), C.byref(h)), "cuMemImportFromShareableHandle")
    return h.value


def mem_retain_allocation_handle(ptr: int) -> int:
    """Handle of the VMM allocation mapped at ``ptr`` (retained: ``mem_release`` it). Raises for memory that
    was not created with the virtual-memory API (``cudaMalloc``'d pools)."""
    h = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_retain_handle(int(ptr), C.byref(h)), "cuMemRetainAllocationHandle")
    return h.value


def export_dmabuf_handle(ptr: int, size: int = 0) -> int:
    """File descriptor for the allocation mapped at ``ptr`` (the reference exports a DMA-BUF of an
    address range; here the range must be a VMM mapping, whose allocation handle is exported)."""
    h = C.c_uint64(0)
    gpu_try(_rt().iris_rt_mem_retain_handle(int(ptr), C.byref(h)), "cuMemRetainAllocationHandle")
    try:
        return mem_export_to_shareable_handle(h.value)
    finally:
        mem_release(h.value)


def import_dmabuf_handle(fd: int, size: int, device_ids=0):
    """Map the allocation behind ``fd`` into this process; returns ``(handle, address)``."""
    h = mem_import_from_shareable_handle(fd)
    ptr = mem_address_reserve(size)
    mem_map(ptr, size, 0, h)
    mem_set_access(ptr, size, device_ids)
    return h, ptr


def destroy_external_memory(handle: int, ptr: int = 0, size: int = 0) -> None:
    """Undo ``import_dmabuf_handle``: unmap and free the range (when given), release the handle."""
    if ptr:
        mem_unmap(ptr, size)
        mem_address_free(ptr, size)
    mem_release(handle)


def get_device_id_for_rank(rank: int, num_gpus: int | None = None) -> int:
    """Device a rank should use: ``LOCAL_RANK`` when a launcher set it, else ``rank % num_gpus``."""
    if num_gpus is None:
        num_gpus = max(torch.cuda.device_count(), 1)
    local = os.environ.get("LOCAL_RANK")
    if local is not None:
        return int(local) % num_gpus
    return rank % num_gpus


_L2_FLUSH = {}


def _flush_l2(device) -> None:
    """Overwrite a buffer larger than the 126 MB L2 so the next iteration starts cold."""
    buf = _L2_FLUSH.get(device)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.int8, device=device)
        _L2_FLUSH[device] = buf
    buf.zero_()


def do_bench(fn, barrier_fn=lambda: None, preamble_fn=lambda: None, n_warmup: int = 25, n_repeat: int = 100,
             quantiles=None, return_mode: str = "mean"):
    """Time ``fn`` with CUDA events on the current stream.

    Protocol of the reference (iris/host/platform/utils.py:137-201): one untimed call, ``n_warmup``
    warm-ups, then ``n_repeat`` timed iterations, each preceded by ``barrier_fn(); preamble_fn();``
    an L2 flush and another ``barrier_fn()``. Returns milliseconds: ``return_mode`` in
    ``mean|min|max|median|all``, or the requested quantiles. Use ``iris_b200.utils.time_max_over_ranks``
    when the number has to be the maximum over ranks.
    """
    if return_mode not in ("mean", "min", "max", "median", "all"):
        raise ValueError(f"unknown return_mode {return_mode!r}")
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else None

    def once(timed: bool):
        barrier_fn()
        preamble_fn()
        if cuda:
            _flush_l2(dev)
        barrier_fn()
        if not timed:
            fn()
            return 0.0
        if cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e)
        import time

        t0 = time.perf_counter()
        fn()
        return (time.perf_counter() - t0) * 1e3

    once(False)
    if cuda:
        torch.cuda.synchronize()
    for _ in range(n_warmup):
        once(False)
    if cuda:
        torch.cuda.synchronize()
    times = [once(True) for _ in range(n_repeat)]
    if quantiles is not None:
        ts = torch.tensor(times, dtype=torch.float64)
        q = torch.quantile(ts, torch.tensor(quantiles, dtype=torch.float64)).tolist()
        return q[0] if len(q) == 1 else q
    if return_mode == "all":
        return times
    return {"mean": statistics.fmean, "min": min, "max": max, "median": statistics.median}[return_mode](times)
