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
