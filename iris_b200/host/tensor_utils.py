"""Wrap raw addresses as torch tensors without copying.

GPU memory goes through ``__cuda_array_interface__`` (as the reference does,
iris/host/memory/tensor_utils.py:13-135); host memory (CPU backend) through a ctypes buffer.
Element types that the array interface cannot name (bf16, fp8) are created as integers of the
same width and re-viewed.
"""
from __future__ import annotations

import ctypes

import torch

_TYPESTR = {
    torch.float32: "<f4", torch.float64: "<f8", torch.float16: "<f2",
    torch.int8: "|i1", torch.uint8: "|u1", torch.int16: "<i2", torch.int32: "<i4", torch.int64: "<i8",
    torch.bool: "|b1",
}
_CARRIER = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}


class CUDAArrayInterface:
    """Minimal object exposing ``__cuda_array_interface__`` for a device pointer."""

    def __init__(self, ptr: int, shape, typestr: str, owner=None):
        self.ptr = int(ptr)
        self.shape = tuple(shape)
        self.typestr = typestr
        self._owner = owner

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": self.typestr, "data": (self.ptr, False), "version": 3, "strides": None}


def tensor_from_ptr(ptr: int, num_elements: int, dtype: torch.dtype, device, keepalive=None) -> torch.Tensor:
    """A flat tensor of ``num_elements`` x ``dtype`` at address ``ptr`` on ``device`` (no copy)."""
    device = torch.device(device)
    esize = torch.empty((), dtype=dtype).element_size()
    if num_elements == 0:
        return torch.empty((0,), dtype=dtype, device=device)
    carrier = dtype if dtype in _TYPESTR else _CARRIER[esize]
    if device.type == "cuda":
        obj = CUDAArrayInterface(ptr, (num_elements,), _TYPESTR[carrier], owner=keepalive)
        t = torch.as_tensor(obj, device=device)
    else:
        buf = (ctypes.c_uint8 * (num_elements * esize)).from_address(ptr)
        buf._owner = keepalive  # torch keeps `buf` alive with the storage, and `buf` the mapping
        t = torch.frombuffer(buf, dtype=carrier, count=num_elements)
    if carrier != dtype:
        t = t.view(dtype)
    return t
