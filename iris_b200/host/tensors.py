"""torch-style tensor factories whose storage lives on the symmetric heap.

Same calling conventions as ``torch.zeros`` & co. (``out=``, ``dtype``, ``layout``, ``device``,
``requires_grad``, ``memory_format``), with the checks the reference applies: the device must be
the context's device, an ``out=`` tensor must already be on the heap with the right element count
and dtype, only the strided layout exists (reference: iris/host/memory/tensors.py:28-881).
All factories funnel through ``_materialise``; values are produced by torch on the heap memory in
place, so no staging copy is made.
"""
from __future__ import annotations

import math

import torch

from .logging import logger


def parse_size(size):
    """Normalise ``f(2, 3)``, ``f((2, 3))``, ``f([2, 3])`` to ``((2, 3), 6)``."""
    while len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
        size = size[0]
    size = tuple(int(s) for s in size)
    return size, math.prod(size)


def is_valid_device(device, iris_device) -> bool:
    if device is None:
        return True
    dev = torch.device(device)
    iris_device = torch.device(iris_device)
    if dev.type != iris_device.type:
        return False
    return dev.index is None or iris_device.index is None or dev.index == iris_device.index


def throw_if_invalid_device(device, iris_device) -> None:
    if not is_valid_device(device, iris_device):
        raise RuntimeError(
            f"Device mismatch: requested device {device} but Iris instance is on device {iris_device}. "
            f"Iris only supports tensors on its own device."
        )


def throw_if_invalid_output_tensor(heap, tensor: torch.Tensor, num_elements: int, dtype: torch.dtype) -> None:
    if tensor.numel() != num_elements:
        raise RuntimeError(f"The output tensor has {tensor.numel()} elements, but {num_elements} are required")
    if tensor.dtype != dtype:
        raise RuntimeError(f"The output tensor has dtype {tensor.dtype}, but {dtype} is required")
    if not heap.is_symmetric(tensor):
        raise RuntimeError("The output tensor is not on the symmetric heap")


def apply_layout(tensor: torch.Tensor, layout) -> torch.Tensor:
    if layout != torch.strided:
        raise ValueError(f"Layout {layout} not supported. Only torch.strided is currently supported.")
    return tensor


def _strided_on_heap(heap, flat_or_tensor: torch.Tensor, size, strides) -> torch.Tensor:
    """Re-lay ``tensor`` (logical shape ``size``) with ``strides`` in fresh heap memory."""
    src = flat_or_tensor.reshape(size)
    buf = heap.allocate(src.numel(), src.dtype)
    out = buf.as_strided(size, strides)
    out.copy_(src)
    return out


def apply_memory_format(heap, tensor: torch.Tensor, size, memory_format, input_tensor: torch.Tensor | None = None):
    if memory_format == torch.contiguous_format:
        return tensor
    if memory_format == torch.channels_last and len(size) == 4:
        _, c, h, w = size
        return _strided_on_heap(heap, tensor, size, (c * h * w, 1, c * w, c))
    if memory_format == torch.channels_last_3d and len(size) == 5:
        _, c, d, h, w = size
        # torch's NDHWC strides; the reference uses c*d*w for the depth stride, which aliases
        # elements whenever d != h (iris/host/memory/tensors.py:250)
        return _strided_on_heap(heap, tensor, size, (c * d * h * w, 1, h * w * c, w * c, c))
    if memory_format == torch.preserve_format and input_tensor is not None:
        st = input_tensor.stride()
        if len(size) in (4, 5) and len(st) == len(size) and st[1] == 1 and tuple(input_tensor.shape) == tuple(size):
            return _strided_on_heap(heap, tensor, size, st)
    return tensor


def _materialise(heap, iris_device, size, fill, *, out=None, dtype=None, layout=torch.strided, device=None,
                 requires_grad=False, memory_format=torch.contiguous_format, default_dtype=None, input_tensor=None):
    """Allocate (or validate ``out``), run ``fill(flat_tensor)`` in place, shape and decorate."""
    if dtype is None:
        dtype = default_dtype if default_dtype is not None else torch.get_default_dtype()
    throw_if_invalid_device(device, iris_device)
    if not isinstance(size, (tuple, list, torch.Size)):
        size = (size,)
    size, n = parse_size(tuple(size))
    if out is not None:
        throw_if_invalid_output_tensor(heap, out, n, dtype)
        flat = out.view(-1) if out.is_contiguous() else out.reshape(-1)
        if fill is not None:
            fill(flat)
        tensor = out.view(size)
    else:
        flat = heap.allocate(n, dtype)
        if fill is not None:
            fill(flat)
        tensor = flat.reshape(size)
    tensor = apply_memory_format(heap, tensor, size, memory_format, input_tensor)
    tensor = apply_layout(tensor, layout)
    if requires_grad:
        tensor.requires_grad_()
    return tensor


def zeros(heap, iris_device, size, **kw):
    logger.debug(f"zeros: size = {size}")
    return _materialise(heap, iris_device, size, lambda t: t.zero_(), **kw)


def ones(heap, iris_device, size, **kw):
    return _materialise(heap, iris_device, size, lambda t: t.fill_(1), **kw)


def full(heap, iris_device, size, fill_value, **kw):
    default = None
    if kw.get("dtype") is None:
        if isinstance(fill_value, bool):
            default = torch.bool
        elif isinstance(fill_value, int):
            default = torch.int64
        elif isinstance(fill_value, float):
            default = torch.get_default_dtype()
        elif isinstance(fill_value, complex):
            default = torch.complex64
    return _materialise(heap, iris_device, size, lambda t: t.fill_(fill_value), default_dtype=default, **kw)


def empty(heap, iris_device, size, *, pin_memory=False, **kw):
    if pin_memory:
        raise RuntimeError("pin_memory is a host-memory option and does not apply to the symmetric heap")
    return _materialise(heap, iris_device, size, None, **kw)


def zeros_like(heap, iris_device, input, *, dtype=None, layout=None, device=None, requires_grad=False,
               memory_format=torch.preserve_format):
    dtype = dtype if dtype is not None else input.dtype
    layout = layout if layout is not None else input.layout
    if device is None and input.device.type == torch.device(iris_device).type:
        device = input.device
    return _materialise(heap, iris_device, tuple(input.shape), lambda t: t.zero_(), dtype=dtype, layout=layout,
                        device=device, requires_grad=requires_grad, memory_format=memory_format, input_tensor=input)


def uniform(heap, iris_device, size, low=0.0, high=1.0, dtype=torch.float):
    return _materialise(heap, iris_device, size, lambda t: t.uniform_(low, high), dtype=dtype)


def rand(heap, iris_device, size, *, generator=None, pin_memory=False, **kw):
    return _materialise(heap, iris_device, size, lambda t: t.uniform_(0, 1, generator=generator), **kw)


def randn(heap, iris_device, size, *, generator=None, pin_memory=False, **kw):
    return _materialise(heap, iris_device, size, lambda t: t.normal_(0, 1, generator=generator), **kw)


def randint(heap, iris_device, low, high, size, *, generator=None, dtype=None, **kw):
    if dtype is None:
        dtype = torch.int64
    return _materialise(heap, iris_device, size, lambda t: t.random_(low, high, generator=generator), dtype=dtype, **kw)


def arange(heap, iris_device, start, end, step, *, out=None, dtype=None, layout=torch.strided, device=None,
           requires_grad=False):
    if step == 0:
        raise ValueError("step must be non-zero")
    if (step > 0 and start >= end) or (step < 0 and start <= end):
        raise ValueError(f"Invalid range: start={start}, end={end}, step={step}")
    n = int(math.ceil((end - start) / step))
    if dtype is None:
        floats = any(isinstance(v, float) for v in (start, end, step))
        dtype = torch.get_default_dtype() if floats else torch.int64

    def fill(t):
        torch.arange(start, end, step, out=t) if t.dtype not in (torch.bfloat16, torch.float16) else t.copy_(
            torch.arange(start, end, step, dtype=torch.float32, device=t.device))

    return _materialise(heap, iris_device, (n,), fill, out=out, dtype=dtype, layout=layout, device=device,
                        requires_grad=requires_grad)


def linspace(heap, iris_device, start, end, steps, *, out=None, dtype=None, layout=torch.strided, device=None,
             requires_grad=False):
    if steps < 0:
        raise ValueError("number of steps must be non-negative")
    if dtype is None:
        dtype = torch.complex64 if isinstance(start, complex) or isinstance(end, complex) else torch.get_default_dtype()
    if isinstance(start, torch.Tensor):
        start = start.item()
    if isinstance(end, torch.Tensor):
        end = end.item()

    def fill(t):
        t.copy_(torch.linspace(start, end, int(steps), dtype=t.dtype if t.dtype.is_floating_point or t.dtype.is_complex else torch.float64, device=t.device))

    return _materialise(heap, iris_device, (int(steps),), fill, out=out, dtype=dtype, layout=layout, device=device,
                        requires_grad=requires_grad)
