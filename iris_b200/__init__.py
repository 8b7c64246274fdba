"""iris_b200: a Blackwell-native symmetric-memory multi-GPU framework.

Same programming model and public surface as Iris (``import iris_b200 as iris``): a context created
with ``iris.iris(heap_size)`` owns a symmetric heap mapped into every rank of the NVLink domain;
tensors come from ``ctx.zeros`` & co.; device code reaches a peer's copy of any heap object with
one address translation (``include/iris/iris.cuh``); ``ctx.ccl`` holds the collectives and
``ctx.ops`` the fused GEMM + collective kernels. Device code is CUDA C++ for sm_100a
(tcgen05 / TMEM / TMA, NVLS multimem) instead of Triton.
"""
from __future__ import annotations

from .host.logging import DEBUG, ERROR, INFO, WARNING, logger, set_logger_level
from .host.iris import Iris, IrisTimeoutError, iris
from .host.watchdog import BarrierTimeoutError
from .host.tensor_utils import CUDAArrayInterface, tensor_from_ptr
from .host.platform import do_bench, get_device_id_for_rank, is_simulation_env
from .host import platform as hip
from .host import tensors as tensor_creation
from .host.tracing import TraceEvent
from . import ccl
from . import ops
from . import bench
from . import experimental
from . import gluon  # noqa: F401
from . import mem  # noqa: F401
from .device import (DeviceContext, Context, Tile, TileView, TensorView, AllReduceConfig, make_tensor_view,
                     load, store, copy, get, put, atomic_add, atomic_cas, atomic_xchg, atomic_xor, atomic_or, atomic_and,
                     atomic_min, atomic_max)

__version__ = "0.1.0"

__all__ = [
    "Iris", "iris", "IrisTimeoutError", "BarrierTimeoutError", "DeviceContext", "Context", "TraceEvent", "Tile", "TileView", "TensorView",
    "AllReduceConfig", "make_tensor_view", "load", "store", "copy", "get", "put", "atomic_add", "atomic_cas",
    "atomic_xchg", "atomic_xor", "atomic_or", "atomic_and", "atomic_min", "atomic_max", "do_bench",
    "get_device_id_for_rank", "is_simulation_env", "CUDAArrayInterface", "tensor_from_ptr", "hip", "experimental",
    "ops", "ccl", "tensor_creation", "bench", "set_logger_level", "logger", "DEBUG", "INFO", "WARNING", "ERROR",
]
