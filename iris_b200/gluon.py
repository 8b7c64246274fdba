"""Names of the reference's Gluon device API (iris/gluon.py: ``IrisDeviceCtx``, ``GluonDeviceTracing``).

Gluon exists in the reference to give Triton kernels explicit layouts and vector widths; CUDA C++
has both natively, so the Gluon and the Triton flavours of the device API are one header library
here. The two names point at the same symbols as ``iris_b200.DeviceContext`` / ``Context`` and the
tracing aggregate."""
from .device import Context as IrisDeviceCtx  # noqa: F401
from .device import Tracing as GluonDeviceTracing  # noqa: F401

__all__ = ["IrisDeviceCtx", "GluonDeviceTracing"]
