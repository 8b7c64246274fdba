"""Experimental features (reference: iris/experimental/__init__.py, whose only entry is the Gluon
device context). Kept as a namespace with the same entry: ``gluon_context`` is the module that holds
``IrisDeviceCtx``; on this backend it names the one CUDA C++ device API."""
from .. import gluon as gluon_context  # noqa: F401

__all__ = ["gluon_context"]
