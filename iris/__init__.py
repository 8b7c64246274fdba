"""``import iris`` for code written against the reference's package name.

Everything here is ``iris_b200``: the same module objects are registered under ``iris.<name>``, so
``import iris``, ``from iris import ccl``, ``import iris.ops`` and ``iris.iris(heap_size)`` resolve to
this framework (name list of the reference: iris/__init__.py:45-136, iris/ccl/__init__.py:13-16,
iris/gluon.py:12-13). ``bench.py --impl reference`` puts the unmodified reference's own directory in
front of this one on ``sys.path``, so that arm never sees this alias.
"""
from __future__ import annotations

import importlib
import sys

import iris_b200 as _impl
from iris_b200 import *  # noqa: F401,F403
from iris_b200 import __all__ as _names, __version__  # noqa: F401

for _sub in ("ccl", "ops", "bench", "experimental", "gluon", "mem", "device", "host", "models", "parallel", "utils",
             "jit", "drivers"):
    _mod = importlib.import_module("iris_b200." + _sub)
    sys.modules[__name__ + "." + _sub] = _mod
    globals()[_sub] = _mod

hip = _impl.hip
tensor_creation = _impl.tensor_creation
sys.modules[__name__ + ".hip"] = hip
sys.modules[__name__ + ".tensor_creation"] = tensor_creation

__all__ = list(_names)
