"""Benchmark harness (decorators + runner); see ``_core`` and ``_runner``."""
from ._core import AxisDef, BenchmarkDef, Result, State, axis, register, power_of_two, linear_range, registry  # noqa: F401
from ._runner import main  # noqa: F401
