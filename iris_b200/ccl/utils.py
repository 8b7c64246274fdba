"""Reduction operators and group helpers of the collectives (reference: iris/ccl/utils.py:44-78)."""
from __future__ import annotations

from enum import IntEnum


class ReduceOp(IntEnum):
    SUM = 0
    PRODUCT = 1
    MIN = 2
    MAX = 3
    BAND = 4
    BOR = 5
    BXOR = 6
