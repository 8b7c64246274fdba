"""Rank-aware logging.

Lines look like ``HH:MM:SS LEVEL [Iris] [rank/world] [module] message``; the level comes from
``IRIS_LOG_LEVEL`` (reference: iris/host/logging/logging.py:19-92).
"""
from __future__ import annotations

import logging
import os

DEBUG, INFO, WARNING, ERROR = logging.DEBUG, logging.INFO, logging.WARNING, logging.ERROR


class IrisFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        stamp = self.formatTime(record, "%H:%M:%S")
        rank = getattr(record, "iris_rank", None)
        world = getattr(record, "iris_num_ranks", None)
        where = f" [{rank}/{world}]" if rank is not None and world is not None else ""
        module = getattr(record, "iris_module", None) or record.module
        return f"{stamp} {record.levelname:<7} [Iris]{where} [{module}] {record.getMessage()}"


logger = logging.getLogger("iris")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(IrisFormatter())
    logger.addHandler(_h)
    logger.propagate = False
    _lvl = os.environ.get("IRIS_LOG_LEVEL", "WARNING").upper()
    logger.setLevel(getattr(logging, _lvl, logging.WARNING))


def set_logger_level(level: int) -> None:
    """Set the level of the ``iris`` logger (``iris.DEBUG`` ... ``iris.ERROR``)."""
    logger.setLevel(level)


def log_rank(level: int, message: str, rank: int | None, num_ranks: int | None, module: str | None = None) -> None:
    """Emit one record tagged with the rank that produced it."""
    if logger.isEnabledFor(level):
        logger.log(level, message, extra={"iris_rank": rank, "iris_num_ranks": num_ranks, "iris_module": module})
