"""Workspace of a fused op: the heap buffers its kernel needs besides the operands
(reference: iris/ops/workspace.py:14-85). Created by the ``*_preamble`` functions, reusable across
calls with the same shapes; buffers are double-buffered by call parity inside the kernels, so no
reset between calls is needed."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class FusedWorkspace:
    operation: str = ""
    shape: tuple = ()
    dtype: torch.dtype | None = None
    world_size: int = 1
    variant: str = ""
    sync_block: torch.Tensor | None = None
    inbox: torch.Tensor | None = None        # all_gather_matmul: gathered A, [2][W][rows][cols]
    flags: torch.Tensor | None = None        # arrival counters
    staging: torch.Tensor | None = None      # reduce ops: partial tiles, [2][W][owned][128*bn]
    aux_buffer: torch.Tensor | None = None   # name used by the reference for the same purpose
    locks: torch.Tensor | None = None
    bn: int = 0
    prepared: bool = False
    extra: dict = field(default_factory=dict)

    def matches(self, operation, shape, dtype, world_size, variant="") -> bool:
        return (self.operation == operation and self.shape == tuple(shape) and self.dtype == dtype
                and self.world_size == world_size and self.variant == variant)
