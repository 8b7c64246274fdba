"""Configuration of the collectives.

Field names follow the reference dataclass (iris/ccl/config.py:13-150) so that call sites carry
over. Knobs that only exist on AMD hardware (``num_xcds``, ``waves_per_eu``, ``use_gluon``,
``threads_per_warp``, ``num_stages``, ``num_warps``) are accepted and ignored. New here:
``all_reduce_variant="auto"`` (choice by message size) and ``"nvls"``, ``use_multicast``.
"""
from __future__ import annotations

from dataclasses import dataclass

ALL_REDUCE_VARIANTS = ("auto", "atomic", "ring", "two_shot", "one_shot", "spinlock", "nvls", "push")
ALL_GATHER_VARIANTS = ("persistent", "partitioned")


@dataclass
class Config:
    block_size_m: int = 32
    block_size_n: int = 64
    swizzle_size: int = 4
    comm_sms: int = 64
    num_xcds: int | None = None
    chunk_size: int | None = None
    use_gluon: bool = False
    all_gather_variant: str = "persistent"
    all_reduce_variant: str = "auto"
    all_reduce_distribution: int = 1
    all_reduce_num_rings: int = 1
    all_reduce_ring_slice_n: int | None = None
    reduce_scatter_variant: str = "two_shot"
    reduce_scatter_rows: bool = False
    use_multicast: bool = True
    num_stages: int = 1
    num_warps: int = 4
    threads_per_warp: int = 32
    waves_per_eu: int = 0

    def __post_init__(self):
        if self.block_size_m <= 0 or self.block_size_n <= 0:
            raise ValueError(f"block sizes must be positive, got {self.block_size_m}x{self.block_size_n}")
        if self.swizzle_size <= 0:
            raise ValueError(f"swizzle_size must be positive, got {self.swizzle_size}")
        if self.comm_sms <= 0:
            raise ValueError(f"comm_sms must be positive, got {self.comm_sms}")
        if self.all_gather_variant not in ALL_GATHER_VARIANTS:
            raise ValueError(f"all_gather_variant must be one of {ALL_GATHER_VARIANTS}, got {self.all_gather_variant!r}")
        if self.all_reduce_variant not in ALL_REDUCE_VARIANTS:
            raise ValueError(f"all_reduce_variant must be one of {ALL_REDUCE_VARIANTS}, got {self.all_reduce_variant!r}")
        if self.all_reduce_distribution not in (0, 1):
            raise ValueError("all_reduce_distribution must be 0 (strided) or 1 (block)")
        if self.all_reduce_num_rings <= 0:
            raise ValueError("all_reduce_num_rings must be positive")
        if self.reduce_scatter_variant != "two_shot":
            raise ValueError("reduce_scatter_variant must be 'two_shot'")
        if self.threads_per_warp not in (32, 64):
            raise ValueError("threads_per_warp must be 32 or 64")
