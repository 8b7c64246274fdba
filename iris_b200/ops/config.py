"""Configuration of the fused GEMM + collective ops (reference: iris/ops/config.py:13-104).

The reference's tile sizes drive a Triton kernel; here the GEMM tile is fixed at 128 rows by the
tcgen05 instruction shape and ``block_size_n`` selects the tile width (128, 224 or 256; anything
else means "choose by wave count"). ``block_size_m`` / ``block_size_k`` are validated and kept for
API compatibility.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class FusedConfig:
    block_size_m: int = 128
    block_size_n: int = 0
    block_size_k: int = 64
    group_size_m: int = 8
    num_sms: int | None = None
    num_xcds: int = 1
    chunk_size: int = 1
    all_reduce_variant: str = "auto"        # matmul_all_reduce: two_shot, one_shot, atomic, or auto (by output size)
    all_reduce_num_rings: int = 1
    comm_sms: int = 0
    use_multicast: bool = True
    two_sm: bool | None = None      # CTA pairs on 256-row tiles (tcgen05 cta_group::2); None = the plan decides
    # matmul_all_gather (GEMM + all-gather / all-scatter): how the collective overlaps the GEMM, after the
    # reference's taxonomy (docs/conceptual/taxonomy.md; examples 07, 10, 11, 12):
    #   "fused"             every epilogue warp stores its fragment to all ranks (fused sequential, example 07)
    #   "wg_specialized"    comm_sms communication CTAs of the same kernel forward finished tiles (example 10;
    #                       also what stands in for the two-kernel producer / consumer of example 11 here)
    #   "bulk_synchronous"  GEMM kernel, then the all-gather kernel (example 12)
    overlap: str = "fused"
    allow_tf32: bool = True

    def __post_init__(self):
        if self.block_size_m <= 0 or self.block_size_k <= 0 or self.block_size_n < 0:
            raise ValueError("block sizes must be positive")
        if self.group_size_m <= 0:
            raise ValueError("group_size_m must be positive")
        if self.overlap not in ("fused", "wg_specialized", "producer_consumer", "bulk_synchronous"):
            raise ValueError(f"unknown overlap pattern {self.overlap!r}")
        if self.all_reduce_variant not in ("atomic", "ring", "one_shot", "two_shot", "spinlock", "auto"):
            raise ValueError(f"unknown all_reduce_variant {self.all_reduce_variant!r}")

    def validate(self, world_size: int | None = None) -> None:
        if world_size is not None and world_size <= 0:
            raise ValueError("world_size must be positive")

    def tile_n(self) -> int:
        return self.block_size_n if self.block_size_n in (128, 224, 256) else 0
