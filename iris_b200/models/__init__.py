"""Model-level building blocks built on the heap, the collectives and the fused ops:
distributed flash-decode, expert-sharded MoE, ring attention, tensor-parallel MLP."""
from .flash_decode import FlashDecodeLayer, merge_partials, reference_decode  # noqa: F401
