"""Model-level building blocks built on the heap, the collectives and the fused ops:
distributed flash-decode, expert-sharded MoE, ring attention, tensor-parallel MLP."""
from .flash_decode import FlashDecodeLayer, merge_partials, reference_decode  # noqa: F401
from .moe import MoELayer, fuse_gate_up, reference_moe, route  # noqa: F401
from .ring_attention import RingAttention, reference_attention, zigzag_positions  # noqa: F401
from .tp_mlp import TensorParallelMLP  # noqa: F401
