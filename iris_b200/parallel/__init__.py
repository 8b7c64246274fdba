"""Parallelism strategies as objects: who talks to whom, and the layers built on that.

================  =============================================================================
tensor parallel   ``ColumnParallelLinear``, ``RowParallelLinear``, ``TensorParallelMLP`` on the fused
                  GEMM + collective kernels (``tensor_parallel``)
data parallel     ``GradientBuckets``: bucketed gradient all-reduce that overlaps backward
                  (``data_parallel``)
sequence/context  ``shard_sequence`` / ``unshard_sequence`` / ``sequence_positions`` for ring attention,
                  ``UlyssesExchange`` head <-> sequence swap over all_to_all (``sequence_parallel``);
                  ``RingAttention`` and ``FlashDecodeLayer`` themselves live in ``iris_b200.models``
expert parallel   ownership and dispatch tables (``expert_parallel``); ``MoELayer`` in ``iris_b200.models``
layout            ``ParallelLayout``: named dimensions over the ranks and their process groups
pipeline          ``P2PChannel``: send / receive between stages (``put`` + release flag, acknowledgements
                  for back-pressure) (``p2p``); schedules are left to the caller, the reference has no
                  pipeline parallelism
================  =============================================================================
"""
from .data_parallel import GradientBuckets  # noqa: F401
from .expert_parallel import (DispatchTables, ExpertAssignment, RaggedSlices, TopkResult, dispatch_tables,  # noqa: F401
                              expert_assignment, ragged_slices, topk_routing, uniform_expert_dict)
from .layout import ParallelLayout  # noqa: F401
from .p2p import P2PChannel  # noqa: F401
from .sequence_parallel import UlyssesExchange, sequence_positions, shard_sequence, unshard_sequence  # noqa: F401
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP  # noqa: F401
