"""Helpers around the framework proper: result validation, result records, timing, roofline arithmetic."""
from .records import JSONWriter, TileTimeline, torch_dtype_from_str, torch_dtype_to_str  # noqa: F401
from .roofline import (Peaks, attention_flops, collective_link_bytes, compute_fraction, fused_target_seconds,  # noqa: F401
                       gemm_flops, load_peaks, memory_fraction)
from .validation import (validate_all_gather, validate_all_reduce, validate_all_scatter, validate_gemm,  # noqa: F401
                         validate_reduce_scatter)
from .timing import time_max_over_ranks  # noqa: F401
