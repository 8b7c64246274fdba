"""Small record keepers used by examples and benchmarks: a JSON result file, dtype names, and the
per-tile timeline of a fused GEMM + collective kernel.

Counterparts in the reference: ``JSONWriter``, ``Timestamps`` and the dtype helpers of
examples/common/utils.py:31-149. Its ``Timestamps`` holds GPU cycle counters that the example
kernels fill with ``atomic_min / atomic_max`` per tile and converts them with a clock rate; here the
fused kernels stamp nanoseconds of the global timer, one row per output tile, so no rate is needed.
"""
from __future__ import annotations

import json
import os

import torch

_DTYPES = {"fp16": torch.float16, "float16": torch.float16, "half": torch.float16, "bf16": torch.bfloat16,
           "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32, "float": torch.float32,
           "fp64": torch.float64, "float64": torch.float64, "int8": torch.int8, "int32": torch.int32, "int64": torch.int64}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES.update({"fp8": torch.float8_e4m3fn, "float8_e4m3fn": torch.float8_e4m3fn})


def torch_dtype_from_str(name: str) -> torch.dtype:
    try:
        return _DTYPES[name.lower().replace("torch.", "")]
    except KeyError:
        raise ValueError(f"unknown datatype {name!r}; known: {', '.join(sorted(_DTYPES))}") from None


def torch_dtype_to_str(dtype: torch.dtype) -> str:
    return str(dtype).replace("torch.", "")


class JSONWriter:
    """Accumulate fields and keep the file on disk in step with them (one flat JSON object)."""

    def __init__(self, file_path: str):
        self.file_path = file_path
        self.data: dict = {}
        if os.path.exists(file_path):
            os.remove(file_path)

    def add_field(self, key: str, value) -> None:
        if isinstance(value, torch.Tensor):
            value = value.item() if value.numel() == 1 else value.tolist()
        elif isinstance(value, torch.dtype):
            value = torch_dtype_to_str(value)
        self.data[key] = value

    def flush(self) -> None:
        tmp = self.file_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=4)
        os.replace(tmp, self.file_path)

    def display(self) -> None:
        print(json.dumps(self.data, indent=4))


class TileTimeline:
    """Per-tile timestamps of one fused-op launch.

    The fused kernels write, for output tile ``t``, nanosecond stamps into row ``t`` of an int64
    ``[tiles + chunks, 4]`` table: column 0 when the tile's main loop starts, 1 when its first
    operands have arrived (for all-gather + GEMM this includes the wait for the peer's chunk),
    2 when the tile has been stored (for GEMM + reduce: handed to the reduction). The first
    communication CTA stamps column 3 of row ``tiles + c`` when chunk ``c`` has been pushed. Attach
    with ``workspace.extra["timeline"] = timeline.table`` before the launch.
    """

    COLUMNS = ("begin", "operands_ready", "end", "chunk_sent")

    def __init__(self, num_tiles: int, num_chunks: int = 0, device=None):
        self.num_tiles, self.num_chunks = int(num_tiles), int(num_chunks)
        self.table = torch.zeros((self.num_tiles + self.num_chunks, 4), dtype=torch.int64, device=device)

    def reset(self) -> None:
        self.table.zero_()

    def rows(self) -> dict:
        """Stamps re-based to the earliest one, in nanoseconds; tiles that were never stamped are left out."""
        t = self.table.cpu()
        stamped = t[t > 0]
        origin = int(stamped.min()) if stamped.numel() else 0
        tiles = []
        for i in range(self.num_tiles):
            b, r, e = (int(v) for v in t[i, :3])
            if b == 0 and e == 0:
                continue
            tiles.append({"tile_id": i, "begin": b - origin, "operands_ready": (r - origin) if r else None,
                          "end": (e - origin) if e else None})
        chunks = [{"chunk": c, "sent": int(t[self.num_tiles + c, 3]) - origin} for c in range(self.num_chunks)
                  if int(t[self.num_tiles + c, 3])]
        return {"unit": "ns", "tiles": tiles, "chunks": chunks}

    def summary(self) -> dict:
        """Span of the launch, mean tile duration and mean wait for operands (ns)."""
        r = self.rows()
        done = [x for x in r["tiles"] if x["end"] is not None]
        if not done:
            return {"tiles": 0}
        waits = [x["operands_ready"] - x["begin"] for x in done if x["operands_ready"] is not None]
        return {"tiles": len(done), "span_ns": max(x["end"] for x in done) - min(x["begin"] for x in done),
                "mean_tile_ns": sum(x["end"] - x["begin"] for x in done) / len(done),
                "mean_operand_wait_ns": (sum(waits) / len(waits)) if waits else None,
                "last_chunk_sent_ns": max((c["sent"] for c in r["chunks"]), default=None)}

    def to_json(self, filename: str) -> None:
        with open(filename, "w") as f:
            json.dump(self.rows(), f, indent=2)
