"""Device event tracing: host-side manager and exporter.

``ctx.tracing.enable(max_events)`` allocates thirteen structure-of-arrays buffers plus two
counters on the device and rebuilds the device context so that kernels compiled with tracing see
them; ``export(filename, merge)`` writes one Chrome/Perfetto JSON per rank and optionally a merged
file on rank 0 with timestamps re-based to the global minimum. Field set, event ids and file layout
follow the reference (iris/host/tracing/core.py:19-333, events.py:18-99); timestamps here are
``%globaltimer`` nanoseconds and the track name is ``SM<n>``.
"""
from __future__ import annotations

import json
import pickle

import torch
import torch.distributed as dist

EVENT_NAMES = {
    0: "load", 1: "store", 2: "get", 3: "put", 4: "copy", 5: "atomic_add", 6: "atomic_sub", 7: "atomic_cas",
    8: "atomic_xchg", 9: "atomic_xor", 10: "atomic_and", 11: "atomic_or", 12: "atomic_min", 13: "atomic_max",
}


class TraceEvent:
    """Event ids usable as ``TraceEvent().put`` (same numbering on the device, tracing.cuh)."""

    load, store, get, put, copy = 0, 1, 2, 3, 4
    atomic_add, atomic_sub, atomic_cas, atomic_xchg = 5, 6, 7, 8
    atomic_xor, atomic_and, atomic_or, atomic_min, atomic_max = 9, 10, 11, 12, 13


_INT32_FIELDS = ["event_id", "pid", "pid_m", "pid_n", "cur_rank", "target_rank", "xcc_id", "cu_id"]
_INT64_FIELDS = ["timestamp", "address", "duration_cycles"]
_TAIL_FIELDS = ["op_index", "payload_size"]
FIELD_ORDER = _INT32_FIELDS + _INT64_FIELDS + _TAIL_FIELDS


class Tracing:
    def __init__(self, ctx):
        self.ctx = ctx
        self.enabled = False
        self.max_events = 0
        self.buffers: dict[str, torch.Tensor] = {}
        self.counter = None
        self.op_index_counter = None

    def context_words(self) -> list[int]:
        """The 17 trailing int64 words of the device context tensor (zeros when tracing is off)."""
        if not self.enabled:
            return [0] * 17
        words = [1, self.max_events, self.counter.data_ptr(), self.op_index_counter.data_ptr()]
        words += [self.buffers[f].data_ptr() for f in FIELD_ORDER]
        return words

    def enable(self, max_events: int = 1_000_000) -> None:
        dev = self.ctx.device
        self.max_events = int(max_events)
        self.buffers = {}
        for f in _INT32_FIELDS + _TAIL_FIELDS:
            self.buffers[f] = torch.zeros(self.max_events, dtype=torch.int32, device=dev)
        for f in _INT64_FIELDS:
            self.buffers[f] = torch.zeros(self.max_events, dtype=torch.int64, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.op_index_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.enabled = True
        self.ctx._build_device_context()

    def reset(self) -> None:
        if self.enabled:
            self.counter.zero_()
            self.op_index_counter.zero_()

    def num_events(self) -> int:
        if not self.enabled:
            return 0
        return min(int(self.counter.item()), self.max_events)

    def _events(self) -> list[dict]:
        n = self.num_events()
        cols = {f: self.buffers[f][:n].cpu().tolist() for f in FIELD_ORDER}
        out = []
        for i in range(n):
            ts, end = cols["timestamp"][i], cols["duration_cycles"][i]
            name = EVENT_NAMES.get(cols["event_id"][i], f"event_{cols['event_id'][i]}")
            ev = {
                "name": name, "cat": "iris", "pid": cols["cur_rank"][i], "tid": f"SM{cols['cu_id'][i]}",
                "ts": ts / 1000.0,
                "args": {
                    "target_rank": cols["target_rank"][i], "address": hex(cols["address"][i] & (2**64 - 1)),
                    "pid": cols["pid"][i], "pid_m": cols["pid_m"][i], "pid_n": cols["pid_n"][i],
                    "op_index": cols["op_index"][i], "payload_size": cols["payload_size"][i], "timestamp_ns": ts,
                },
            }
            if end and end >= ts:
                ev["ph"], ev["dur"] = "X", (end - ts) / 1000.0
            else:
                ev["ph"], ev["s"] = "i", "t"
            out.append(ev)
        return out

    def export(self, filename: str = "trace.json", merge: bool = False) -> None:
        """Write ``<stem>_rank<r>.json`` on every rank; with ``merge`` also ``filename`` on rank 0."""
        if not self.enabled:
            raise RuntimeError("tracing is not enabled")
        if not self.ctx.is_cpu:
            torch.cuda.synchronize(self.ctx.device)
        events = self._events()
        rank, world = self.ctx.cur_rank, self.ctx.num_ranks
        stem = filename[:-5] if filename.endswith(".json") else filename
        doc = {"traceEvents": events, "displayTimeUnit": "ns", "metadata": {"rank": rank, "num_ranks": world, "time_unit": "ns"}}
        with open(f"{stem}_rank{rank}.json", "w") as f:
            json.dump(doc, f)
        if not merge:
            return
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, pickle.dumps(events))
            gathered = [pickle.loads(g) for g in gathered]
        else:
            gathered = [events]
        if rank == 0:
            merged = [e for evs in gathered for e in evs]
            if merged:
                t0 = min(e["ts"] for e in merged)
                for e in merged:
                    e["ts"] -= t0
            with open(filename, "w") as f:
                json.dump({"traceEvents": merged, "displayTimeUnit": "ns", "metadata": {"num_ranks": world, "time_unit": "ns"}}, f)
        if world > 1:
            dist.barrier()
