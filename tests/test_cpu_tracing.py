"""Host side of device event tracing on gloo ranks: buffers, context words, Chrome-trace export.

The reference's tests reach tracing only through traced kernels on GPUs
(tests/unittests/test_device_context*.py); the manager itself (iris/host/tracing/core.py:39-333) is
plain host code. Here the buffers a kernel would fill are filled by hand and the exported files are
read back.
"""
import json

import pytest
import torch

from helpers import run_ranks


def _tracing(rank, world, outdir):
    import iris_b200 as iris
    from iris_b200.host.tracing import EVENT_NAMES, FIELD_ORDER

    ctx = iris.iris(1 << 24)
    tr = ctx.tracing
    # off: the trailing 17 words of the context tensor are zero, export is refused
    dc = ctx.get_device_context()
    assert dc.numel() == 2 + world + 17 and torch.all(dc[2 + world:] == 0)
    assert tr.num_events() == 0
    with pytest.raises(RuntimeError):
        tr.export(f"{outdir}/never.json")
    # event ids: the reference's numbering
    ev = iris.TraceEvent()
    assert (ev.load, ev.store, ev.get, ev.put, ev.copy, ev.atomic_add, ev.atomic_cas, ev.atomic_max) == (0, 1, 2, 3, 4, 5, 7, 13)
    assert len(EVENT_NAMES) == 14 and EVENT_NAMES[3] == "put"
    assert FIELD_ORDER == ["event_id", "pid", "pid_m", "pid_n", "cur_rank", "target_rank", "xcc_id", "cu_id", "timestamp", "address",
                           "duration_cycles", "op_index", "payload_size"]

    tr.enable(max_events=8)
    dc = ctx.get_device_context()                       # rebuilt: kernels see the buffers through it
    tail = dc[2 + world:].tolist()
    assert tail[0] == 1 and tail[1] == 8 and tail[2] == tr.counter.data_ptr() and tail[3] == tr.op_index_counter.data_ptr()
    assert tail[4:] == [tr.buffers[f].data_ptr() for f in FIELD_ORDER]
    assert int(dc[0]) == rank and int(dc[1]) == world
    for f in FIELD_ORDER:
        want = torch.int64 if f in ("timestamp", "address", "duration_cycles") else torch.int32
        assert tr.buffers[f].dtype == want and tr.buffers[f].numel() == 8
    cs = ctx.ctx_struct()
    assert cs.trace_enabled == 1 and cs.trace_max_events == 8

    # what a traced kernel leaves behind: three events, the second one instantaneous
    base = 5_000_000 + 1000 * rank
    rows = [dict(event_id=3, pid=0, pid_m=1, pid_n=2, cur_rank=rank, target_rank=(rank + 1) % world, xcc_id=0, cu_id=17,
                 timestamp=base, address=0x7F00_0000_1000, duration_cycles=base + 400, op_index=0, payload_size=4096),
            dict(event_id=5, pid=1, pid_m=0, pid_n=0, cur_rank=rank, target_rank=rank, xcc_id=0, cu_id=3,
                 timestamp=base + 100, address=-16, duration_cycles=0, op_index=1, payload_size=4),
            dict(event_id=0, pid=2, pid_m=0, pid_n=1, cur_rank=rank, target_rank=0, xcc_id=0, cu_id=140,
                 timestamp=base + 250, address=0x10, duration_cycles=base + 300, op_index=2, payload_size=512)]
    for i, r in enumerate(rows):
        for f, v in r.items():
            tr.buffers[f][i] = v
    tr.counter.fill_(3)
    assert tr.num_events() == 3
    tr.export(f"{outdir}/trace.json", merge=True)
    doc = json.load(open(f"{outdir}/trace_rank{rank}.json"))
    assert doc["metadata"] == {"rank": rank, "num_ranks": world, "time_unit": "ns"} and doc["displayTimeUnit"] == "ns"
    evs = doc["traceEvents"]
    assert [e["name"] for e in evs] == ["put", "atomic_add", "load"] and all(e["pid"] == rank and e["cat"] == "iris" for e in evs)
    assert evs[0]["ph"] == "X" and evs[0]["dur"] == pytest.approx(0.4) and evs[0]["ts"] == pytest.approx(base / 1000.0)
    assert evs[0]["tid"] == "SM17" and evs[0]["args"]["target_rank"] == (rank + 1) % world
    assert evs[0]["args"]["address"] == hex(0x7F00_0000_1000) and evs[0]["args"]["payload_size"] == 4096
    assert evs[1]["ph"] == "i" and "dur" not in evs[1] and evs[1]["args"]["address"] == hex(2**64 - 16)
    assert evs[2]["args"] == {"target_rank": 0, "address": "0x10", "pid": 2, "pid_m": 0, "pid_n": 1, "op_index": 2,
                              "payload_size": 512, "timestamp_ns": base + 250}
    if rank == 0:
        merged = json.load(open(f"{outdir}/trace.json"))
        assert merged["metadata"]["num_ranks"] == world and len(merged["traceEvents"]) == 3 * world
        assert min(e["ts"] for e in merged["traceEvents"]) == 0.0                     # re-based to the earliest event
        assert sorted({e["pid"] for e in merged["traceEvents"]}) == list(range(world))
        firsts = sorted(e["ts"] for e in merged["traceEvents"] if e["name"] == "put")
        assert firsts == pytest.approx([1.0 * r for r in range(world)])              # ranks keep their relative offsets
    # more events than the buffers hold: the count is clamped
    tr.counter.fill_(100)
    assert tr.num_events() == 8
    tr.reset()
    assert tr.num_events() == 0 and int(tr.op_index_counter.item()) == 0
    tr.export(f"{outdir}/empty.json", merge=True)
    assert json.load(open(f"{outdir}/empty_rank{rank}.json"))["traceEvents"] == []
    # enabling again replaces the buffers and the context words
    tr.enable(max_events=16)
    assert tr.max_events == 16 and ctx.get_device_context()[2 + world + 1] == 16
    assert tr.buffers["timestamp"].numel() == 16
    ctx.barrier()


def test_tracing_manager_and_export_world2(tmp_path):
    run_ranks(_tracing, 2, args=(str(tmp_path),))


def test_tracing_manager_and_export_world1(tmp_path):
    run_ranks(_tracing, 1, args=(str(tmp_path),))
