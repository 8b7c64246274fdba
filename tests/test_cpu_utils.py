"""iris_b200.utils on the CPU: result records, roofline arithmetic, validation helpers (gloo ranks).

The reference's counterparts (examples/common/utils.py, validation.py) have no tests of their own;
they are exercised through the example harnesses.
"""
import json

import pytest
import torch

from helpers import run_ranks


def test_json_writer_and_dtype_names(tmp_path, capsys):
    from iris_b200.utils import JSONWriter, torch_dtype_from_str, torch_dtype_to_str

    path = tmp_path / "log.json"
    path.write_text("stale")
    w = JSONWriter(str(path))
    assert not path.exists()                       # a new writer starts from a clean file
    w.add_field("tflops", 1234.5)
    w.add_field("dtype", torch.bfloat16)
    w.add_field("loss", torch.tensor(0.25))
    w.add_field("shape", torch.tensor([8192, 4608]))
    w.add_field("success", True)
    w.flush()
    assert json.loads(path.read_text()) == {"tflops": 1234.5, "dtype": "bfloat16", "loss": 0.25, "shape": [8192, 4608], "success": True}
    w.add_field("tflops", 1300.0)
    w.flush()
    assert json.loads(path.read_text())["tflops"] == 1300.0
    w.display()
    assert '"tflops": 1300.0' in capsys.readouterr().out
    for name, dt in (("fp16", torch.float16), ("bf16", torch.bfloat16), ("fp32", torch.float32), ("torch.float16", torch.float16),
                     ("BFLOAT16", torch.bfloat16), ("int8", torch.int8)):
        assert torch_dtype_from_str(name) == dt
    assert torch_dtype_to_str(torch.float16) == "float16" and torch_dtype_from_str(torch_dtype_to_str(torch.int32)) == torch.int32
    with pytest.raises(ValueError):
        torch_dtype_from_str("fp12")


def test_tile_timeline(tmp_path):
    from iris_b200.utils import TileTimeline

    tl = TileTimeline(num_tiles=4, num_chunks=2)
    assert tl.table.shape == (6, 4) and tl.table.dtype == torch.int64
    assert tl.rows() == {"unit": "ns", "tiles": [], "chunks": []} and tl.summary() == {"tiles": 0}
    base = 1_000_000_000
    tl.table[0, :3] = torch.tensor([base + 100, base + 150, base + 400])
    tl.table[1, :3] = torch.tensor([base + 120, base + 300, base + 620])
    tl.table[3, :3] = torch.tensor([base + 500, 0, base + 900])     # operands stamp missing
    tl.table[4, 3] = base + 50                                      # chunk 0 sent first of all
    tl.table[5, 3] = base + 250
    r = tl.rows()
    assert [t["tile_id"] for t in r["tiles"]] == [0, 1, 3]          # tile 2 never ran
    assert r["tiles"][0] == {"tile_id": 0, "begin": 50, "operands_ready": 100, "end": 350}
    assert r["tiles"][2]["operands_ready"] is None
    assert r["chunks"] == [{"chunk": 0, "sent": 0}, {"chunk": 1, "sent": 200}]
    s = tl.summary()
    assert s["tiles"] == 3 and s["span_ns"] == 800 and s["mean_tile_ns"] == pytest.approx((300 + 500 + 400) / 3)
    assert s["mean_operand_wait_ns"] == pytest.approx((50 + 180) / 2) and s["last_chunk_sent_ns"] == 200
    out = tmp_path / "timeline.json"
    tl.to_json(str(out))
    assert json.loads(out.read_text()) == r
    tl.reset()
    assert int(tl.table.abs().sum()) == 0


def test_roofline_arithmetic(tmp_path, monkeypatch):
    from iris_b200.utils import (attention_flops, collective_link_bytes, compute_fraction, fused_target_seconds, gemm_flops, load_peaks,
                                 memory_fraction)
    from iris_b200.utils.roofline import FALLBACK, Peaks

    f = tmp_path / "peaks.json"
    f.write_text(json.dumps({"hbm_gbs": 6000.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0}))
    p = load_peaks(f)
    assert (p.hbm_gbs, p.bf16_tflops, p.bf16_tflops_sustained) == (6000.0, 1600.0, 1400.0) and p.label == "of measured"
    monkeypatch.setenv("IRIS_PEAKS_FILE", str(f))
    assert load_peaks().source == str(f)
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    assert load_peaks(bad).source == str(f)                        # unreadable file: next candidate
    fb = Peaks(**FALLBACK)
    assert fb.label == "of fallback"
    assert gemm_flops(8192, 4608, 36864) == 2 * 8192 * 4608 * 36864
    assert attention_flops(1024, 1024, 8, 128) == 4 * 1024 * 1024 * 8 * 128
    assert attention_flops(1024, 1024, 8, 128, causal=True) == attention_flops(1024, 1024, 8, 128) / 2
    assert compute_fraction(1600e12, 1.0, p) == pytest.approx(1.0) and compute_fraction(1400e12, 1.0, p, sustained=True) == pytest.approx(1.0)
    assert memory_fraction(3000e9, 1.0, p) == pytest.approx(0.5)
    # compute bound and link bound cases of a fused op
    assert fused_target_seconds(1400e12, 1e9, p) == pytest.approx(1.0)
    assert fused_target_seconds(1e12, 770e9, p) == pytest.approx(1.0)
    assert collective_link_bytes("all_reduce", 1e9, 8) == pytest.approx(2 * 7 / 8 * 1e9)
    assert collective_link_bytes("all_reduce_nvls", 1e9, 8) == 1e9
    assert collective_link_bytes("all_gather", 1e9, 4) == pytest.approx(0.75e9)
    assert collective_link_bytes("all_to_all", 1e9, 1) == 0.0
    with pytest.raises(ValueError):
        collective_link_bytes("broadcast", 1.0, 2)


def _validation(rank, world):
    import iris_b200 as iris
    from iris_b200.utils import validate_all_gather, validate_all_reduce, validate_all_scatter, validate_gemm, validate_reduce_scatter

    ctx = iris.iris(1 << 24)
    g = torch.Generator().manual_seed(3)
    A, B = torch.randn(8, 16, generator=g), torch.randn(16, 12, generator=g)
    bias = torch.randn(12, generator=g)
    C = A @ B
    assert validate_gemm(A, B, C, ctx, atol=1e-5)
    assert validate_gemm(A, B, C + bias, ctx, atol=1e-5, bias=bias)
    wrong = C.clone()
    wrong[3, 4] += 5.0
    assert not validate_gemm(A, B, wrong, ctx, atol=1e-3)
    local = torch.full((4, 6), float(rank + 1))
    cols = torch.cat([torch.full((4, 6), float(r + 1)) for r in range(world)], dim=1)
    rows = torch.cat([torch.full((4, 6), float(r + 1)) for r in range(world)], dim=0)
    assert validate_all_scatter(local, cols, ctx, atol=0.0)
    assert validate_all_gather(local, rows, ctx)
    assert not validate_all_scatter(local, cols.flip(1) if world > 1 else cols + 1, ctx, atol=0.0)
    assert not validate_all_gather(local, rows + 1, ctx)
    total = torch.full((4, 6), float(sum(range(1, world + 1))))
    assert validate_all_reduce(local, total, ctx, atol=0.0)
    assert not validate_all_reduce(local, total - 1, ctx, atol=0.5)
    big = (torch.arange(4 * world * 6, dtype=torch.float32).view(4 * world, 6) + rank)
    summed = sum(torch.arange(4 * world * 6, dtype=torch.float32).view(4 * world, 6) + r for r in range(world))
    assert validate_reduce_scatter(big, summed[rank * 4:(rank + 1) * 4], ctx, atol=0.0)
    assert not validate_reduce_scatter(big, summed[((rank + 1) % world) * 4:((rank + 1) % world + 1) * 4] + 1000, ctx, atol=0.0)
    # results produced by the library pass the same checks
    inp = ctx.full((4, 6), float(rank + 1))
    out = ctx.zeros((4, 6))
    ctx.ccl.all_reduce(out, inp)
    assert validate_all_reduce(inp, out, ctx, atol=0.0)
    ag = ctx.zeros((4 * world, 6))
    ctx.ccl.all_gather(ag, inp)
    assert validate_all_gather(inp, ag, ctx)
    ctx.barrier()


def test_validation_helpers_world2(capfd):
    run_ranks(_validation, 2)


def test_validation_helpers_world1():
    run_ranks(_validation, 1)
