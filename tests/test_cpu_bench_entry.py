"""The parts of bench.py that need no GPU: the reference arm's record and the clock summary."""
import importlib.util
import json
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_entry", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_record_and_exits_zero():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                           "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and ("unavailable" in rec or "value" in rec)


def test_clock_summary_prefers_the_timed_window_and_collects_reasons():
    bench = _bench_module()
    s = bench.ClockSampler(0)
    s.source, s.max_mhz, s.stop_flag = "nvml", 1965.0, True

    class _Done:
        def join(self, timeout=None):
            return None

    s.thread = _Done()
    t0 = time.time()
    s.load_from = t0
    s.timed = [t0 + 1.0, t0 + 2.0]
    s.rows = [(t0 + 0.5, 1965.0, 300.0, set()), (t0 + 1.1, 1400.0, 990.0, {"sw_power_cap"}), (t0 + 1.5, 1350.0, 1000.0, {"sw_power_cap"}),
              (t0 + 1.9, 1380.0, 995.0, set()), (t0 + 2.5, 1900.0, 400.0, {"hw_slowdown"})]
    out = s.stop()
    assert out["window"] == "timed region" and out["samples"] == 3
    assert out["sm_mhz"] == 1380.0 and out["sm_max_mhz"] == 1965.0 and out["power_w_max"] == 1000.0
    assert out["reasons"] == ["sw_power_cap"]          # the slowdown sample lies outside the timed region
    # too few samples inside the timed region: the loaded span is used instead
    s.timed = [t0 + 1.05, t0 + 1.2]
    out = s.stop()
    assert out["window"].startswith("warm-up") and out["samples"] == 5 and "hw_slowdown" in out["reasons"]


def test_benchmark_runner_end_to_end_on_the_cpu_backend(tmp_path):
    """The runner spawns one process per rank, sweeps the axes given on the command line and writes
    the formatted results: here one collective on two gloo ranks."""
    out = tmp_path / "ag.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "ccl", "bench_collectives.py"), "--axis_num_ranks=2", "--axis_bytes=4096,8192",
           "--axis_impl=iris", "--axis_dtype=float32", "--benchmark_filter", "all_gather", "--n_warmup", "1", "--n_repeat", "2",
           "--benchmark_format", "json", "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = json.loads(out.read_text())["results"]
    assert [r["params"]["bytes"] for r in res] == ["4096", "8192"]
    assert all(r["benchmark"] == "all_gather" and r["world_size"] == 2 and r["gpu_time_ms"] > 0 and not r["skipped"] for r in res)


def test_serving_shape_all_reduce_benchmark_on_the_cpu_backend(tmp_path):
    """``(tokens, 2880)`` bf16 all-reduce sweep: the library baseline is skipped without NCCL, the
    variants check their result before timing."""
    out = tmp_path / "serving.csv"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "ccl", "bench_all_reduce_serving_shapes.py"), "--axis_num_ranks=2",
           "--axis_tokens=1,64", "--axis_variant=auto,two_shot,nvls", "--n_warmup", "1", "--n_repeat", "2", "--benchmark_format", "csv",
           "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    import csv

    rows = list(csv.DictReader(out.open()))
    assert len(rows) == 2 * 3 * 2                             # impl x variant x tokens
    timed = [r for r in rows if r["skipped"] == "0"]
    assert {(r["impl"], r["variant"]) for r in timed} == {("iris", "auto"), ("iris", "two_shot")}
    assert all(float(r["gpu_time_ms"]) > 0 and float(r["bandwidth_gbps"]) > 0 for r in timed)
    assert all(r["skipped"] == "1" for r in rows if r["impl"] == "nccl" or r["variant"] == "nvls")


def test_sweep_table_from_a_csv(tmp_path, capsys):
    sys.path.insert(0, os.path.join(ROOT, "benchmark", "ccl"))
    try:
        import plot_sweep_results as plot
    finally:
        sys.path.pop(0)
    src = tmp_path / "sweep.csv"
    src.write_text("benchmark,impl,bytes,gpu_time_ms,bandwidth_gbps,skipped\n"
                   "all_reduce,iris,4096,0.010,0.4,0\nall_reduce,nccl,4096,0.020,0.2,0\n"
                   "all_reduce,iris,1024,0.008,0.1,0\nall_reduce,nccl,1024,0.016,0.05,0\n"
                   "all_reduce,iris,16384,0.0,,1\nall_gather,iris,1024,0.004,0.2,0\n")
    rows = plot.load(str(src), {"benchmark": "all_reduce"})
    assert len(rows) == 4                                   # the skipped point and the other benchmark are gone
    xs, names, table = plot.pivot(rows, "bytes", ["impl"], "gpu_time_ms")
    assert xs == ["1024", "4096"] and names == ["iris", "nccl"] and table["nccl"]["4096"] == 0.020
    text = plot.render(xs, names, table, "bytes", "gpu_time_ms", "nccl")
    assert "iris / nccl" in text and text.splitlines()[-1].split()[-1] == "0.500"
    assert plot.main([str(src), "--x", "bytes", "--series", "benchmark,impl", "--y", "bandwidth_gbps"]) == 0
    assert "all_gather/iris" in capsys.readouterr().out
    assert plot.main([str(src), "--x", "nope"]) == 2
    assert plot.main([str(src), "--where", "impl=none"]) == 1
    with pytest.raises(SystemExit):
        plot.main([str(src), "--baseline", "missing"])


def test_performance_gate(tmp_path, capsys):
    sys.path.insert(0, os.path.join(ROOT, "benchmark"))
    try:
        import check_regression as gate
    finally:
        sys.path.pop(0)
    thresholds = json.load(open(os.path.join(ROOT, "benchmark", "dataset", "perf_thresholds.json")))
    assert {r["n_gpus"] for r in thresholds["bench"]} == {1, 2, 4, 8}
    good = tmp_path / "good.json"
    good.write_text("NCCL version banner\n" + json.dumps({"metric": "tflops", "value": 1200.0, "n_gpus": 1}) + "\n"
                    + json.dumps({"impl": "reference", "unavailable": "not installable"}) + "\n")
    slow = tmp_path / "slow.json"
    slow.write_text(json.dumps({"metric": "tflops", "value": 900.0, "n_gpus": 1}) + "\n")
    assert gate.main(["--bench", str(good)]) == 0
    out = capsys.readouterr().out
    assert "ok    bench.py at 1 GPU(s)" in out and out.count("not measured") == 3
    assert gate.main(["--bench", str(good), "--require-all"]) == 1
    assert gate.main(["--bench", str(slow)]) == 1
    assert "FAIL  bench.py at 1 GPU(s) value: 900" in capsys.readouterr().out
    sweep = tmp_path / "sweep.json"
    rows = [{"benchmark": "all_gather_matmul", "params": {"num_ranks": "8", "impl": "iris", "M": "8192"}, "gpu_time_ms": 0.45, "skipped": False},
            {"benchmark": "all_gather_matmul", "params": {"num_ranks": "8", "impl": "nccl", "M": "8192"}, "gpu_time_ms": 0.56, "skipped": False},
            {"benchmark": "matmul_reduce", "params": {"num_ranks": "8", "impl": "iris", "op": "all_reduce", "M": "8192"}, "gpu_time_ms": 0.9, "skipped": False},
            {"benchmark": "matmul_reduce", "params": {"num_ranks": "8", "impl": "iris", "op": "reduce_scatter", "M": "8192"}, "gpu_time_ms": 0.0, "skipped": True}]
    sweep.write_text(json.dumps({"results": rows}))
    assert gate.main(["--sweep", str(sweep)]) == 1
    out = capsys.readouterr().out
    assert "ok    all_gather_matmul" in out and "FAIL  matmul_reduce" in out and "op': 'all_reduce'" in out
    assert out.count("not measured") == 2                                 # the skipped point and the collective sweep
    rows[2]["gpu_time_ms"] = 0.6
    sweep.write_text(json.dumps({"results": rows}))
    assert gate.main(["--sweep", str(sweep), "--bench", str(good)]) == 0
    assert gate.main([]) == 2 and gate.main(["--bench", str(tmp_path / "absent.json")]) == 2


@pytest.mark.parametrize("script,args,expect", [
    ("benchmark/ops/bench_matmul_all_reduce_stages.py", ["--axis_M=32", "--axis_K=128", "--axis_N=64"],
     {"gemm", "all_reduce", "sequential", "fused", "library_pair"}),
    ("benchmark/examples/bench_all_gather_gemm.py", ["--axis_m=1,64", "--axis_n=64", "--axis_k=256"], {"k", "m"}),
])
def test_stage_and_sweep_benchmarks_on_the_cpu_backend(tmp_path, script, args, expect):
    """The stage breakdown of GEMM + all-reduce and the small-M all-gather + GEMM sweep check their
    results before timing; on gloo ranks they run the unfused path end to end."""
    import csv

    out = tmp_path / "out.csv"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, script), "--axis_num_ranks=2", *args, "--n_warmup", "1", "--n_repeat", "2",
           "--benchmark_format", "csv", "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    rows = list(csv.DictReader(out.open()))
    timed = [r for r in rows if r["skipped"] == "0"]
    assert timed and all(float(r["gpu_time_ms"]) > 0 for r in timed)
    assert {r.get("stage") or r.get("layout") for r in timed} == expect
    if "layout" in rows[0]:
        assert all(r["skipped"] == "1" for r in rows if r["layout"] == "m" and r["m"] == "1")     # one row cannot be split over two ranks
    else:
        # the fused stage carries the library pair's time, measured by the same loop, and the ratio of the two
        fused = next(r for r in timed if r["stage"] == "fused")
        assert float(fused["nccl_baseline_us"]) > 0
        assert float(fused["speedup_vs_baseline"]) == pytest.approx(float(fused["nccl_baseline_us"]) / (float(fused["gpu_time_ms"]) * 1e3), rel=1e-6)
        assert all(r["nccl_baseline_us"] == "" for r in timed if r["stage"] != "fused")


def test_runner_reports_a_failing_rank_instead_of_waiting(tmp_path):
    """A benchmark whose check fails on one rank: the launcher ends with an error naming the rank,
    within seconds, and leaves no worker behind."""
    script = tmp_path / "bench_failing.py"
    script.write_text(f'''import sys
sys.path.insert(0, {ROOT!r})
import iris_b200.bench as bench


@bench.register
@bench.axis("num_ranks", [2])
def sometimes_wrong(state, ctx):
    assert ctx.get_rank() != 1, "result mismatch on this rank"
    state.exec(lambda: None)


if __name__ == "__main__":
    bench.main()
''')
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    t0 = time.time()
    proc = subprocess.run([sys.executable, str(script), "--n_warmup", "1", "--n_repeat", "1"], env=env, capture_output=True, text=True,
                          timeout=240)
    assert proc.returncode != 0
    assert "benchmark workers failed" in proc.stderr and "result mismatch on this rank" in proc.stderr
    assert time.time() - t0 < 120


def test_runner_skips_a_point_that_exhausts_the_heap_and_goes_on(tmp_path):
    """A sweep point that asks the symmetric heap for more than it has is reported as skipped (all ranks run the
    same allocation sequence and fail alike); the points after it still run and the results are written."""
    script = tmp_path / "bench_big.py"
    script.write_text(f'''import sys
sys.path.insert(0, {ROOT!r})
import torch
import iris_b200.bench as bench


@bench.register
@bench.axis("num_ranks", [2])
@bench.axis("mb", [1, 64, 2])
def grows(state, ctx):
    buf = ctx.zeros(state["mb"] << 20, dtype=torch.uint8)
    state.exec(lambda: buf.add_(1))


if __name__ == "__main__":
    bench.main()
''')
    out = tmp_path / "big.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.run([sys.executable, str(script), "--heap_size", str(16 << 20), "--n_warmup", "1", "--n_repeat", "1",
                           "--benchmark_format", "json", "--benchmark_out", str(out)], env=env, capture_output=True, text=True, timeout=240)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = json.loads(out.read_text())["results"]
    assert [r["params"]["mb"] for r in res] == ["1", "64", "2"]
    assert [bool(r["skipped"]) for r in res] == [False, True, False]
    assert "heap too small" in res[1]["skip_reason"]


def test_fused_ops_benchmark_on_the_cpu_backend(tmp_path):
    """The fused-ops sweep on two gloo ranks (host fallbacks, fp32): every point is timed and carries the deviation of
    a row sample from an fp32 product, which is rounding noise there."""
    out = tmp_path / "fused.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "ops", "bench_fused_ops.py"), "--axis_num_ranks=2", "--axis_impl=iris",
           "--axis_M=256", "--axis_N=64", "--axis_K=128", "--n_warmup", "1", "--n_repeat", "2", "--benchmark_format", "json",
           "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = json.loads(out.read_text())["results"]
    assert {r["benchmark"] for r in res} == {"all_gather_matmul", "matmul_reduce", "matmul_all_gather"}
    assert len(res) == 4 and all(not r["skipped"] and r["gpu_time_ms"] > 0 for r in res)
    assert all(0 <= r["counters"]["max_rel_err"] < 1e-4 for r in res)


def test_overlap_pattern_benchmark_on_the_cpu_backend(tmp_path):
    """GEMM + all-scatter under every overlap pattern on two gloo ranks: all patterns give the same, correct result."""
    out = tmp_path / "patterns.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "examples", "bench_gemm_all_scatter_patterns.py"), "--axis_num_ranks=2",
           "--axis_pattern=bulk_synchronous,fused,wg_specialized", "--axis_M=128", "--axis_N=128", "--axis_K=64", "--n_warmup", "1",
           "--n_repeat", "2", "--benchmark_format", "json", "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = json.loads(out.read_text())["results"]
    assert [r["params"]["pattern"] for r in res] == ["bulk_synchronous", "fused", "wg_specialized"]
    assert all(not r["skipped"] and r["gpu_time_ms"] > 0 and 0 <= r["counters"]["max_rel_err"] < 1e-4 for r in res)


def test_moe_benchmark_on_the_cpu_backend(tmp_path):
    """The MoE sweep on two gloo ranks: the layer's host path agrees with the stock PyTorch form of the benchmark (all-to-all,
    per-expert GEMM loop, weighted index_add) exactly in fp32, and within the e4m3 quantisation error in fp8 mode."""
    out = tmp_path / "moe.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "benchmark", "examples", "bench_moe.py"), "--axis_num_ranks=2", "--axis_tokens=16",
           "--axis_hidden=128", "--axis_ffn=128", "--axis_experts_per_rank=2", "--axis_top_k=2", "--n_warmup", "1", "--n_repeat", "1",
           "--benchmark_format", "json", "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    res = {r["params"]["impl"]: r for r in json.loads(out.read_text())["results"]}
    assert set(res) == {"iris", "iris_fp8", "nccl"} and all(not r["skipped"] and r["gpu_time_ms"] > 0 for r in res.values())
    assert res["iris"]["counters"]["max_rel_err_vs_unfused"] < 1e-5
    import torch

    if hasattr(torch, "float8_e4m3fn"):
        assert 1e-4 < res["iris_fp8"]["counters"]["max_rel_err_vs_unfused"] < 0.15


@pytest.mark.parametrize("script,args,points", [
    ("benchmark/examples/bench_ring_attention.py", ["--axis_seq_per_rank=256"], 3),       # not causal, causal, causal zigzag
    ("benchmark/examples/bench_flash_decode.py", ["--axis_batch=2", "--axis_total_kv=2048,4096"], 2),
])
def test_attention_benchmarks_on_the_cpu_backend(tmp_path, script, args, points):
    """Ring attention and distributed flash decode sweeps on two gloo ranks: every timed point carries the deviation of a
    sample of the layer's output from fp32 attention over the keys of all ranks."""
    out = tmp_path / "attn.json"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, script), "--axis_num_ranks=2", "--axis_impl=iris", *args, "--n_warmup", "1", "--n_repeat", "2",
           "--benchmark_format", "json", "--benchmark_out", str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-3000:]
    timed = [r for r in json.loads(out.read_text())["results"] if not r["skipped"]]
    assert len(timed) == points and all(r["gpu_time_ms"] > 0 and 0 <= r["counters"]["max_rel_err"] < 1e-4 for r in timed)
