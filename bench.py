#!/usr/bin/env python3
"""Headline benchmark: the tensor-parallel MLP step made of the two fused ops

    H = all_gather(X_local) @ W1_local          all_gather_matmul   [M, K] x [K, F/N]
    Y_local = reduce_scatter(H @ W2_local)      matmul_reduce_scatter [M, F/N] x [F/N, K]

with M = 8192 rows, K = 8192, F/N = 3584 per rank (the TP=8 slice of F = 28672), bf16, random
weights N(0, 0.02) and activations N(0, 1) (synthetic data). Per-rank work is fixed as the number
of GPUs grows (weak scaling); the value is the aggregate TFLOPS over all ranks, timed on the
device with CUDA events, maximum over ranks.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      (the unmodified reference, when it can run here)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
M_TOTAL, K_DIM, F_LOCAL = 8192, 8192, 3584
# The only comparable figure the reference publishes: GEMM + all-scatter at 16384^3 fp16 on
# 8 x MI325X, producer/consumer variant, 2190 TFLOPS aggregate (274 TFLOPS per GPU).
PUBLISHED_TFLOPS_PER_GPU = 2190.0 / 8


class ClockSampler:
    """Reads SM clock, power and throttle reasons while the benchmark runs.

    NVML is polled from a thread every few milliseconds (read-only queries), so that even a timed
    region of a few tens of milliseconds yields samples; ``nvidia-smi -lms`` is the fallback when
    the NVML bindings are missing. Samples taken between ``mark_timed(True)`` and
    ``mark_timed(False)`` are the ones reported; if that window caught fewer than three, the
    samples of the whole loaded span (warm-up to the end of the end-to-end loop) are used.
    """

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                   0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []            # (wall time, sm MHz, power W, set of reasons)
        self.max_mhz = None
        self.proc = None
        self.thread = None
        self.stop_flag = False
        self.source = None
        self.load_from = None     # wall time from which the GPU is under the benchmark's load
        self.timed = [None, None]

    def mark_timed(self, begin: bool):
        self.timed[0 if begin else 1] = time.time()

    # ---- NVML
    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            props = torch.cuda.get_device_properties(self.gpu_index)
            uuid = getattr(props, "uuid", None)
            if uuid is not None:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
        except Exception:
            pass
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = self.gpu_index
        if visible:
            try:
                idx = int(visible.split(",")[self.gpu_index])
            except (ValueError, IndexError):
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(idx)

    def _poll_nvml(self, pynvml, handle):
        reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                sm = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                power = pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0
                mask = int(reasons_fn(handle))
                self.rows.append((time.time(), float(sm), power, {n for b, n in self.REASON_BITS.items() if mask & b}))
            except Exception:
                pass
            time.sleep(0.003)

    def start(self):
        try:
            pynvml, handle = self._nvml_handle()
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.source = "nvml"
            self.thread = threading.Thread(target=self._poll_nvml, args=(pynvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.source = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.source = "nvidia-smi"
        self.thread = threading.Thread(target=self._read_smi, daemon=True)
        self.thread.start()

    def _read_smi(self):
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                self.max_mhz = float(parts[2])
                self.rows.append((time.time(), float(parts[1]), float(parts[3]),
                                  {n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active")}))
            except ValueError:
                continue

    def stop(self) -> dict:
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"]}
        if self.source == "nvidia-smi":
            deadline = time.time() + 3.0
            while not self.rows and time.time() < deadline:   # a slow first sample (many ranks start nvidia-smi at once)
                time.sleep(0.05)
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        else:
            self.stop_flag = True
            self.thread.join(timeout=2)
        rows = list(self.rows)
        window = "timed region"
        t0, t1 = self.timed
        use = [r for r in rows if t0 is not None and t1 is not None and t0 <= r[0] <= t1]
        if len(use) < 3:
            window = "warm-up to end of the end-to-end loop"
            use = [r for r in rows if self.load_from is None or r[0] >= self.load_from]
        if not use:
            window = "whole run"
            use = rows
        reasons = set()
        for r in use:
            reasons |= r[3]
        return {"sm_mhz": statistics.median([r[1] for r in use]) if use else None, "sm_max_mhz": self.max_mhz,
                "power_w_max": max([r[2] for r in use]) if use else None, "samples": len(use), "window": window,
                "source": self.source, "reasons": sorted(reasons)}


def run_reference(args) -> int:
    """The reference arm: the unmodified reference package installed under baseline/_ref."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "iris")):
        why = "baseline/_ref is missing: the offline pip install of the reference has not been run on this machine"
    else:
        sys.path.insert(0, ref_dir)
        try:
            import iris  # noqa: F401  (the reference package)
        except Exception as e:  # tritonblas is a git dependency that cannot be fetched offline
            why = f"the reference cannot be imported here: {type(e).__name__}: {e} (its fused ops need the git-only tritonblas package and a HIP DMA-BUF heap)"
    if why is None:
        why = "the reference imports but its heap needs hipMemGetHandleForAddressRange (AMD only)"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    # stdout carries ONE line (the JSON record). Libraries write to file descriptor 1 on their own
    # (NCCL prints its version banner there), so the descriptor is pointed at stderr for the run and
    # the record goes to a saved copy of the original stdout at the end.
    sys.stdout.flush()
    record_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    sampler = ClockSampler(local)
    sampler.start()          # runs from here to the end of the end-to-end loop
    if not dist.is_initialized():
        if "MASTER_ADDR" not in os.environ:
            os.environ["MASTER_ADDR"] = "127.0.0.1"
            os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))

    import iris_b200 as iris

    W = world
    M_local = M_TOTAL // W
    dtype = torch.bfloat16
    ctx = iris.iris(6 << 30)
    dev = ctx.get_device()
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    # weights: random init of the architecture's shapes; activations: synthetic N(0, 1)
    # stored as nn.Linear stores them, (out_features, in_features); the kernels take the transposed views as they are
    W1 = (torch.randn(F_LOCAL, K_DIM, device=dev, dtype=torch.float32, generator=g) * 0.02).to(dtype).t()
    W2 = (torch.randn(K_DIM, F_LOCAL, device=dev, dtype=torch.float32, generator=g) * 0.02).to(dtype).t()
    X_host = torch.randn(M_local, K_DIM, dtype=torch.float32).to(dtype).pin_memory()
    X = torch.empty(M_local, K_DIM, device=dev, dtype=dtype)
    X.copy_(X_host)
    H = torch.empty(M_TOTAL, F_LOCAL, device=dev, dtype=dtype)
    Y = torch.empty(M_local, K_DIM, device=dev, dtype=dtype)
    ws1 = ctx.ops.all_gather_matmul(H, X, W1, shard_dim=0)
    ws2 = ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True)

    # The record is about the fused kernels: a plan that could not take the shape would silently run
    # GEMM + collective instead, which is not what this benchmark claims to time.
    if ws1.variant != "fused" or ws2.variant != "fused":
        raise SystemExit(f"bench.py: the fused kernels were not selected (all_gather_matmul: {ws1.variant}, matmul_reduce_scatter: {ws2.variant})")

    def step():
        ctx.ops.all_gather_matmul(H, X, W1, shard_dim=0, workspace=ws1, async_op=True)
        ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True, workspace=ws2, async_op=True)

    flops_per_rank = 2.0 * M_TOTAL * K_DIM * F_LOCAL * 2
    from iris_b200 import _lib as _iris_lib

    def verify() -> dict:
        """Outside every timed region: 16 rows of each rank's block against an fp32 product of the
        gathered inputs (NCCL gathers the rows, torch multiplies in fp32). H is checked against
        X_all @ W1; Y against the sum over ranks of H @ W2 taken from the bf16 H the kernel wrote."""
        rows = torch.linspace(0, M_local - 1, 16, device=dev).long()
        xs = X[rows].contiguous()
        x_all = torch.empty(W * 16, K_DIM, device=dev, dtype=dtype)
        dist.all_gather_into_tensor(x_all, xs)
        grow = (torch.arange(W, device=dev)[:, None] * M_local + rows[None, :]).flatten()
        h_ref = x_all.float() @ W1.float()
        h_got = H[grow]
        y_part = h_got.float() @ W2.float()
        dist.all_reduce(y_part)
        y_ref = y_part[rank * 16:(rank + 1) * 16]
        y_got = Y[rows].float()
        eh = float((h_got.float() - h_ref).abs().max() / h_ref.abs().max())
        ey = float((y_got - y_ref).abs().max() / y_ref.abs().max())
        t = torch.tensor([eh, ey], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        eh, ey = float(t[0]), float(t[1])
        ok = eh < 1e-2 and ey < 1e-2          # bf16 outputs: one rounding of values up to the maximum
        return {"rows_checked": W * 16, "h_max_err_over_max": round(eh, 6), "y_max_err_over_max": round(ey, 6), "ok": ok,
                "oracle": "fp32 torch.matmul of NCCL-gathered rows"}

    # ---------------- device-timed region: exactly `steps` steps between barriers
    # (the clock sampler runs from the warm-up to the end of the end-to-end loop, all of it the
    # same load, so that a short timed region still yields samples)
    sampler.load_from = time.time()
    for _ in range(max(args.warmup, 3)):
        step()
    ctx.barrier()
    numerics = verify()
    if not numerics["ok"]:
        raise SystemExit(f"bench.py: the fused step does not match the fp32 oracle: {numerics}")
    ctx.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    launches_before = _iris_lib.launch_count()
    sampler.mark_timed(True)
    start.record()
    for _ in range(args.steps):
        step()
    end.record()
    torch.cuda.synchronize()
    sampler.mark_timed(False)
    gpu_launches = _iris_lib.launch_count() - launches_before     # counted where the library launches its kernels
    dist.barrier()
    ms = start.elapsed_time(end) / args.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ctx.check()

    # ---------------- the same step done unfused on the same box, in the same process, with the same
    # steps and warm-up: NCCL all-gather, two cuBLAS GEMMs, NCCL reduce-scatter (what stock PyTorch
    # tensor parallelism runs; at one GPU just the two cuBLAS GEMMs). Device-timed, max over ranks.
    Xall = torch.empty(M_TOTAL, K_DIM, device=dev, dtype=dtype) if W > 1 else None
    P = torch.empty(M_TOTAL, K_DIM, device=dev, dtype=dtype) if W > 1 else None
    H2 = torch.empty(M_TOTAL, F_LOCAL, device=dev, dtype=dtype)
    Y2 = torch.empty(M_local, K_DIM, device=dev, dtype=dtype)

    def unfused_step():
        if W > 1:
            dist.all_gather_into_tensor(Xall, X)
            torch.matmul(Xall, W1, out=H2)
            torch.matmul(H2, W2, out=P)
            dist.reduce_scatter_tensor(Y2, P)
        else:
            torch.matmul(X, W1, out=H2)
            torch.matmul(H2, W2, out=Y2)

    for _ in range(max(args.warmup, 3)):
        unfused_step()
    dist.barrier()
    torch.cuda.synchronize()
    bs, be = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bs.record()
    for _ in range(args.steps):
        unfused_step()
    be.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([bs.elapsed_time(be) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    base_ms = float(t.item())
    base_err = float((Y2.float() - Y.float()).abs().max() / Y.float().abs().max())    # both paths computed the same step
    del Xall, P, H2, Y2

    # ---------------- end-to-end region: every step copies its input from pinned host memory,
    # runs the two ops through the public API and reads the step's scalar result back. The copy
    # of step i+1 runs on a second stream while step i computes (two device buffers); all K
    # copies and all K result reads, the first and the last included, are inside the timed region.
    copy_stream = torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    Xb = [X, torch.empty_like(X)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]

    def prefetch(i):
        b = i & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])
            Xb[b].copy_(X_host, non_blocking=True)
            ready[b].record(copy_stream)

    # The step's scalar result (one reduction kernel over Y) is copied to pinned host memory every
    # step (4 bytes) and read by the host ONE STEP LATER, so the host never drains the GPU: while it
    # waits for step i-1's value, step i is already queued.
    loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
    loss_done = [torch.cuda.Event(), torch.cuda.Event()]

    def e2e_loop(n):
        res = 0.0
        for ev in consumed:
            ev.record(main_stream)
        prefetch(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                prefetch(i + 1)
            main_stream.wait_event(ready[b])
            ctx.ops.all_gather_matmul(H, Xb[b], W1, shard_dim=0, workspace=ws1, async_op=True)
            consumed[b].record(main_stream)
            ctx.ops.matmul_reduce_scatter(Y, H, W2, scatter_rows=True, workspace=ws2, async_op=True)
            loss_host[b:b + 1].copy_(torch.linalg.vector_norm(Y, dtype=torch.float32).reshape(1), non_blocking=True)
            loss_done[b].record(main_stream)
            if i > 0:
                loss_done[b ^ 1].synchronize()
                res = float(loss_host[b ^ 1]) ** 2 / Y.numel()
        loss_done[(n - 1) & 1].synchronize()
        res = float(loss_host[(n - 1) & 1]) ** 2 / Y.numel()
        return res

    e2e_loop(3)
    ctx.barrier()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    last = e2e_loop(args.steps)
    e2.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e_ms = max(s2.elapsed_time(e2) / args.steps, wall_ms)
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    clocks = sampler.stop()
    ctx.check()

    value = flops_per_rank * W / (ms * 1e-3) / 1e12
    e2e_value = flops_per_rank * W / (e2e_ms * 1e-3) / 1e12
    out = {
        "metric": "fused all_gather_matmul + matmul_reduce_scatter TFLOPS (aggregate over ranks, device time, max over ranks)",
        "value": round(value, 2),
        "unit": "TFLOPS",
        "n_gpus": W,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": round(value / (PUBLISHED_TFLOPS_PER_GPU * W), 3),
        "dtype": "bf16",
        "data": "synthetic (activations N(0,1), random-init weights N(0,0.02))",
        "config": {
            "model": "tensor-parallel MLP slice: all_gather_matmul [8192,8192]x[8192,3584] then matmul_reduce_scatter [8192,3584]x[3584,8192]",
            "global_batch": M_TOTAL, "seq_len": 1, "parallelism": f"tp{W}",
            "rows_per_rank": M_local, "l2": "inputs larger than L2 (about 500 MB touched per step)",
            "vs_baseline_note": "reference's published GEMM+all-scatter 2190 TFLOPS on 8 x MI325X, scaled per GPU",
            "nvls": bool(ctx.has_multicast()), "tile_n": [ws1.bn, ws2.bn], "weights": "nn.Linear layout (out, in), used as transposed views",
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": "TFLOPS", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": X_host.numel() * X_host.element_size(), "d2h_bytes_per_step": 4, "last_result": last,
                "read": "every step's result is copied to pinned host memory and read by the host one step later"},
        "gpu_launches": gpu_launches,        # this library's kernels launched inside the device-timed region (one fused kernel per op per step)
        "numerics": numerics,
        "same_box_nccl_cublas": {"ms_per_step": round(base_ms, 4), "value": round(flops_per_rank * W / (base_ms * 1e-3) / 1e12, 2),
                                 "unit": "TFLOPS", "steps": args.steps, "warmup": max(args.warmup, 3),
                                 "what": "NCCL all_gather_into_tensor + 2 x torch.matmul (cuBLAS) + NCCL reduce_scatter_tensor, same shapes, same process",
                                 "max_diff_vs_fused_over_max": round(base_err, 6)},
        "impl": "ours",
    }
    if rank == 0:
        sys.stdout.flush()
        os.write(record_fd, (json.dumps(out) + "\n").encode())
    ctx.barrier()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
