#!/usr/bin/env python
"""Benchmark of the batch-1 decode hot path (see DESIGN.md for definitions).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemv] [--impl reference]

Prints ONE JSON line on rank 0.  Timing is done with CUDA events on the library's own
stream (lb_timer_*), bracketed by a barrier and a stream synchronise on both sides, max
over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PEAKS_FILE = ROOT / "MEASURED_PEAKS.json"
FALLBACK_HBM_GBS = 6650.0


def measured_hbm_peak():
    try:
        return float(json.loads(PEAKS_FILE.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """samples nvidia-smi SM clocks and throttle reasons during the timed region"""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([p.strip() for p in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init_dist(world):
    if world == 1:
        return None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend="nccl")
    return dist


def barrier(dist):
    if dist is not None:
        import torch
        dist.barrier()
        torch.cuda.synchronize()


def max_over_ranks(dist, v):
    if dist is None:
        return v
    import torch
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gemv_bytes(K, N, xb=2, yb=2):
    return K // 8 * N * 4 + K // 128 * N * 2 + K // 128 * (N // 8) * 4 + K * xb + N * yb


# ------------------------------------------------------------------------------------------
# workload "gemv": BASELINE config 0 (17408 x 5120 int4 GEMV), rotating over weight sets
# larger than L2 so that every launch streams its weights from HBM
# ------------------------------------------------------------------------------------------
def cpu_gemv_sample(K, N, qw, sc, qz, x, budget_s=12.0):
    from oracle import oracle as orc
    t0 = time.perf_counter()
    orc.gptq_gemv(qw, sc, qz, x, K, N)
    one = time.perf_counter() - t0
    reps = max(1, min(200, int(budget_s / max(one, 1e-4))))
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.gptq_gemv(qw, sc, qz, x, K, N)
    dt = (time.perf_counter() - t0) / reps
    return dt, reps, orc.num_threads()


def bench_gemv(args, rank, local, world, dist):
    import lithos_b200 as lb
    K, N, SETS = 5120, 17408, 8   # 8 x 46 MB of weights: 371 MB, about 3x the 126 MB L2
    ctx = lb.Context(local)
    host = []
    dev = []
    for s in range(SETS):
        qw = lb.fill_u32(K // 8 * N, 100 + s, 1)
        sc = lb.fill_scales_f16(K // 128 * N, 100 + s, 2)
        qz = lb.fill_u32(K // 128 * (N // 8), 100 + s, 3)
        host.append((qw, sc, qz))
        dev.append([ctx.to_device(a) for a in (qw, sc, qz)])
    x = lb.fill_normal(K, 100, 4, dtype="f16")
    d_x, d_y = ctx.to_device(x), ctx.alloc(N * 2)
    per_step = 16  # GEMV launches per step (a step = 16 projections' worth of the 448 per token)

    # one step = 16 GEMV launches captured once as a CUDA graph (the way the decode step submits them)
    ctx.begin_capture()
    for j in range(per_step):
        w = dev[j % SETS]
        ctx.gemv_int4(w[0], w[1], w[2], d_x, d_y, K, N, 0)
    graph = ctx.end_capture()

    def step(i):
        graph.launch()

    # bring the SM clocks up from idle before anything is timed (not one of the W warm-up steps)
    t_ramp = time.perf_counter()
    while time.perf_counter() - t_ramp < args.ramp_s:
        for i in range(8):
            step(i)
        ctx.sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for i in range(args.warmup):
        step(i)
    ctx.sync()
    barrier(dist)
    ctx.reset_launches()
    ctx.timer_start()
    for i in range(args.steps):
        step(i)
    ms = ctx.timer_stop()
    barrier(dist)
    launches = ctx.launches
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(dist, ms)
    assert ctx.device_status() == 0

    # end to end through the host-buffer entry point: x in (pinned copy inside), y out, every step
    y_host = np.empty(N, dtype=np.float16)
    ctx.gemv_int4_host(host[0][0], host[0][1], host[0][2], x, y_host, K, N, 0, weights_resident=False)
    e2e_steps = max(args.steps, 20)
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        ctx.gemv_int4_host(host[0][0], host[0][1], host[0][2], x, y_host, K, N, 0, weights_resident=True)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = max_over_ranks(dist, e2e_s)

    algo = gemv_bytes(K, N)
    per_launch_s = ms * 1e-3 / (args.steps * per_step)
    achieved = algo / per_launch_s / 1e9
    peak, which = measured_hbm_peak()
    out = {
        "metric": "int4 GEMV HBM GB/s (batch-1 decode projection 5120->17408)", "value": achieved * world,
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights, fp16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "config0: GPTQ int4 GEMV 17408x5120 g128 asymmetric, batch 1", "gemv_per_step": per_step,
                   "l2": f"rotating over {SETS} weight sets ({SETS * algo / 1e6:.0f} MB > 126 MB L2)",
                   "parallelism": f"replicas x{world}"},
        "e2e": {"value": algo / e2e_s / 1e9 * world, "unit": "GB/s", "h2d_bytes_per_step": K * 2, "d2h_bytes_per_step": N * 2},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": which, "kernel": "gemv_int4_w256",
                     "us_per_launch": per_launch_s * 1e6, "algorithmic_bytes": algo},
        "clocks": clocks,
    }
    if rank == 0:
        dt, reps, cores = cpu_gemv_sample(K, N, host[0][0], host[0][1], host[0][2], x)
        out["cpu_baseline"] = {"value": algo / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                               "sample": f"{reps} full 17408x5120 GEMVs with the C oracle (OpenMP), {dt * 1e3:.2f} ms each"}
    ctx.close()
    return out


def reference_gemv(args, rank):
    """--impl reference: the reference has no CPU implementation of these kernels that can run (its
    interpreters evaluate the integer host dialect only), so the CPU arm is the plain-C restatement."""
    import lithos_b200 as lb
    K, N = 5120, 17408
    qw = lb.fill_u32(K // 8 * N, 100, 1)
    sc = lb.fill_scales_f16(K // 128 * N, 100, 2)
    qz = lb.fill_u32(K // 128 * (N // 8), 100, 3)
    x = lb.fill_normal(K, 100, 4, dtype="f16")
    from oracle import oracle as orc
    per_step = 16
    for _ in range(min(args.warmup, 2)):
        orc.gptq_gemv(qw, sc, qz, x, K, N)
    t0 = time.perf_counter()
    n = 0
    for _ in range(args.steps):
        orc.gptq_gemv(qw, sc, qz, x, K, N)   # bounded sample: 1 of the step's 16 GEMVs
        n += 1
    dt = (time.perf_counter() - t0) / n
    algo = gemv_bytes(K, N)
    v = algo / dt / 1e9
    return {"impl": "reference", "metric": "int4 GEMV HBM GB/s (batch-1 decode projection 5120->17408)", "value": v,
            "unit": "GB/s", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * per_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": "config0: GPTQ int4 GEMV 17408x5120 g128 asymmetric, batch 1"},
            "cpu_baseline": {"value": v, "unit": "GB/s", "cores": orc.num_threads(), "kind": "port",
                             "sample": f"1 GEMV per step x {n} steps, C oracle with OpenMP"},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="gemv", choices=["gemv"])
    ap.add_argument("--ramp-s", type=float, default=1.5, help="seconds of untimed work before warm-up (clock ramp)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local, world = dist_env()
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(reference_gemv(args, rank)), flush=True)
        return
    dist = init_dist(world)
    out = bench_gemv(args, rank, local, world, dist)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
