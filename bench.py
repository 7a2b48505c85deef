#!/usr/bin/env python
"""Benchmark of the batch-1 decode hot path: BASELINE config 3 (the 64-layer decode step) is the timed workload; the
default single-GPU line also carries one measurement each for configs 0, 1 and 2.

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


def host_threads(world=1):
    """threads for host-side work.  torchrun exports OMP_NUM_THREADS=1 when the variable is unset; a CPU baseline on one
    core or a model build on one core per rank is not what anyone wants to time, so that setting (and only that one) is
    replaced by the cores this process may use, shared between the ranks of the job."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, cores // max(world, 1))


def fix_omp_env(world):
    if os.environ.get("OMP_NUM_THREADS", "1") == "1" and "TORCHELASTIC_RUN_ID" in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(host_threads(world))
    elif "OMP_NUM_THREADS" not in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(host_threads(world))


TRAFFIC_FILE = ROOT / "profiles" / "gemv_chain_traffic.json"


def chain_traffic_bytes(lb):
    """dram__bytes_read.sum + dram__bytes_write.sum of one gemv_chain launch of the roofline workload, from the ncu capture
    summarised under profiles/; None when no capture is recorded for the packed-weight layout this library uses"""
    try:
        rec = json.loads(TRAFFIC_FILE.read_text())
        if int(rec["pack_version"]) != int(lb.lib().lb_gemv_pack_version()):
            return None
        return int(rec["dram_bytes_read"]) + int(rec["dram_bytes_write"])
    except Exception:
        return None


def logits_hash(a):
    import hashlib
    return hashlib.blake2b(np.ascontiguousarray(a, dtype=np.float32).tobytes(), digest_size=8).hexdigest()


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
    """--impl reference --workload gemv: the plain-C restatement on config 0 (the reference has no CPU implementation of
    its kernels that can run); inputs from the oracle's own twin of the generator."""
    from oracle import oracle as orc
    if orc.num_threads() == 1 and host_threads() > 1:
        orc.set_num_threads(host_threads())
    K, N = 5120, 17408
    qw = orc.fill_u32(K // 8 * N, 100, 1)
    sc = orc.fill_scales_f16(K // 128 * N, 100, 2)
    qz = orc.fill_u32(K // 128 * (N // 8), 100, 3)
    x = orc.fill_normal(K, 100, 4, dtype="f16")
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


# ------------------------------------------------------------------------------------------
# workload "decode": BASELINE config 3 — the full 64-layer Qwen3.5-27B-shaped decode step,
# random-init weights, recurrent state and KV cache pre-filled to 4096 tokens by direct seeded
# fill, greedy decoding, the whole step replayed as one CUDA graph
# ------------------------------------------------------------------------------------------
CTX_PREFILL = 4096


def decode_algorithmic_bytes(cfg, model_weight_bytes, ctx_len):
    """bytes one token must move: all weights of the step (as laid out on the device: int4 words +
    fp16 scales + zero-points, bf16 LM head, a/b projections, conv taps) + DeltaNet state read and
    write + the KV cache rows attended"""
    n_dn = sum(0 if cfg.is_fa(l) else 1 for l in range(cfg.n_layers))
    n_fa = cfg.n_layers - n_dn
    state = n_dn * 2 * cfg.dn_v_heads * 128 * 128 * 4
    kv = n_fa * ctx_len * cfg.fa_kv_heads * 256 * 2 * 2
    return model_weight_bytes + state + kv


def time_gemv_mix(ctx, lb, cfg, args, tp_size=1, chained=False):
    """The step's own int4 GEMV launch mix (5 per layer, real shapes, norm prologues and fused
    epilogues, weights rotating over > L2 worth of distinct matrices), captured as one graph and
    timed alone with CUDA events: average duration and algorithmic bytes per launch.
    chained: the four GEMVs between two token mixers (out, gate/up, down, next input projection) go out as
    ONE persistent gemv_chain launch, as the single-GPU decode step issues them; a launch is then a whole chain."""
    H, I = cfg.hidden, cfg.inter
    C_, V, I = cfg.conv_channels // tp_size, cfg.dn_v_heads * 128 // tp_size, I // tp_size   # this shard's slices
    shapes = [(H, C_ + V, "in"), (V, H, "out"), (H, 2 * I, "gateup"), (I, H, "down")]
    sets = 3   # 3 x ~196 MB of distinct weights per shape group: > 126 MB L2 between reuses
    mats = []
    for s_ in range(sets):
        row = []
        for (K, N, _) in shapes:
            qw = ctx.to_device(lb.fill_u32(K // 8 * N, 7 + s_, 1))
            sc = ctx.to_device(lb.fill_scales_f16(K // 128 * N, 7 + s_, 2))
            qz = ctx.to_device(lb.fill_u32(K // 128 * (N // 8), 7 + s_, 3))
            pk = ctx.gemv_pack(qw, sc, qz, K, N, swiglu=(len(row) == 2)) if chained else None
            row.append((qw, sc, qz, K, N, pk))
        mats.append(row)
    X = ctx.to_device(lb.fill_normal(H, 7, 4))
    nw = ctx.to_device(lb.fill_normal(H, 7, 5, std=0.02, dtype="bf16"))
    hw = ctx.to_device(lb.fill_normal(128, 7, 6, mean=1.0, std=0.02))
    y_in, y_mix, y_m = ctx.alloc((C_ + V) * 4), ctx.to_device(lb.fill_normal(V, 7, 8)), ctx.alloc(I * 2)
    xn = ctx.alloc(H * 2)
    ctx.begin_capture()
    n_layers = 12
    for l in range(n_layers):
        m_ = mats[l % sets]
        if chained:
            op = lambda w, x, y, xm, ym, **kw: dict(packed=w[5], x=x, y=y, K=w[3], N=w[4], x_mode=xm, y_mode=ym, **kw)
            ctx.gemv_chain([op(m_[1], y_mix, X, lb.X_F32_HEADNORM_SILU, lb.Y_F32_ACCUM, aux0=hw, aux1=y_in),
                            op(m_[2], X, y_m, lb.X_F32_RMSNORM, lb.Y_SWIGLU_F16, aux0=nw),
                            op(m_[3], y_m, X, lb.X_F16, lb.Y_F32_ACCUM),
                            op(mats[(l + 1) % sets][0], X, y_in, lb.X_F32_RMSNORM, lb.Y_F32, aux0=nw, x_out=xn)])
            continue
        ctx.gemv_int4_fused(m_[0][0], m_[0][1], m_[0][2], X, y_in, H, C_ + V, lb.X_F32_RMSNORM, lb.Y_F32, aux0=nw, x_out=xn)
        ctx.gemv_int4_fused(m_[1][0], m_[1][1], m_[1][2], y_mix, X, V, H, lb.X_F32_HEADNORM_SILU, lb.Y_F32_ACCUM, aux0=hw, aux1=y_in)
        ctx.gemv_int4_fused(m_[2][0], m_[2][1], m_[2][2], X, y_m, H, 2 * I, lb.X_F32_RMSNORM, lb.Y_SWIGLU_F16, aux0=nw)
        ctx.gemv_int4_fused(m_[3][0], m_[3][1], m_[3][2], y_m, X, I, H, lb.X_F16, lb.Y_F32_ACCUM)
    g = ctx.end_capture()
    launches = g.kernels
    algo = n_layers * sum(gemv_bytes(K, N, 4, 4) for (K, N, _) in shapes)
    for _ in range(5):
        g.launch()
    ctx.sync()
    reps = 30
    ctx.timer_start()
    for _ in range(reps):
        g.launch()
    ms = ctx.timer_stop()
    g.destroy()
    return ms * 1e-3 / (reps * launches), algo / launches, launches * reps


WORKLOAD = ("config3: 64-layer Qwen3.5-27B-shaped decode step, hidden 5120, 3 DeltaNet + 1 attention per 4 layers, SwiGLU 17408, "
            "vocab 248320, int4 g128 linears, bf16 LM head, state pre-filled to 4096 tokens by seeded fill, greedy, one CUDA graph per step")
METRIC = "batch-1 decode tok/s (Qwen3.5-27B-shaped hybrid, GPTQ int4, 4096-token state)"


def oracle_decode_run(seed, ctx_len, warm, steps, n_layers=64):
    """The C oracle (OpenMP over the host cores) decoding the benchmark's model: full steps of all layers + LM head from
    (token 1, position ctx_len), greedy.  Inputs come from the oracle's own twin of the seeded generator, so nothing
    of the product library is loaded.  Returns (tokens of all warm + timed steps, seconds per timed step, threads,
    seconds spent building the model)."""
    from oracle import oracle as orc
    if orc.num_threads() == 1 and host_threads() > 1:
        orc.set_num_threads(host_threads())
    t0 = time.perf_counter()
    cfg = orc.qwen35_27b(max_ctx=ctx_len + warm + steps + 8, n_layers=n_layers)
    slots = [orc.synthetic_layer_slots(cfg, seed, l) for l in range(cfg.n_layers)]
    om = orc.Model(cfg, slots, orc.synthetic_globals(cfg, seed))
    orc.seed_state(om, ctx_len, seed)
    build_s = time.perf_counter() - t0
    tok, toks = 1, []
    for i in range(warm):
        tok = om.decode(tok, ctx_len + i)
        toks.append(tok)
    t0 = time.perf_counter()
    for i in range(steps):
        tok = om.decode(tok, ctx_len + warm + i)
        toks.append(tok)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    om.close()
    return toks, dt, orc.num_threads(), build_s


def bench_small_configs(ctx, lb):
    """One device-timed figure each for BASELINE configs 0, 1 and 2, so that every config has a number in the default
    line: config 0 (17408 x 5120 int4 GEMV, 8 rotating weight sets > L2), config 1 (one DeltaNet step, 48/16 heads, 64
    rotating states > L2), config 2 (decode attention at 4096 / 32768 / 131072 rows, rotating caches > L2)."""
    peak, _ = measured_hbm_peak()
    out = {}
    # ---- config 0 ----
    K, N, SETS = 5120, 17408, 8
    dev = [[ctx.to_device(lb.fill_u32(K // 8 * N, 100 + s_, 1)), ctx.to_device(lb.fill_scales_f16(K // 128 * N, 100 + s_, 2)),
            ctx.to_device(lb.fill_u32(K // 128 * (N // 8), 100 + s_, 3))] for s_ in range(SETS)]
    d_x, d_y = ctx.to_device(lb.fill_normal(K, 100, 4, dtype="f16")), ctx.alloc(N * 2)

    def timed(graph, launches, reps=40):
        for _ in range(5):
            graph.launch()
        ctx.sync()
        ctx.timer_start()
        for _ in range(reps):
            graph.launch()
        us = ctx.timer_stop() * 1e3 / (reps * launches)
        graph.destroy()
        return us

    def run_gemv_int4():
        ctx.begin_capture()
        for j in range(16):
            w = dev[j % SETS]
            ctx.gemv_int4(w[0], w[1], w[2], d_x, d_y, K, N, 0)
        return timed(ctx.end_capture(), 16)

    algo = gemv_bytes(K, N)
    rec = lambda kernel, us: {"kernel": kernel, "us_per_launch": round(us, 2), "GBps": round(algo / us / 1e3, 1),
                              "frac_of_measured_peak": round(algo / us / 1e3 / peak, 3)}
    us_plain = run_gemv_int4()     # reference-format weights only: split-K over 2-CTA clusters
    out["gemv_config0"] = {"workload": "config0: int4 GEMV 17408x5120 g128 asymmetric, fp16 x and y, batch 1; 8 rotating weight sets (371 MB > L2), "
                                       "lb_gemv_int4 each launch"}
    if ctx.gemv_chain_supports(K, N):
        # the library's fast path: lb_gemv_pack once per matrix, after which the same lb_gemv_int4 call streams the strip-packed copy
        packed = [ctx.gemv_pack(w[0], w[1], w[2], K, N) for w in dev]
        us = run_gemv_int4()
        out["gemv_config0"].update(rec("gemv_chain (one entry; lb_gemv_int4 after lb_gemv_pack)", us))
        out["gemv_config0"]["algorithmic_bytes"] = algo
        out["gemv_config0"]["frac_of_8TBps"] = round(algo / us / 1e3 / 8000.0, 3)
        out["gemv_config0"]["without_packed_copy"] = rec("gemv_int4_w256", us_plain)
        for b in packed:
            b.free()
    else:
        out["gemv_config0"].update(rec("gemv_int4_w256", us_plain))
        out["gemv_config0"]["algorithmic_bytes"] = algo
    # the kernel to beat: the reference's own GEMV (minds/gptq_gemv_safe.ptx assembled unmodified for sm_100a) on the same matrices in
    # its native mode (fp32 x and y, zero-point 8, result added to y), launched as src/launcher.s:1479-1535 launches it.  A baseline leg:
    # it is timed beside the product, never inside its timed region.
    ref_cubin = ROOT / "oracle" / "_ref" / "gptq_gemv_safe.cubin"
    if ref_cubin.exists():
        import ctypes as C
        L = lb.lib()
        L.lb_module_load.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int)]
        L.lb_module_get_kernel.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.POINTER(C.c_uint64)]
        L.lb_launch_kernel.argtypes = [C.c_void_p, C.c_uint64] + [C.c_uint] * 7 + [C.POINTER(C.c_void_p)]
        mod, fn = C.c_int(), C.c_uint64()
        ctx._check(L.lb_module_load(ctx.h, str(ref_cubin).encode(), C.byref(mod)))
        ctx._check(L.lb_module_get_kernel(ctx.h, mod, b"gptq_gemv_safe", C.byref(fn)))
        d_x32, d_y32 = ctx.to_device(lb.fill_normal(K, 100, 4)), ctx.alloc(N * 4).zero()

        def ref_launch(w):
            vals = [C.c_uint64(w[0].ptr), C.c_uint64(w[1].ptr), C.c_uint64(d_x32.ptr), C.c_uint64(d_y32.ptr), C.c_uint32(N), C.c_uint32(K),
                    C.c_uint32(1), C.c_uint32(K // 8)]
            params = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
            ctx._check(L.lb_launch_kernel(ctx.h, fn, (N + 255) // 256, 1, 1, 64, 1, 1, 4 * K, params))

        for j in range(SETS):
            ref_launch(dev[j])
        ctx.sync()
        ctx.timer_start()
        for j in range(3 * SETS):
            ref_launch(dev[j % SETS])
        us_ref = ctx.timer_stop() * 1e3 / (3 * SETS)
        out["gemv_config0"]["reference_kernel"] = {"kernel": "gptq_gemv_safe (the reference's PTX, assembled for sm_100a; fp32 x/y, zero-point 8)",
                                                   "us_per_launch": round(us_ref, 2), "GBps": round(algo / us_ref / 1e3, 1),
                                                   "frac_of_measured_peak": round(algo / us_ref / 1e3 / peak, 3),
                                                   "ours_speedup": round(us_ref / out["gemv_config0"]["us_per_launch"], 1)}
        d_x32.free()
        d_y32.free()
    for w in dev:
        for b in w:
            b.free()
    # ---- config 1 ----
    HV, HK, NS = 48, 16, 64
    st = ctx.alloc(NS * HV * 128 * 128 * 4)
    one = lb.fill_normal(HV * 128 * 128, 7, 10, std=0.02)
    for i in range(NS):
        lb.lib().lb_memcpy_h2d(ctx.h, st.ptr + i * one.nbytes, one.ctypes.data, one.nbytes)
    ctx.sync()
    q = ctx.to_device(lb.fill_normal(HK * 128, 7, 11, std=0.088, dtype="bf16"))
    k = ctx.to_device(lb.fill_normal(HK * 128, 7, 12, std=0.088, dtype="bf16"))
    v = ctx.to_device(lb.fill_normal(HV * 128, 7, 13, dtype="bf16"))
    g = ctx.to_device(np.full(HV, 0.9, np.float32))
    beta = ctx.to_device(np.full(HV, 0.5, np.float32))
    o = ctx.alloc(HV * 128 * 4)
    from lithos_b200 import DeviceBuffer

    def view(buf, off, n):
        b = DeviceBuffer.__new__(DeviceBuffer)
        b.ctx, b.ptr, b.nbytes = ctx, buf.ptr + off, n
        return b

    ctx.begin_capture()
    for i in range(NS):
        ctx.deltanet_step(view(st, i * one.nbytes, one.nbytes), q, k, v, None, g, beta, o, HV, HK)
    us = timed(ctx.end_capture(), NS)
    algo = 2 * HV * 128 * 128 * 4
    out["deltanet_step"] = {"workload": "config1: one Gated DeltaNet decode step, 48 value / 16 key heads, fp32 state [48,128,128]; 64 rotating states (201 MB > L2)",
                            "kernel": "deltanet_step_bf16", "us_per_launch": round(us, 2), "algorithmic_bytes": algo, "GBps": round(algo / us / 1e3, 1),
                            "frac_of_measured_peak": round(algo / us / 1e3 / peak, 3)}
    for b in (st, q, k, v, g, beta, o):
        b.free()
    # ---- config 2 ----
    HQ, HKV, POOL = 24, 4, 4 * 131072          # pool of cache rows: 1.07 GB each for K and V
    row = HKV * 256 * 2
    chunk = lb.fill_normal(32768 * HKV * 256, 7, 20, dtype="bf16")
    kc, vc = ctx.alloc(POOL * row), ctx.alloc(POOL * row)
    for buf in (kc, vc):
        for i in range(POOL // 32768):
            lb.lib().lb_memcpy_h2d(ctx.h, buf.ptr + i * chunk.nbytes, chunk.ctypes.data, chunk.nbytes)
    ctx.sync()
    ins = {n: ctx.to_device(lb.fill_normal(h * 256, 7, 21 + i, dtype="bf16")) for i, (n, h) in enumerate((("q", HQ), ("k", HKV), ("v", HKV), ("gate", HQ)))}
    qw = ctx.to_device(lb.fill_normal(256, 7, 26, mean=1.0, std=0.02, dtype="bf16"))
    kw = ctx.to_device(lb.fill_normal(256, 7, 27, mean=1.0, std=0.02, dtype="bf16"))
    d_o = ctx.alloc(HQ * 256 * 4)
    sweep = []
    for L in (4096, 32768, 131072):
        sets = min(POOL // L, 32)
        ctx.begin_capture()
        for i in range(sets):
            ctx.attention_decode(ins["q"], ins["k"], ins["v"], ins["gate"], qw, kw, view(kc, i * L * row, L * row), view(vc, i * L * row, L * row),
                                 d_o, L - 1, HQ, HKV)
        us = timed(ctx.end_capture(), sets, reps=20 if L < 131072 else 6)
        algo = L * HKV * 256 * 2 * 2
        sweep.append({"rows": L, "us_per_launch": round(us, 2), "algorithmic_bytes": algo, "GBps": round(algo / us / 1e3, 1),
                      "frac_of_measured_peak": round(algo / us / 1e3 / peak, 3), "rotating_caches": sets})
    out["attention_sweep"] = {"workload": "config2: GQA decode attention, 24 query / 4 KV heads, head_dim 256, bf16 cache, q/k norm + RoPE + append + gate fused",
                              "kernel": "attn_decode_mma", "sweep": sweep}
    for b in [kc, vc, qw, kw, d_o] + list(ins.values()):
        b.free()
    assert ctx.device_status() == 0
    return out


def bench_decode(args, rank, local, world, dist):
    import lithos_b200 as lb
    from lithos_b200 import model as M
    from lithos_b200 import tp
    cfg = M.qwen35_27b(max_ctx=CTX_PREFILL + args.warmup + args.steps + 64, n_layers=args.layers)
    ctx = lb.Context(local)
    t0 = time.perf_counter()
    comm = None
    if world > 1:   # tensor parallel: exchange buffers mapped into every peer (CUDA IPC), handles passed over the process group
        def all_gather(b):
            out_ = [None] * world
            dist.all_gather_object(out_, b)
            return out_
        comm = tp.make_comm(ctx, rank, world, cfg.hidden, all_gather)
    model = M.Model(ctx, cfg, rank, world)
    if comm is not None:
        tp.attach(model, comm)
    model.fill_synthetic(args.seed)
    prefill_rec = None
    if args.prefill and world == 1:
        # the state is PRODUCED by the model: a seeded random token stream of 4096 tokens through the prompt pass
        prompt = (lb.fill_u32(CTX_PREFILL, args.seed, 500000) % cfg.vocab).astype(np.int64).tolist()
        model.prefill(prompt[:256])                      # untimed: allocates the prompt-pass buffers, loads the kernels
        model.reset_state()
        ctx.sync()
        t_p = time.perf_counter()
        model.prefill(prompt)
        ctx.sync()
        t_p = time.perf_counter() - t_p
        prefill_rec = {"tokens": CTX_PREFILL, "seconds": round(t_p, 3), "tok_s": round(CTX_PREFILL / t_p, 1),
                       "how": "lb_model_prefill: 16 chunks of 256 tokens, batched int4 projections (tcgen05, 128 columns x 256 tokens per product), recurrence on chip per chunk, causal tensor-core attention per chunk"}
    else:
        model.seed_state(CTX_PREFILL, args.seed)     # ONE global seeded state; every rank takes its heads of it
    model.checkpoint()                           # the recurrent state is restored before every measured pass
    build_s = time.perf_counter() - t0
    if args.no_chain:
        model.set_chain(False)
    model.capture()
    kernels_per_step = model.step_kernels

    # clock ramp (untimed, not one of the W warm-up steps), then W warm-up steps
    # (every rank must replay the same number of steps: the ramp is sized from a step time all ranks agree on)
    model.set_input(1, CTX_PREFILL)
    t_ramp = time.perf_counter()
    model.replay(4)
    ctx.sync()
    t4 = max_over_ranks(dist, time.perf_counter() - t_ramp)
    for _ in range(min(2000, int(args.ramp_s / max(t4 / 4, 1e-4))) // 4):
        model.set_input(1, CTX_PREFILL)
        model.replay(4)
    ctx.sync()
    # parity pass (untimed): the first 16 greedy tokens from (token 1, position 4096) on the restored state.  They do not
    # depend on N (tensor-parallel shards of ONE model and ONE state) nor on how long the ramp ran.
    model.rollback()
    model.set_input(1, CTX_PREFILL)
    first_tokens = []
    for _ in range(16):
        model.replay(1)
        first_tokens.append(int(model.read_next()))
    lhash = logits_hash(model.logits())
    if dist is not None:
        hs = [None] * world
        dist.all_gather_object(hs, lhash)
        lhash = "+".join(hs)
    model.rollback()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    model.set_input(1, CTX_PREFILL)
    model.replay(args.warmup)
    ctx.sync()
    barrier(dist)
    ctx.reset_launches()
    ctx.timer_start()
    model.replay(args.steps)          # K decode steps back to back: each consumes the previous step's token
    ms = ctx.timer_stop()
    barrier(dist)
    launches = ctx.launches
    last_token = model.read_next()
    ms = max_over_ranks(dist, ms)
    clocks = sampler.stop() if rank == 0 else None

    # end to end through the public call: token id in (H2D), next token out (D2H), every step
    model.rollback()
    tok, e2e_steps = 1, max(16, min(args.steps, 64))
    model.set_input(tok, CTX_PREFILL)
    model.replay(2); ctx.sync()
    tok = model.read_next()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        model.set_input(tok, CTX_PREFILL + 2 + i)
        model.replay(1)
        tok = model.read_next()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = max_over_ranks(dist, e2e_s)

    step_s = ms * 1e-3 / args.steps
    algo_step = decode_algorithmic_bytes(cfg, model.weight_bytes, CTX_PREFILL) if world == 1 else None
    if world > 1:   # whole-job bytes: every rank streams its shard
        import torch
        t_ = torch.tensor([float(model.weight_bytes)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t_)
        algo_step = decode_algorithmic_bytes(cfg, int(t_.item()), CTX_PREFILL)
    peak, which = measured_hbm_peak()
    chained = not args.no_chain
    gemv_s, gemv_algo, _ = time_gemv_mix(ctx, lb, cfg, args, world, chained=chained)
    out = {
        "metric": METRIC, "value": 1.0 / step_s,
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 weights, fp16 activations (exact integer dot products), fp32 state", "data": "synthetic",
        "config": {"workload": (WORKLOAD if cfg.n_layers == 64 else WORKLOAD.replace("64-layer", f"{cfg.n_layers}-layer")).replace(
                       "by seeded fill", "by the prompt pass over a seeded random token stream" if prefill_rec else "by seeded fill"),
                   "parallelism": f"tp{world}", "l2": f"every step streams {algo_step / 1e9:.2f} GB of weights/state (>> 126 MB L2)",
                   "kernels_per_step": kernels_per_step, "build_seconds": round(build_s, 1), "last_token": int(last_token)},
        "prefill": prefill_rec,
        "parity": {"first_tokens": first_tokens, "logits_hash_after_16": lhash,
                   "what": "greedy tokens of the first 16 steps from (token 1, position 4096) on the seeded state: the same list at every N "
                           "is the tensor-parallel parity (TP=n tokens == TP=1 tokens); at N=1 the first of them are also checked against the CPU oracle"},
        "e2e": {"value": 1.0 / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches),
        "step_roofline": {"algorithmic_bytes_per_step": algo_step, "achieved_GBs": algo_step / step_s / 1e9, "peak_GBs": peak * world,
                          "frac": algo_step / step_s / 1e9 / (peak * world), "tok_s_at_peak": peak * world * 1e9 / algo_step},
        "roofline": {"bound": "hbm", "achieved": gemv_algo / gemv_s / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": gemv_algo / gemv_s / 1e9 / peak,
                     "traffic": chain_traffic_bytes(lb) if chained and world == 1 else None, "peak_source": which,
                     "kernel": "gemv_chain" if chained else "gemv_int4_w256",
                     "us_per_launch": gemv_s * 1e6, "algorithmic_bytes": gemv_algo,
                     "how": ("the step's four int4 GEMVs between two token mixers (out, gate/up + SwiGLU, down, next input projection; fused norm "
                             "prologues) as ONE persistent gemv_chain launch, 12 launches over rotating weights replayed alone as a graph; bytes = "
                             "the four matrices in the reference format") if chained else
                            "this GPU's int4 GEMV launch mix of the step (4 shapes x 12 layers, fused prologues/epilogues) replayed alone as a graph"},
        "clocks": clocks,
    }
    model.close()
    if comm is not None:
        barrier(dist)
        comm.close()
    if world == 1 and not args.no_small and cfg.n_layers == 64:
        out.update(bench_small_configs(ctx, lb))
    ctx.close()
    if rank == 0 and not args.no_cpu and world == 1 and cfg.n_layers == 64 and not prefill_rec:
        toks, dt, cores, b_s = oracle_decode_run(args.seed, CTX_PREFILL, 1, 2)
        out["cpu_baseline"] = {"value": 1.0 / dt, "unit": "tok/s", "cores": cores, "kind": "port",
                               "sample": f"3 full decode steps (64 layers + LM head) of the same seeded model and state with the C oracle (OpenMP, {cores} "
                                         f"threads): 1 warm-up + 2 timed, {dt * 1e3:.0f} ms per step; building the model on the host took {b_s:.0f} s"}
        out["parity"]["oracle_first_tokens"] = [int(t) for t in toks]
        out["parity"]["matches_oracle"] = first_tokens[:len(toks)] == [int(t) for t in toks]
    return out


def bench_prompt_chunks(args, local):
    """--workload prompt: two chunks of 256 prompt tokens at positions 3584..4095 through 8 layers of the benchmark's widths
    (6 DeltaNet + 2 attention, vocabulary 4096; 1.6 GB on the device): the small case the prompt pass is profiled on.  The
    caches below the chunk hold zeros (the time of a chunk does not depend on their values)."""
    import lithos_b200 as lb
    from lithos_b200 import model as M
    full = M.qwen35_27b(max_ctx=4224, n_layers=8)
    cfg = M.ModelCfg(**{**{n: getattr(full, n) for n, _ in M.ModelCfg._fields_}, "vocab": 4096})
    ctx = lb.Context(local)
    m = M.Model(ctx, cfg)
    m.fill_synthetic(3)
    toks = [int(t) for t in lb.fill_u32(512, 3, 999) % cfg.vocab]
    m.prefill(toks[:256], pos0=0)          # untimed: allocates the prompt-pass buffers, loads the kernels
    best = None
    for _ in range(max(1, min(args.steps, 10))):
        ctx.sync()
        t0 = time.perf_counter()
        m.prefill(toks, pos0=3584)
        ctx.sync()
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    m.close()
    ctx.close()
    return {"metric": "prompt pass, 512 tokens at a 4k context through 8 layers", "value": round(best * 1e3, 3), "unit": "ms", "n_gpus": 1,
            "higher_is_better": False, "data": "synthetic", "timing": "host clock around lb_model_prefill + synchronize, best of the repeats",
            "config": {"workload": "2 chunks x 256 tokens, positions 3584..4095, 6 DeltaNet + 2 attention layers of the 27B widths, vocabulary 4096"}}


def bench_chain(args, local):
    """--workload chain: gemv_chain on the decode step's GEMV mix, alone (1.2 GB on the device)"""
    import lithos_b200 as lb
    from lithos_b200 import model as M
    ctx = lb.Context(local)
    cfg = M.qwen35_27b(max_ctx=64)
    s_, algo, n = time_gemv_mix(ctx, lb, cfg, args, 1, chained=True)
    peak, which = measured_hbm_peak()
    out = {"metric": "gemv_chain launch (4 int4 GEMVs of one layer)", "value": s_ * 1e6, "unit": "us", "n_gpus": 1,
           "higher_is_better": False, "data": "synthetic", "launches_timed": n,
           "roofline": {"bound": "hbm", "achieved": algo / s_ / 1e9, "peak": peak, "unit": "GB/s", "frac": algo / s_ / 1e9 / peak,
                        "peak_source": which, "kernel": "gemv_chain", "algorithmic_bytes": algo}}
    ctx.close()
    return out


def bench_timeline(args, rank, local, world, dist):
    """--workload timeline: where the time of one persistent-chain launch goes, per kind of entry, from the %globaltimer
    stamps of lb_set_chain_timeline (no profiler).  Three DeltaNet layers of the benchmark's widths (one chain launch of 12
    entries: per layer input projection, mixer, out projection, gate/up, down; under tensor parallelism the out and down
    projections carry the exchange in their epilogue) decoded at position 4096; the stamps of the last of 40 replays are
    read on every rank, rank 0 prints medians over the SMs in microseconds.  Intervals inside an entry come from the SM's
    cycle counter; one %globaltimer stamp per entry gives the skew between the SMs and the cycle time."""
    import lithos_b200 as lb
    from lithos_b200 import model as M
    from lithos_b200 import tp
    cfg = M.qwen35_27b(max_ctx=CTX_PREFILL + 64, n_layers=3)
    cfg.vocab = 8192
    ctx = lb.Context(local)
    comm = None
    if world > 1:
        def all_gather(b):
            out_ = [None] * world
            dist.all_gather_object(out_, b)
            return out_
        comm = tp.make_comm(ctx, rank, world, cfg.hidden, all_gather)
    model = M.Model(ctx, cfg, rank, world)
    if comm is not None:
        tp.attach(model, comm)
    model.fill_synthetic(args.seed)
    model.seed_state(CTX_PREFILL, args.seed)
    sms, MAXOPS = ctx.sm_count, 32
    tl = ctx.alloc(sms * MAXOPS * 8 * 8).zero()
    lb.lib().lb_set_chain_timeline(ctx.h, tl.ptr)
    model.capture()
    lb.lib().lb_set_chain_timeline(ctx.h, 0)
    barrier(dist)
    model.set_input(1, CTX_PREFILL)
    model.replay(40)
    ctx.sync()
    barrier(dist)
    t = tl.download(np.uint64, sms * MAXOPS * 8).reshape(sms, MAXOPS, 8).astype(np.int64)
    names = ["input projection (5120 -> 16384/tp, RMSNorm prologue)", "DeltaNet mixer", "out projection (6144/tp -> 5120, head norm + gate prologue" + (", exchange" if world > 1 else "") + ")",
             "gate/up projection (5120 -> 34816/tp, RMSNorm prologue, SwiGLU)", "down projection (17408/tp -> 5120" + (", exchange" if world > 1 else "") + ")"]
    rows = []
    n_ops = 15
    if not (t[:, :n_ops, 0] > 0).all() or (t[:, n_ops, 0] != 0).any():
        raise SystemExit("timeline: the three layers did not run as one launch of %d entries" % n_ops)
    # stamp [0] is %globaltimer (ns), [1..7] the SM's cycle counter: ns per cycle of every SM from the first and the last entry
    ns_per_cyc = (t[:, n_ops - 1, 0] - t[:, 0, 0]) / np.maximum(t[:, n_ops - 1, 1] - t[:, 0, 1], 1)
    us = lambda cyc: float(np.median(cyc * ns_per_cyc)) / 1e3
    for o in range(n_ops):
        e = t[:, o, :]
        kind = o % 5
        rec = {"entry": o, "kind": names[kind], "arrival_skew_us": round(float(e[:, 0].max() - e[:, 0].min()) / 1e3, 2),
               "barrier_us": round(us(e[:, 2] - e[:, 1]), 2)}
        if kind == 1:
            rec.update({"mixer_us": round(us(e[:, 7] - e[:, 2]), 2)})
        else:
            rec.update({"input_wait_us": round(us(e[:, 3] - e[:, 2]), 2), "table_us": round(us(e[:, 4] - e[:, 3]), 2),
                        "body_us": round(us(e[:, 5] - e[:, 4]), 2), "column_sum_us": round(us(e[:, 6] - e[:, 5]), 2),
                        "store_exchange_us": round(us(e[:, 7] - e[:, 6]), 2)})
        rec["entry_total_us"] = round(us(e[:, 7] - e[:, 1]), 2)
        rows.append(rec)
    last = t[:, n_ops - 1, :]
    total = float((last[:, 0] + (last[:, 7] - last[:, 1]) * ns_per_cyc).max() - t[:, 0, 0].min()) / 1e3
    by_kind = {}
    for r_ in rows[5:]:      # layers 2 and 3: the first layer of the launch starts without a barrier
        k = by_kind.setdefault(r_["kind"], {"n": 0})
        for f, v in r_.items():
            if f.endswith("_us"):
                k[f] = k.get(f, 0.0) + v
        k["n"] += 1
    for k in by_kind.values():
        n = k.pop("n")
        for f in k:
            k[f] = round(k[f] / n, 2)
    out = {"metric": "persistent-chain timeline (3 DeltaNet layers, one launch)", "unit": "us", "n_gpus": world, "launch_total_us": round(total, 1),
           "per_layer_us": round(total / 3, 1), "by_kind_mean_of_layers_2_3": by_kind, "entries": rows}
    model.close()
    if comm is not None:
        barrier(dist)
        comm.close()
    ctx.close()
    return out


def bench_batched(args, local):
    """--workload batched: the batched int4 projection sweep (BASELINE config 4): the four projection shapes of the
    model at batch 1 / 4 / 16 / 64, fp16 N(0,1) activations, each launch reading a weight set that is not in L2
    (the sets of a shape rotate and together exceed the 126 MB L2).  One JSON line with one record per
    (shape, batch): microseconds per launch and algorithmic GB/s (weights + scales + zero-points + X + Y)."""
    import lithos_b200 as lb
    ctx = lb.Context(local)
    peak, which = measured_hbm_peak()
    shapes = [("gate_up 5120->17408", 5120, 17408, 8), ("down 17408->5120", 17408, 5120, 8),
              ("qkv 5120->22528", 5120, 22528, 6), ("lm_head 5120->248320", 5120, 248320, 1)]
    reps = 24
    sweep = []
    only = [w for w in args.batched_shapes.split(",") if w]
    batches = [int(b) for b in args.batched_batches.split(",")]
    for name, K, N, sets in shapes:
        if only and not any(w in name for w in only):
            continue
        dev = []
        for s_ in range(sets):
            dev.append([ctx.to_device(lb.fill_u32(K // 8 * N, 300 + s_, 1)), ctx.to_device(lb.fill_scales_f16(K // 128 * N, 300 + s_, 2)),
                        ctx.to_device(lb.fill_u32(K // 128 * (N // 8), 300 + s_, 3))])
        wbytes = K // 8 * N * 4 + K // 128 * N * 2 + K // 128 * (N // 8) * 4
        d_x = ctx.to_device(lb.fill_normal(max(batches + [128]) * K, 300, 4, dtype="f16"))
        d_y = ctx.alloc(max(batches + [128]) * N * 4)
        for B, flag in [(B, f) for B in batches for f in ((lb.GEMM_TCGEN05,) if B > 64 else (lb.GEMM_TCGEN05, lb.GEMM_MMA_SYNC) if B > 8 else (0, lb.GEMM_MMA_SYNC) if B == 1 else (0,))]:
            ctx.begin_capture()
            for j in range(reps):
                w = dev[j % sets]
                ctx.gemm_int4(w[0], w[1], w[2], d_x, d_y, K, N, B, lb.GEMV_Y_F32 | flag)
            graph = ctx.end_capture()
            for _ in range(max(args.warmup, 3)):
                graph.launch()
            ctx.sync()
            n = max(2, min(args.steps, 2000) // 50)
            ctx.timer_start()
            for _ in range(n):
                graph.launch()
            us = ctx.timer_stop() * 1e3 / (n * reps)
            algo = wbytes + B * K * 2 + B * N * 4
            sweep.append({"shape": name, "K": K, "N": N, "batch": B, "path": "tcgen05" if flag == lb.GEMM_TCGEN05 else "mma.sync" if (B > 1 or flag) else "gemv", "default": (flag == lb.GEMM_TCGEN05) == (B > 32) if B > 8 else flag == 0,
                          "us": round(us, 2), "GBps": round(algo / us / 1e3, 1),
                          "frac_of_hbm_peak": round(algo / us / 1e3 / peak, 3), "TFLOPs": round(2.0 * B * K * N / us / 1e6, 1)})
            graph.destroy()
            assert ctx.device_status() == 0
        for w in dev:
            for b in w:
                b.free()
        d_x.free()
        d_y.free()
    ctx.close()
    return {"metric": "batched int4 projection sweep (config 4)", "unit": "us per launch", "n_gpus": 1, "data": "synthetic",
            "higher_is_better": False, "dtype": "int4 weights, fp16 activations, fp32 accumulation", "peak": peak, "peak_source": which,
            "kernels": "gemm_int4_tc_ta (tcgen05.mma 128 x NT x 16, accumulator and dequantised weights in TMEM), gemm_int4_mma_b8/b16/b32/b64 (mma.sync m16n8k16)", "l2": "weight sets of a shape rotate, together > L2", "sweep": sweep}


def reference_decode(args, rank):
    """--impl reference: the reference's kernels have no CPU implementation that can run (its interpreters evaluate the
    integer host dialect only), so this arm times the plain-C restatement (oracle/, OpenMP over the host cores) on the SAME
    workload: W warm-up + K timed full decode steps, all 64 layers + LM head, same seeded model and state."""
    toks, dt, cores, b_s = oracle_decode_run(args.seed, CTX_PREFILL, args.warmup, args.steps)
    v = 1.0 / dt
    return {"impl": "reference", "metric": METRIC, "value": v, "unit": "tok/s", "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp32 (int4 weights, fp16 activations)",
            "data": "synthetic", "config": {"workload": WORKLOAD, "parallelism": f"{cores} host threads", "build_seconds": round(b_s, 1), "last_token": int(toks[-1])},
            "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port",
                             "sample": f"{args.warmup} warm-up + {args.steps} timed full decode steps (64 layers + LM head) with the C oracle, OpenMP, {cores} threads"},
            "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "gemv", "chain", "batched", "timeline", "small", "prompt"],
                    help="decode: the benchmark; gemv: config 0 alone; chain: the decode step's four GEMVs between two token "
                         "mixers as persistent gemv_chain launches alone (the small case used for ncu captures); small: the "
                         "one-figure measurements of configs 0, 1 and 2 alone (the ncu target for the DeltaNet and attention kernels)")
    ap.add_argument("--layers", type=int, default=64, help="decode workload: number of layers (64 = the benchmark definition)")
    ap.add_argument("--batched-shapes", default="", help="batched workload: comma-separated substrings of the shape names to run (default all)")
    ap.add_argument("--batched-batches", default="1,4,16,32,64,128,256", help="batched workload: batch sizes")
    ap.add_argument("--seed", type=int, default=20260413)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--prefill", action="store_true", help="decode workload, 1 GPU: build the 4096-token state by running a seeded random prompt through "
                    "lb_model_prefill instead of filling it directly; reports prompt tok/s (the CPU leg is skipped: the oracle would need 4096 steps)")
    ap.add_argument("--no-small", action="store_true", help="decode workload: skip the one-figure measurements of configs 0, 1 and 2")
    ap.add_argument("--no-chain", action="store_true", help="decode workload: one launch per projection instead of persistent chains")
    ap.add_argument("--ramp-s", type=float, default=1.5, help="seconds of untimed work before warm-up (clock ramp)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps is None:
        args.steps = (20 if args.impl == "reference" else 256) if args.workload == "decode" else 2000
    rank, local, world = dist_env()
    fix_omp_env(1 if args.impl == "reference" else world)   # before any OpenMP library is loaded
    if args.impl == "reference":
        if rank == 0:
            ref = reference_decode(args, rank) if args.workload == "decode" else reference_gemv(args, rank)
            print(json.dumps(ref), flush=True)
        return
    dist = init_dist(world)
    if args.workload == "timeline":
        out = bench_timeline(args, rank, local, world, dist)
        if rank == 0:
            print(json.dumps(out), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return
    if args.workload == "small":
        import lithos_b200 as lb
        ctx = lb.Context(local)
        out = bench_small_configs(ctx, lb)
        ctx.close()
        if rank == 0:
            print(json.dumps(out), flush=True)
        return
    if args.workload in ("chain", "batched", "prompt"):
        out = {"chain": bench_chain, "batched": bench_batched, "prompt": bench_prompt_chunks}[args.workload](args, local)
        if rank == 0:
            print(json.dumps(out), flush=True)
        return
    out = (bench_decode if args.workload == "decode" else bench_gemv)(args, rank, local, world, dist)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
