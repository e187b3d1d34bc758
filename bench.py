#!/usr/bin/env python3
"""Headline benchmark: HQ4_G32 dequant-GEMV effective HBM bandwidth (M = 1) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--sections LIST] [--case NAME]

One step = one decode GEMV y[1, N] = x[1, K] . W^T over one packed HQ4_G32 weight bank, N = 12288, K = 4096 (the
reference's own decode-race shape).  The timed loop rotates through enough distinct weight banks to exceed the 126 MB
L2 three times over, so every step streams its weights from HBM.  Synthetic data: W ~ N(0, 0.02) (seeded) quantized on
the device by the library's own packer; x ~ N(0, 1) f16.

`--impl reference` times the CPU restatement of the reference's path (oracle/) on the host cores for the same metric.
Prints ONE JSON line.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = {"name": "decode GEMV: HQ4_G32 N=12288 K=4096 M=1", "n": 12288, "k": 4096, "m": 1}
METRIC = "HQ4_G32 dequant-GEMV effective HBM bandwidth (M=1)"
UNIT = "GB/s"
L2_BYTES = 126 * 1024 * 1024
REPEATS = 7   # timed regions of `--steps` steps each; the line reports their median


def gemv_bytes(n, k, m, block_bytes=20, group=32, out_bytes=4):
    """Algorithmic bytes of one call: packed weights + activations + outputs."""
    return n * (k // group) * block_bytes + m * k * 2 + m * n * out_bytes


def bank_copies(n, k, block_bytes=20, group=32):
    per_bank = n * (k // group) * block_bytes
    return max(2, -(-3 * L2_BYTES // per_bank)), per_bank


def headline_config(world):
    """The same dictionary in both arms (ours and --impl reference)."""
    copies, per_bank = bank_copies(WORKLOAD["n"], WORKLOAD["k"])
    return {"workload": WORKLOAD["name"], "n": WORKLOAD["n"], "k": WORKLOAD["k"], "m": WORKLOAD["m"], "format": "HQ4_G32",
            "l2": f"rotation over distinct weight banks, larger than the caches together ({copies} banks = {copies * per_bank / 1e6:.0f} MB > 126 MB L2 on the device)",
            "parallelism": "1 GPU" if world == 1 else f"{world} replicas of the projection, one per rank (column-parallel shards, no collective)"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def count(self):
        return len(self.lines)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference's CPU path for this metric: the C restatement of its decode + group dot (the reference ships no
    fused CPU kernel; its own Python decode + numpy matmul takes seconds per call and is not timed here), OpenMP over
    rows on all host cores, over banks in rotation like the device arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import qw_oracle as qo
    qo.build()
    cores = qo.set_num_threads(host_cores())   # launchers export OMP_NUM_THREADS=1: ask for every core explicitly
    n, k, m = WORKLOAD["n"], WORKLOAD["k"], WORKLOAD["m"]
    rng = np.random.default_rng(1)
    copies = min(bank_copies(n, k)[0], 4)   # 4 banks = 126 MB: beyond the host's caches, quick to build
    banks = [qo.quantize(rng.normal(0.0, 0.02, (n, k)).astype(np.float32), qo.HQ4_G32) for _ in range(copies)]
    x = rng.standard_normal((m, k)).astype(np.float16)
    nbytes = gemv_bytes(n, k, m)
    for i in range(max(args.warmup, 1)):
        qo.matmul(banks[i % copies], qo.HQ4_G32, x)
    t0 = time.perf_counter()
    for i in range(args.steps):
        qo.matmul(banks[i % copies], qo.HQ4_G32, x)
    dt = time.perf_counter() - t0
    val = nbytes * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 weights x f16 activations, f64 accumulate", "data": "synthetic",
        "config": headline_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full GEMV calls of the workload over {copies} banks in rotation (C restatement of the "
                                   "reference's decode + group dot, OpenMP over rows; the reference's Python decode + numpy matmul is not timed)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
GRAPH_STEPS = 500   # calls per captured graph; a timed region of K steps replays it K // 500 times (+ one graph of K % 500)


def build_graphs(fn, steps):
    """CUDA graphs holding exactly `steps` calls of fn(i): the way a decode loop submits its kernels, so that the host's
    per-call cost (ctypes + launch, ~15 us from Python) is not what is measured.  One untimed replay of each."""
    import torch
    plan = []   # (graph, replays)
    side = torch.cuda.Stream()
    done = 0
    for size, reps in ((GRAPH_STEPS, steps // GRAPH_STEPS), (steps % GRAPH_STEPS, 1)):
        if size == 0 or reps == 0:
            continue
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(size):
                    fn(done + i)
        torch.cuda.synchronize()
        g.replay()
        plan.append((g, reps))
        done += size
    torch.cuda.synchronize()
    return plan


def time_region(fn, steps, dist, stream, graph=False, plan=None):
    """Barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks (ms).  Exactly `steps`
    calls run between the events (graph=True: as replays of the graphs of build_graphs)."""
    import torch
    if graph and plan is None:
        plan = build_graphs(fn, steps)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    if graph:
        for g, reps in plan:
            for _ in range(reps):
                g.replay()
    else:
        for i in range(steps):
            fn(i)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def make_banks(q, hal, n, k, container, copies, seed):
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    banks = []
    for _ in range(copies):
        w = torch.randn((n, k), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        bank = q.QWGemm.quantize(hal, w, container)
        banks.append(q.QWWeightView(bank, n, k, container))
        del w
    return banks


def bench_gemv_point(q, hal, n, k, m, cname, steps, warmup, dist=None, seed=0, rotated=False):
    """Device-resident timing of one (format, M) point; returns (ms_per_step, bytes_per_step, banks, x, y)."""
    import torch
    cont = q.CONTAINERS[cname]
    per_bank = n * cont.row_bytes(k)
    copies = max(2, -(-3 * L2_BYTES // per_bank))   # >= 3x L2 of distinct weights in rotation
    banks = make_banks(q, hal, n, k, cont, copies, seed)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed + 1000)
    x = torch.randn((m, k), generator=gen, device="cuda", dtype=torch.float32).to(torch.float16)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream()
    nws = q.QWGemm.workspaceBytes(hal, banks[0], m)
    ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None

    if rotated:   # the reference's dataflow: the norm kernel before the matmul hands over rotated activations
        q.QWGemm.encodeRMSNorm(hal, x.clone(), torch.zeros(k, dtype=torch.float16, device="cuda"), x)

    def step(i):
        q.QWGemm.encode(hal, banks[i % copies], x, y, workspace=ws, x_is_rotated=rotated)

    torch.cuda.synchronize()
    hal.set_static_weights(True)
    for i in range(warmup):
        step(i)
    ms = time_region(step, steps, dist, stream, graph=True)
    hal.set_static_weights(False)
    nbytes = gemv_bytes(n, k, m, cont.block_bytes, cont.group)
    return ms / steps, nbytes, banks, x, y


def profile_traffic(kernel, workload):
    """DRAM bytes per call from the committed ncu summary of this kernel on this workload; None (with the reason) when
    the summary on file is for another kernel or shape."""
    import re
    path = os.path.join(ROOT, "profiles", "qwc_gemv_stream_kernel_hq4g32_n12288_k4096_m1.md")
    if not os.path.exists(path):
        return None, "no ncu summary on file for this kernel and workload"
    text = open(path).read()
    mk, mw = re.search(r"^kernel:\s*(\S+)", text, re.M), re.search(r"^workload:\s*(.+)$", text, re.M)
    mt = re.search(r"dram_bytes_per_call:\s*(\d+)", text)
    if not (mk and mw and mt) or mk.group(1) != kernel or mw.group(1).strip() != workload:
        return None, "the ncu summary on file is for another kernel or workload"
    return int(mt.group(1)), os.path.relpath(path, ROOT)


def run_ours(args):
    import torch
    import qwegn_b200 as q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    hal = q.QWHal(local_rank)
    peaks = measured_peaks()
    n, k, m = WORKLOAD["n"], WORKLOAD["k"], WORKLOAD["m"]
    sections = set(args.sections.split(",")) if args.sections else {"sweep", "c1", "cpu", "prefill", "moe", "parallel"}

    # ---- headline: device-resident GEMV, weights rotating through > 3 x L2 of distinct banks ----------------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    cont = q.CONTAINERS["HQ4_G32"]
    copies, per_bank = bank_copies(n, k)
    banks = make_banks(q, hal, n, k, cont, copies, seed=rank)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)
    x = torch.randn((m, k), generator=gen, device="cuda", dtype=torch.float32).to(torch.float16)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream()

    def step(i):
        q.QWGemm.encode(hal, banks[i % copies], x, y)

    torch.cuda.synchronize()
    hal.set_static_weights(True)   # the banks are complete: from here on weights are load-time data, as in a decode loop
    sampler.start()                # samples SM clocks and throttle reasons from here to the end of the e2e region
    for i in range(args.warmup):
        step(i)
    plan = build_graphs(step, args.steps)
    regions = [time_region(step, args.steps, dist, stream, graph=True, plan=plan) for _ in range(REPEATS)]
    ms = statistics.median(regions)
    nbytes = gemv_bytes(n, k, m)
    ms_per_step = ms / args.steps
    value = world * nbytes / (ms_per_step * 1e-3) / 1e9
    del plan

    # ---- end to end through the public API with host buffers: H2D of x and D2H of y inside the timed region ----
    x_host = x.cpu().pin_memory()
    y_host = torch.empty((m, n), dtype=torch.float32).pin_memory()
    x_dev = torch.empty_like(x)

    hal.set_static_weights(False)   # every e2e step ends in a synchronize: nothing to overlap with
    # One CUDA graph per weight bank: H2D copy of x, the GEMV, D2H copy of y.  A step = one replay + a stream
    # synchronize (the caller reads y on the host every step); the graphs only remove Python's per-call cost.
    side = torch.cuda.Stream()
    e2e_graphs = []
    for b in range(copies):
        g = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                x_dev.copy_(x_host, non_blocking=True)
                q.QWGemm.encode(hal, banks[b], x_dev, y)
                y_host.copy_(y, non_blocking=True)
        e2e_graphs.append(g)
    torch.cuda.synchronize()

    def step_e2e(i):
        e2e_graphs[i % copies].replay()
        stream.synchronize()

    for i in range(max(args.warmup, copies)):
        step_e2e(i)
    ms_e2e = time_region(step_e2e, args.steps, dist, stream)
    e2e_val = world * nbytes / (ms_e2e / args.steps * 1e-3) / 1e9
    if sampler.count() < 5:
        # a short run (small --steps) ends before nvidia-smi has sampled: keep the same load up, untimed, for ~0.3 s
        t_end = time.perf_counter() + 0.3
        while time.perf_counter() < t_end:
            for i in range(200):
                step(i)
            torch.cuda.synchronize()
    clocks = sampler.stop()

    status = hal.device_status()
    achieved = nbytes / (ms_per_step * 1e-3) / 1e9
    traffic, traffic_src = profile_traffic("qwc_gemv_stream_kernel", f"n={n} k={k} m={m} HQ4_G32")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 (f16 weights decoded from u4, f16 activations, f32 accumulate)", "data": "synthetic",
        "config": headline_config(world),
        "method": {"launch": "the K calls are captured in CUDA graphs of <= 500 calls and replayed inside the timed region; static-weights "
                             "mode: programmatic dependent launch between calls and an L2 prefetch kernel per call that runs beside the previous call",
                   "timed_regions": REPEATS, "value_is": "median over the timed regions of K steps each",
                   "ms_per_step_regions": [round(r / args.steps, 6) for r in regions],
                   "spread": round((max(regions) - min(regions)) / ms, 4)},
        "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel() * 2),
                "d2h_bytes_per_step": int(y_host.numel() * 4), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": 2 * args.steps,   # per step: the L2 prefetch kernel and the stream kernel
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_src,
                     "peak_source": peaks["source"], "kernel": "qwc_gemv_stream_kernel<HQ4_G32_M5, M<=8> (+ qwc_gemv_prefetch_kernel)",
                     "algorithmic_bytes_per_launch": nbytes},
        "device_status": status,
    }

    hal.set_static_weights(False)   # the sections below build fresh banks on the same stream
    extra = {}
    if rank == 0 and world == 1:
        del banks, e2e_graphs
        torch.cuda.empty_cache()
        if "c1" in sections:
            t, b, *_ = bench_gemv_point(q, hal, 17408, 5120, 1, "HQ4_G32", args.steps, args.warmup)
            extra["c2_gemv_N17408_K5120_M1"] = {"GBps": b / (t * 1e-3) / 1e9, "us": t * 1e3, "frac_of_peak": b / (t * 1e-3) / 1e9 / peaks["hbm_gbs"]}
            torch.cuda.empty_cache()
            t, b, *_ = bench_gemv_point(q, hal, n, k, 1, "HQ4_G32", args.steps, args.warmup, rotated=True)
            extra["headline_with_rotated_activations_in"] = {"GBps": b / (t * 1e-3) / 1e9, "us": t * 1e3,
                                                             "note": "x_is_rotated=1: activations rotated by qwc_rmsnorm_fwht outside the timed loop, as in the reference's engine"}
            torch.cuda.empty_cache()
            extra["lm_head_greedy_N248320_K5120_M1"] = bench_lm_head(q, hal, peaks)
            torch.cuda.empty_cache()
            extra["f32_activation_door_N17408_K5120"] = bench_f32_door(q, hal, 17408, 5120, args.warmup)
            torch.cuda.empty_cache()
        if "sweep" in sections:
            sweep = {}
            for cname in ("HQ4_G32", "HQ8_G32", "HQ4_G64"):
                for mm in (1, 2, 4, 8, 16):
                    t, b, *_ = bench_gemv_point(q, hal, 17408, 5120, mm, cname, max(20, args.steps // 4), args.warmup)
                    sweep[f"{cname}_M{mm}"] = {"GBps": round(b / (t * 1e-3) / 1e9, 1), "us": round(t * 1e3, 2)}
                    torch.cuda.empty_cache()
            extra["verify_sweep_N17408_K5120"] = sweep
        if "prefill" in sections:
            extra["prefill_M4096"] = bench_prefill(q, hal, peaks)
        if "moe" in sections:
            extra["moe_T2048_E256_top8"] = bench_moe(q, hal, peaks)
        if "cpu" in sections:
            line["cpu_baseline"] = cpu_baseline(q, hal, n, k, m)
    if world > 1 and "parallel" in sections:
        par = bench_parallel(q, hal, rank, world, dist, peaks)
        if rank == 0:
            extra.update(par)
    if extra:
        line["extra"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def bench_lm_head(q, hal, peaks, steps=60):
    """Greedy LM head (the largest GEMV of a decode step): logits = HQ4_G32 [248320, 5120] x, then the key-ordered argmax.
    Two banks in rotation (1.6 GB > L2)."""
    import torch
    n, k = 248320, 5120
    cont = q.CONTAINERS["HQ4_G32"]
    banks = make_banks(q, hal, n, k, cont, 2, seed=5)
    x = torch.randn((1, k), device="cuda", dtype=torch.float32).to(torch.float16)
    y = torch.empty((1, n), dtype=torch.float32, device="cuda")
    tok = torch.empty(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream()

    def step(i):
        q.QWGemm.encode(hal, banks[i % 2], x, y)
        q.QWGemm.encodeArgmax(hal, y, tok)

    hal.set_static_weights(True)
    for i in range(4):
        step(i)
    ms = time_region(step, steps, None, stream, graph=True) / steps
    hal.set_static_weights(False)
    nbytes = gemv_bytes(n, k, 1)
    ref = int(torch.argmax(y[0]).item())
    return {"us": ms * 1e3, "GBps": nbytes / (ms * 1e-3) / 1e9, "frac_of_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "token_matches_torch_argmax": bool(int(tok.item()) == ref)}


def bench_f32_door(q, hal, n, k, warmup, steps=400):
    """The f32-activation door (rotated f32 rows in, f32 out): stage kernel + GEMV (+ epilogue kernel for the silu + FWHT
    epilogue).  Banks in rotation, larger than L2 together."""
    import torch
    cont = q.CONTAINERS["HQ4_G32"]
    nb = max(2, -(-3 * L2_BYTES // (n * (k // 32) * 20)))
    banks = make_banks(q, hal, n, k, cont, nb, seed=11)
    stream = torch.cuda.current_stream()
    out = {}
    torch.cuda.synchronize()
    hal.set_static_weights(True)   # the banks are complete
    for m, epi in ((1, 0), (1, 3), (4, 0)):
        x = torch.randn((m, k), device="cuda")
        y = torch.empty((m, n), device="cuda")
        ws = torch.empty(q.QWGemm.f32WorkspaceBytes(hal, banks[0], m, epi) + 256, dtype=torch.uint8, device="cuda")

        def step(i):
            q.QWGemm.encodeHQ4F32V4(hal, banks[i % nb], x, y, rows=m, epi=epi, scale=1.0, workspace=ws)

        for i in range(max(3, warmup)):
            step(i)
        ms = time_region(step, steps, None, stream, graph=True) / steps
        b = gemv_bytes(n, k, m)
        out[f"M{m}_epi{epi}"] = {"us": round(ms * 1e3, 2), "GBps": round(b / (ms * 1e-3) / 1e9, 1)}
    torch.cuda.synchronize()
    hal.set_static_weights(False)
    return out


def _time_call(fn, iters, warm=3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_prefill(q, hal, peaks):
    """Prefill GEMMs of one layer of the 27B-shaped dense transformer: M = 4096, hidden 5120, intermediate 17408,
    QKV width 7168; rotated f16 activations resident; f16 out.  TFLOP/s = 2 M N K / time (decode, SwiGLU, FWHT not
    counted)."""
    import torch
    out = {}
    m = 4096
    cases = {"gate_up_N34816_K5120": (34816, 5120, "HQ4_G32", 0), "down_N5120_K17408": (5120, 17408, "HQ4_G32", 0),
             "qkv_N7168_K5120": (7168, 5120, "HQ4_G32", 0), "qkv_N7168_K5120_HQ8_G32": (7168, 5120, "HQ8_G32", 0),
             "qkv_N7168_K5120_HQ4_G64": (7168, 5120, "HQ4_G64", 0),
             "gate_up_fused_swiglu_fwht_N34816_K5120": (34816, 5120, "HQ4_G32", q.EPI_SILU_PAIR_FWHT)}
    for name, (n, k, cname, epi) in cases.items():
        cont = q.CONTAINERS[cname]
        w = torch.randn((n, k), device="cuda", dtype=torch.float32) * 0.02
        view = q.QWWeightView(q.QWGemm.quantize(hal, w, cont), n, k, cont)
        del w
        x = torch.randn((m, k), device="cuda", dtype=torch.float32).to(torch.float16)
        q.QWGemm.encodeFwht32(hal, x)
        y = torch.empty((m, n if epi == 0 else n // 2), dtype=torch.float16, device="cuda")
        ms = _time_call(lambda: q.QWGemm.encode(hal, view, x, y, epi=epi, x_is_rotated=True), 10)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out[name] = {"ms": round(ms, 4), "TFLOPs": round(tf, 1), "frac_of_burst_peak": round(tf / peaks["bf16_tflops"], 3),
                     "frac_of_sustained_peak": round(tf / peaks["bf16_tflops_sustained"], 3)}
        del view, x, y
        torch.cuda.empty_cache()
    return out


def bench_moe(q, hal, peaks):
    """The 35B-A3B-shaped sparse MoE block: 2048 tokens, 256 experts, top-8, hidden 2048, expert intermediate 512,
    HQ4_G32; router logits N(0, 1); the whole operator chain (route .. combine) per step, submitted as CUDA graphs (8
    different routings in rotation)."""
    import torch
    t, e, k, h, inter = 2048, 256, 8, 2048, 512
    cont = q.CONTAINERS["HQ4_G32"]
    gu = q.QWGemm.quantize(hal, torch.randn((e * 2 * inter, h), device="cuda") * 0.02, cont)
    dn = q.QWGemm.quantize(hal, torch.randn((e * h, inter), device="cuda") * 0.02, cont)
    op = q.QWMoEOperator(hal, q.QWWeightView(gu, e * 2 * inter, h, cont), q.QWWeightView(dn, e * h, inter, cont), e, inter, k)
    x = torch.randn((t, h), device="cuda").to(torch.float16)
    lgs = [torch.randn((t, e), device="cuda") for _ in range(8)]
    outp = torch.empty((t, h), device="cuda")
    sc = torch.empty(op.scratchBytes(t), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    for i in range(3):
        op.encodeResident(x, lgs[i], outp, sc)
    ms = time_region(lambda i: op.encodeResident(x, lgs[i % 8], outp, sc), 80, None, stream, graph=True) / 80
    flops = 2.0 * t * k * (2 * inter * h + h * inter)
    wbytes = e * (2 * inter * (h // 32) * 20 + h * (inter // 32) * 20)
    # the decode / verify size of the same block (8 tokens = 64 pairs, up to 64 experts touched): per-expert streaming
    # GEMVs; CUDA-graph replay, weights declared static, 16 routings in rotation so that the experts touched differ
    x8, out8 = x[:8].contiguous(), torch.empty((8, h), device="cuda")
    lg8 = [torch.randn((8, e), device="cuda") for _ in range(16)]
    torch.cuda.synchronize()
    hal.set_static_weights(True)
    for i in range(3):
        op.encodeResident(x8, lg8[i], out8, sc)
    ms8 = time_region(lambda i: op.encodeResident(x8, lg8[i % 16], out8, sc), 320, None, stream, graph=True) / 320
    torch.cuda.synchronize()
    hal.set_static_weights(False)
    tf = flops / (ms * 1e-3) / 1e12
    return {"us": round(ms * 1e3, 1), "TFLOPs": round(tf, 1), "frac_of_burst_tensor_peak": round(tf / peaks["bf16_tflops"], 3),
            "weight_GBps": round(wbytes / (ms * 1e-3) / 1e9, 1), "frac_of_hbm_peak": round(wbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
            "decode_T8_us": round(ms8 * 1e3, 1),
            "bound": "the HBM roof (503 MB of expert weights: ~78 us) and the tensor roof (~65 us) are close; neither binds yet: with ~64 "
                     "tokens per expert every decoded 128 x 64 weight tile feeds one short MMA, and the MMA warp's turn per operand "
                     "stage (barrier wait, fences, eight short MMAs, commit: ~0.4 us per 128 k per SM, with the copies into shared "
                     "memory on its critical path) sets the pace, not the decode"}


def _max_rel_and_cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    err = float((a - b).abs().max() / (b.abs().max() + 1e-30))
    cos = float((a * b).sum() / (a.norm() * b.norm() + 1e-30))
    return err, cos


def bench_parallel(q, hal, rank, world, dist, peaks):
    """Tensor-parallel and expert-parallel steps at N > 1, each checked on EVERY rank against the single-device result of
    the same call before it is timed (a failed check fails the run), each timed as the max over ranks.
      * TP MLP decode (hidden 8192, intermediate 28672, HQ4_G32, M = 1): NCCL all-reduce and the fused matmul + all-reduce.
      * The 70B-class layer stack: 8 layers of hidden 8192 / intermediate 28672 / 64 query + 8 KV heads of 128, HQ8_G32
        attention projections + HQ4_G32 MLP, two all-reduces per layer, at M = 1 (CUDA graph, fused all-reduces) and at
        M = 8192 (NCCL all-reduces of token chunks overlapped with the matmuls), with the same stack on ONE GPU timed in
        the same run (every rank runs it; max over ranks) as the strong-scaling anchor.
      * Expert-parallel MoE (2048 tokens and 256 experts sharded over the ranks): peer-store dispatch / return
        (qwc_ep_moe) and the NCCL all-to-all form, against the single-device block."""
    import torch
    from qwegn_b200 import parallel as par
    out = {}
    stream = torch.cuda.current_stream()

    def tmax(ms):
        tt = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def all_ok(flag):
        tt = torch.tensor([1 if flag else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MIN)
        return bool(tt.item())

    def check(name, got, ref, bits_equal_across_ranks=False, recompute=None):
        """Parity of `got` against the single-device `ref` on every rank.  A mismatch fails the run, except that a caller may
        pass `recompute` (runs the same call again into `got`): one mismatch that does not repeat is then reported in the
        entry (`first_attempt`) instead of ending the run -- a second mismatch ends it."""
        first = None
        for attempt in (0, 1):
            err, cos = _max_rel_and_cos(got, ref)
            ok = err <= 1e-2 and cos >= 0.9999
            if bits_equal_across_ranks:
                gathered = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(gathered, got.contiguous())
                ok = ok and all(torch.equal(gathered[0], g) for g in gathered)
            ok = all_ok(ok)
            if ok:
                entry = {"parity_ok": True, "max_rel_err": round(err, 6), "cosine": round(cos, 7)}
                if first is not None:
                    entry["first_attempt"] = first
                return entry
            where = ""
            if got.dim() == 2 and got.shape == ref.shape:   # which rows are off: says whether a chunk, a rank's share or everything is wrong
                d = (got.double() - ref.double()).abs()
                bad = (d > 1e-2 * float(ref.double().abs().max())).any(dim=1).nonzero().flatten()
                if bad.numel():
                    where = f"; {bad.numel()} of {got.shape[0]} rows off, first {int(bad[0])}, last {int(bad[-1])}"
            msg = (f"parity check failed on rank {rank}: {name}: max-rel {err:.3e}, cosine {cos:.6f}{where}; "
                   f"kernel status word {hal.device_status()}")
            if attempt == 1 or recompute is None:
                raise RuntimeError(msg)
            first = {"parity_ok": False, "max_rel_err": round(err, 6), "cosine": round(cos, 7), "where": where.lstrip("; "),
                     "note": "the same call was run a second time and checked again"}
            print(msg + " -- running the call once more", file=sys.stderr, flush=True)
            recompute()
            torch.cuda.synchronize()
            dist.barrier()

    hq4, hq8 = q.CONTAINERS["HQ4_G32"], q.CONTAINERS["HQ8_G32"]
    hidden, inter, qh, kvh, hd, nlayers = 8192, 28672, 64, 8, 128, 8
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)   # the same planes on every rank; each keeps its shard

    def plane(n, k, cont):
        return q.QWGemm.quantize(hal, torch.randn((n, k), generator=gen, device="cuda") * 0.02, cont)

    # ---- TP MLP decode: NCCL all-reduce vs the fused kernel -------------------------------------------------------
    gu_plane, dn_plane = plane(2 * inter, hidden, hq4), plane(hidden, inter, hq4)
    x1 = torch.randn((1, hidden), generator=gen, device="cuda").to(torch.float16)
    ref_mlp = par.TPMlp(hal, gu_plane, dn_plane, hidden, inter, hq4, 0, 1)
    h_ref = torch.empty((1, inter), dtype=torch.float16, device="cuda")
    y_ref = torch.empty((1, hidden), dtype=torch.float32, device="cuda")
    ref_mlp.forward(x1, h_ref, y_ref)
    wbytes = (2 * inter * (hidden // 32) + hidden * (inter // 32)) * 20
    torch.cuda.synchronize()
    hal.set_static_weights(True)
    ms_ref = tmax(time_region(lambda i: ref_mlp.forward(x1, h_ref, y_ref), 40, None, stream, graph=True) / 40)
    out["tp1_mlp_decode_M1_H8192_I28672"] = {"us": round(ms_ref * 1e3, 1), "weight_GBps": round(wbytes / (ms_ref * 1e-3) / 1e9, 1),
                                             "note": "the unsharded MLP on one GPU (every rank runs it; max over ranks)"}
    hal.set_static_weights(False)
    del ref_mlp
    for label, fused in (("nccl_allreduce", False), ("fused_allreduce", True)):
        mlp = par.TPMlp(hal, gu_plane, dn_plane, hidden, inter, hq4, rank, world, fused_allreduce=fused)
        h_loc = torch.empty((1, mlp.inter_local), dtype=torch.float16, device="cuda")
        y = torch.empty((1, hidden), dtype=torch.float32, device="cuda")
        mlp.forward(x1, h_loc, y)
        entry = check(f"tp mlp {label}", y, y_ref, bits_equal_across_ranks=fused)
        torch.cuda.synchronize()
        dist.barrier()
        hal.set_static_weights(True)
        ms = time_region(lambda i: mlp.forward(x1, h_loc, y), 40, dist, stream, graph=True) / 40
        hal.set_static_weights(False)
        entry.update({"graph_us": round(ms * 1e3, 1), "graph_aggregate_weight_GBps": round(wbytes / (ms * 1e-3) / 1e9, 1),
                      "strong_scaling_efficiency": round(ms_ref / ms / world, 3)})
        out[f"tp{world}_mlp_decode_M1_H8192_I28672_{label}"] = entry
        del mlp
        torch.cuda.empty_cache()
    del gu_plane, dn_plane
    torch.cuda.empty_cache()

    # ---- the layer stack ------------------------------------------------------------------------------------------
    qn, kvn = qh * hd, kvh * hd
    planes = [{"qkv": plane(qn + 2 * kvn, hidden, hq8), "o": plane(hidden, qn, hq8), "gate_up": plane(2 * inter, hidden, hq4),
               "down": plane(hidden, inter, hq4)} for _ in range(nlayers)]
    layer_bytes = sum(int(p.numel()) for p in planes[0].values())
    layer_flops = 2.0 * hidden * (qn + 2 * kvn + qn + 3 * inter)

    def build(rk, wd, fused):
        return par.TPLayerStack([par.TPLayer(hal, pl, hidden, inter, qh, kvh, hd, hq8, hq4, rk, wd, fused_allreduce=fused)
                                 for pl in planes], hal)

    one = build(0, 1, False)
    tp = build(rank, world, True)
    for mtok, chunk in ((1, 0), (8192, 2048)):
        x0 = torch.randn((mtok, hidden), generator=gen, device="cuda").to(torch.float16)
        xn_a, res_a = torch.empty_like(x0), x0.clone()
        q.QWGemm.encodeRMSNorm(hal, x0, one.layers[0].gamma1, xn_a)
        xn_b, res_b = xn_a.clone(), res_a.clone()
        xn_in, res_in = xn_a.clone(), res_a.clone()
        buf_a, buf_b = one.buffers(mtok), tp.buffers(mtok)
        one.forward(xn_a, res_a, buf_a)
        tp.forward(xn_b, res_b, buf_b, chunk=chunk)
        torch.cuda.synchronize()

        def again():   # both sides of the comparison from the same inputs
            for xn, res in ((xn_a, res_a), (xn_b, res_b)):
                xn.copy_(xn_in)
                res.copy_(res_in)
            one.forward(xn_a, res_a, buf_a)
            tp.forward(xn_b, res_b, buf_b, chunk=chunk)

        entry = check(f"tp layer stack M={mtok}", res_b, res_a, recompute=again)

        def run_one(i):
            xn_a.copy_(xn_in)
            res_a.copy_(res_in)
            one.forward(xn_a, res_a, buf_a)

        def run_tp(i):
            xn_b.copy_(xn_in)
            res_b.copy_(res_in)
            tp.forward(xn_b, res_b, buf_b, chunk=chunk)

        iters = 20 if mtok == 1 else 3
        hal.set_static_weights(True)
        dist.barrier()
        if mtok == 1:
            ms1 = tmax(time_region(run_one, iters, None, stream, graph=True) / iters)
            msn = time_region(run_tp, iters, dist, stream, graph=True) / iters
        else:   # the chunked prefill uses a second stream and NCCL: submitted eagerly (host time is small against ~100 ms)
            ms1 = tmax(time_region(run_one, iters, None, stream) / iters)
            msn = time_region(run_tp, iters, dist, stream) / iters
        hal.set_static_weights(False)
        key = f"tp{world}_layer_stack_8L_H8192_I28672_M{mtok}"
        entry.update({"ms": round(msn, 4), "one_gpu_ms": round(ms1, 4), "strong_scaling_efficiency": round(ms1 / msn / world, 3)})
        if mtok == 1:
            entry["aggregate_weight_GBps"] = round(nlayers * layer_bytes / (msn * 1e-3) / 1e9, 1)
            entry["one_gpu_weight_GBps"] = round(nlayers * layer_bytes / (ms1 * 1e-3) / 1e9, 1)
        else:
            entry["aggregate_TFLOPs"] = round(nlayers * layer_flops * mtok / (msn * 1e-3) / 1e12, 1)
            entry["one_gpu_TFLOPs"] = round(nlayers * layer_flops * mtok / (ms1 * 1e-3) / 1e12, 1)
            entry["chunk_tokens"] = chunk
        out[key] = entry
        del buf_a, buf_b, xn_a, xn_b, res_a, res_b, x0
        torch.cuda.empty_cache()
    del one, tp, planes
    torch.cuda.empty_cache()

    # ---- expert parallel ------------------------------------------------------------------------------------------
    t, e, k, h, it = 2048, 256, 8, 2048, 512
    gu, dn = plane(e * 2 * it, h, hq4), plane(e * h, it, hq4)
    xs_all = torch.randn((t, h), generator=gen, device="cuda").to(torch.float16)
    lg_all = torch.randn((t, e), generator=gen, device="cuda")
    t0, t1 = t * rank // world, t * (rank + 1) // world
    xs, lg = xs_all[t0:t1].contiguous(), lg_all[t0:t1].contiguous()
    single = q.QWMoEOperator(hal, q.QWWeightView(gu, e * 2 * it, h, hq4), q.QWWeightView(dn, e * h, it, hq4), e, it, k)
    sc1 = torch.empty(single.scratchBytes(t), dtype=torch.uint8, device="cuda")
    out_all = torch.empty((t, h), device="cuda")
    single.encodeResident(xs_all, lg_all, out_all, sc1)
    ms1 = tmax(time_region(lambda i: single.encodeResident(xs_all, lg_all, out_all, sc1), 20, None, stream, graph=True) / 20)
    flops = 2.0 * t * k * (2 * it * h + h * it)
    out["ep1_moe_T2048_E256_top8"] = {"us": round(ms1 * 1e3, 1), "TFLOPs": round(flops / (ms1 * 1e-3) / 1e12, 1),
                                      "note": "the whole block on one GPU (every rank runs it; max over ranks)"}
    ref_slice = out_all[t0:t1].clone()
    del single, sc1
    fusedep = par.EPMoEFused(hal, gu, dn, e, h, it, k, hq4, rank, world, max_tokens=t1 - t0 + 1)
    o_f = torch.empty((t1 - t0, h), device="cuda")
    fusedep.forward(xs, lg, o_f)
    torch.cuda.synchronize()
    entry = check("ep moe (peer stores)", o_f, ref_slice)
    dist.barrier()
    ms = time_region(lambda i: fusedep.forward(xs, lg, o_f), 20, dist, stream, graph=True) / 20
    entry.update({"us": round(ms * 1e3, 1), "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1), "speedup_over_one_gpu": round(ms1 / ms, 2),
                  "strong_scaling_efficiency": round(ms1 / ms / world, 3)})
    out[f"ep{world}_moe_T2048_E256_top8_peer_stores"] = entry
    del fusedep
    torch.cuda.empty_cache()
    ep = par.EPMoE(hal, gu, dn, e, h, it, k, hq4, rank, world)
    o_n = ep.forward(xs, lg)
    entry = check("ep moe (NCCL all-to-all)", o_n, ref_slice)
    dist.barrier()
    ms = tmax(_time_call(lambda: ep.forward(xs, lg), 10, warm=3))
    entry.update({"us": round(ms * 1e3, 1), "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1)})
    out[f"ep{world}_moe_T2048_E256_top8_nccl_all_to_all"] = entry
    assert hal.device_status() == 0
    return out


def cpu_baseline(q, hal, n, k, m):
    """The CPU restatement timed on this box's host cores on a bounded sample, and used as the checker of the
    device result at the timed shape."""
    import numpy as np
    import torch
    from oracle import qw_oracle as qo
    qo.build()
    cores = qo.set_num_threads(host_cores())
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    w = torch.randn((n, k), generator=gen, device="cuda", dtype=torch.float32) * 0.02
    bank = q.QWGemm.quantize(hal, w, q.CONTAINERS["HQ4_G32"])
    view = q.QWWeightView(bank, n, k, q.CONTAINERS["HQ4_G32"])
    x = torch.randn((m, k), generator=gen, device="cuda", dtype=torch.float32).to(torch.float16)
    y = torch.empty((m, n), dtype=torch.float32, device="cuda")
    q.QWGemm.encode(hal, view, x, y)
    blocks = bank.cpu().numpy().reshape(n, k // 32, 20)
    xh = x.cpu().numpy()
    yref = qo.matmul(blocks, qo.HQ4_G32, xh)
    err = float(np.abs(y.cpu().numpy() - yref).max() / np.abs(yref).max())
    qo.matmul(blocks, qo.HQ4_G32, xh)
    reps, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 10.0 and reps < 500:
        qo.matmul(blocks, qo.HQ4_G32, xh)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": gemv_bytes(n, k, m) / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{reps} full GEMV calls of the workload in ~10 s", "ms_per_call": dt * 1e3,
            "device_vs_cpu_max_rel_err": err}


def run_case(args):
    """A small named case of one kernel for profiler captures (few launches, a few hundred MB on the device at most):
         gemv:<container>:<n>:<k>:<m>     the matmul door over four banks in rotation (static-weights mode)
         moe:<experts>:<tokens>            the sparse-MoE chain, hidden 2048, intermediate 512, top-8, HQ4_G32
    Prints one JSON line with the mean time per call (CUDA events; not a bench value)."""
    import torch
    import qwegn_b200 as q
    torch.cuda.set_device(0)
    hal = q.QWHal(0)
    parts = args.case.split(":")
    iters = max(1, min(args.steps, 20))
    stream = torch.cuda.current_stream()
    if parts[0] == "gemv":
        cname, n, k, m = parts[1], int(parts[2]), int(parts[3]), int(parts[4])
        cont = q.CONTAINERS[cname]
        banks = make_banks(q, hal, n, k, cont, 4, seed=3)
        x = torch.randn((m, k), device="cuda").to(torch.float16)
        y = torch.empty((m, n), dtype=torch.float32, device="cuda")
        nws = q.QWGemm.workspaceBytes(hal, banks[0], m)
        ws = torch.empty(nws, dtype=torch.uint8, device="cuda") if nws else None
        torch.cuda.synchronize()
        hal.set_static_weights(True)
        fn = lambda i: q.QWGemm.encode(hal, banks[i % 4], x, y, workspace=ws)
    elif parts[0] == "moe":
        e, t = int(parts[1]), int(parts[2])
        k, h, inter = 8, 2048, 512
        cont = q.CONTAINERS["HQ4_G32"]
        gu = q.QWGemm.quantize(hal, torch.randn((e * 2 * inter, h), device="cuda") * 0.02, cont)
        dn = q.QWGemm.quantize(hal, torch.randn((e * h, inter), device="cuda") * 0.02, cont)
        op = q.QWMoEOperator(hal, q.QWWeightView(gu, e * 2 * inter, h, cont), q.QWWeightView(dn, e * h, inter, cont), e, inter, k)
        x = torch.randn((t, h), device="cuda").to(torch.float16)
        lg = torch.randn((t, e), device="cuda")
        outp = torch.empty((t, h), device="cuda")
        sc = torch.empty(op.scratchBytes(t), dtype=torch.uint8, device="cuda")
        if t <= 8:
            hal.set_static_weights(True)
        fn = lambda i: op.encodeResident(x, lg, outp, sc)
    else:
        raise SystemExit(f"unknown case {args.case}")
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(iters):
        fn(i)
    e1.record(stream)
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "calls": iters, "us_per_call": e0.elapsed_time(e1) / iters * 1e3,
                      "device_status": hal.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sections", default="", help="comma list of extra sections: sweep,c1,cpu,prefill,moe (N=1), parallel (N>1)")
    ap.add_argument("--case", default="", help="run one small named case instead of the bench (profiler captures): see run_case")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
