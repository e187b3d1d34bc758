#!/usr/bin/env python3
"""Headline benchmark: HQ4_G32 dequant-GEMV effective HBM bandwidth (M = 1) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--sections LIST]

One step = one decode GEMV y[1, N] = x[1, K] . W^T over one packed HQ4_G32 weight bank (N = 17408, K = 5120,
the M = 1 point of the speculative-verify sweep).  The timed loop rotates through enough distinct weight banks
to exceed the 126 MB L2, so every step streams its weights from HBM.  Synthetic data: W ~ N(0, 0.02) (seeded)
quantized on the device by the library's own packer; x ~ N(0, 1) f16.

`--impl reference` times the CPU restatement of the reference's path (oracle/) on the host cores for the same
metric.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = {"name": "verify-sweep M=1 point: HQ4_G32 GEMV N=17408 K=5120", "n": 17408, "k": 5120, "m": 1}
METRIC = "HQ4_G32 dequant-GEMV effective HBM bandwidth (M=1)"
UNIT = "GB/s"
L2_BYTES = 126 * 1024 * 1024


def gemv_bytes(n, k, m, block_bytes=20, group=32, out_bytes=4):
    """Algorithmic bytes of one call: packed weights + activations + outputs."""
    return n * (k // group) * block_bytes + m * k * 2 + m * n * out_bytes


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


# ---------------------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference's CPU path for this metric (fused dequant-GEMV restatement, all host threads)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import qw_oracle as qo
    qo.build()
    n, k, m = WORKLOAD["n"], WORKLOAD["k"], WORKLOAD["m"]
    rng = np.random.default_rng(1)
    w = rng.normal(0.0, 0.02, (n, k)).astype(np.float32)
    blocks = qo.quantize(w, qo.HQ4_G32)
    x = rng.standard_normal((m, k)).astype(np.float16)
    nbytes = gemv_bytes(n, k, m)
    for _ in range(max(args.warmup, 1)):
        qo.matmul(blocks, qo.HQ4_G32, x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        qo.matmul(blocks, qo.HQ4_G32, x)
    dt = time.perf_counter() - t0
    val = nbytes * args.steps / dt / 1e9
    cores = qo.num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 weights x f16 activations, f64 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "n": n, "k": k, "m": m, "format": "HQ4_G32"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full GEMV calls of the workload (the reference ships no fused CPU kernel; "
                                   "this is the C restatement of its decode + group dot, OpenMP over rows)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------
GRAPH_STEPS = 500   # calls per captured graph; a timed region of K steps replays it K // 500 times (+ one graph of K % 500)


def time_region(fn, steps, dist, stream, graph=False):
    """Barrier + synchronize on both sides, CUDA events on the launching stream, max over ranks (ms).

    graph=True captures the calls in CUDA graphs (the way a decode loop submits its kernels) and replays them inside
    the timed region, so the host's per-call cost (ctypes + launch, ~15 us from Python) is not what is measured.
    Exactly `steps` calls run between the events; one untimed replay of each graph precedes the timed region."""
    import torch
    plan = []   # (graph, replays)
    if graph:
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

    # ---- headline: device-resident GEMV, weights rotating through > L2 of distinct banks -------------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    cont = q.CONTAINERS["HQ4_G32"]
    per_bank = n * cont.row_bytes(k)
    copies = max(2, -(-3 * L2_BYTES // per_bank))
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
    ms = time_region(step, args.steps, dist, stream, graph=True)
    nbytes = gemv_bytes(n, k, m)
    ms_per_step = ms / args.steps
    value = world * nbytes / (ms_per_step * 1e-3) / 1e9

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
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 (f16 weights decoded from u4, f16 activations, f32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "n": n, "k": k, "m": m, "format": "HQ4_G32",
                   "l2": f"rotation over {copies} distinct weight banks ({copies * per_bank / 1e6:.0f} MB > 126 MB L2)",
                   "launch": "the K calls are captured in CUDA graphs of <= 500 calls and replayed inside the timed region; static-weights mode: programmatic dependent launch between calls (weights prefetch under the previous kernel's tail)",
                   "parallelism": "one replica of the projection per GPU (column-parallel shards, no collective)" if world > 1 else "1 GPU"},
        "clocks": clocks,
        "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel() * 2),
                "d2h_bytes_per_step": int(y_host.numel() * 4), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": nbytes / (ms_per_step * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": nbytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": peaks["source"], "kernel": "qwc_gemv_stream_kernel<HQ4_G32_M5, M<=8>",
                     "algorithmic_bytes_per_launch": nbytes},
        "device_status": status,
    }
    # DRAM traffic per launch of this kernel on this workload, from the committed ncu summary (read + write bytes)
    traffic_file = os.path.join(ROOT, "profiles", "qwc_gemv_stream_kernel_hq4g32_n17408_k5120_m1.md")
    if os.path.exists(traffic_file):
        import re
        mt = re.search(r"dram_bytes_per_launch:\s*(\d+)", open(traffic_file).read())
        if mt:
            line["roofline"]["traffic"] = int(mt.group(1))

    hal.set_static_weights(False)   # the sections below build fresh banks on the same stream
    extra = {}
    if rank == 0 and world == 1:
        del banks
        torch.cuda.empty_cache()
        if "c1" in sections:
            t, b, *_ = bench_gemv_point(q, hal, 12288, 4096, 1, "HQ4_G32", args.steps, args.warmup)
            extra["c1_gemv_N12288_K4096"] = {"GBps": b / (t * 1e-3) / 1e9, "us": t * 1e3, "frac_of_peak": b / (t * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        if "c1" in sections:
            t, b, *_ = bench_gemv_point(q, hal, n, k, 1, "HQ4_G32", args.steps, args.warmup, rotated=True)
            extra["c2_gemv_M1_rotated_activations_in"] = {"GBps": b / (t * 1e-3) / 1e9, "us": t * 1e3,
                                                          "note": "x_is_rotated=1: activations rotated by qwc_rmsnorm_fwht outside the timed loop, as in the reference's engine"}
        if "c1" in sections:
            extra["lm_head_greedy_N248320_K5120_M1"] = bench_lm_head(q, hal, peaks)
            torch.cuda.empty_cache()
        if "c1" in sections:
            extra["f32_activation_door_N17408_K5120"] = bench_f32_door(q, hal, n, k, args.warmup)
            torch.cuda.empty_cache()
        if "sweep" in sections:
            sweep = {}
            for cname in ("HQ4_G32", "HQ8_G32", "HQ4_G64"):
                for mm in (1, 2, 4, 8, 16):
                    t, b, *_ = bench_gemv_point(q, hal, n, k, mm, cname, max(20, args.steps // 4), args.warmup)
                    sweep[f"{cname}_M{mm}"] = {"GBps": round(b / (t * 1e-3) / 1e9, 1), "us": round(t * 1e3, 2)}
                    torch.cuda.empty_cache()
            extra["verify_sweep_N17408_K5120"] = sweep
        if "prefill" in sections:
            extra["prefill_M4096"] = bench_prefill(q, hal, peaks)
        if "moe" in sections:
            extra["moe_T2048_E256_top8"] = bench_moe(q, hal)
        if "cpu" in sections:
            line["cpu_baseline"] = cpu_baseline(q, hal, n, k, m)
    if world > 1 and "parallel" in sections:
        par = bench_parallel(q, hal, rank, world, dist)
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

    for i in range(4):
        step(i)
    ms = time_region(step, steps, None, stream, graph=True) / steps
    nbytes = gemv_bytes(n, k, 1)
    ref = int(torch.argmax(y[0]).item())
    return {"us": ms * 1e3, "GBps": nbytes / (ms * 1e-3) / 1e9, "frac_of_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "token_matches_torch_argmax": bool(int(tok.item()) == ref)}


def bench_f32_door(q, hal, n, k, warmup, steps=400):
    """The f32-activation door (rotated f32 rows in, f32 out) at the headline shape: stage kernel + GEMV (+ epilogue
    kernel for the silu + FWHT epilogue).  Banks in rotation, larger than L2 together."""
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
    QKV width 7168; HQ4_G32; rotated f16 activations resident; f16 out.  TFLOP/s = 2 M N K / time."""
    import torch
    out = {}
    m = 4096
    cont = q.CONTAINERS["HQ4_G32"]
    for name, (n, k) in {"gate_up_N34816_K5120": (34816, 5120), "down_N5120_K17408": (5120, 17408), "qkv_N7168_K5120": (7168, 5120)}.items():
        w = torch.randn((n, k), device="cuda", dtype=torch.float32) * 0.02
        view = q.QWWeightView(q.QWGemm.quantize(hal, w, cont), n, k, cont)
        del w
        x = torch.randn((m, k), device="cuda", dtype=torch.float32).to(torch.float16)
        q.QWGemm.encodeFwht32(hal, x)
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        ms = _time_call(lambda: q.QWGemm.encode(hal, view, x, y, x_is_rotated=True), 10)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out[name] = {"ms": round(ms, 4), "TFLOPs": round(tf, 1), "frac_of_burst_peak": round(tf / peaks["bf16_tflops"], 3),
                     "frac_of_sustained_peak": round(tf / peaks["bf16_tflops_sustained"], 3)}
        del view, x, y
        torch.cuda.empty_cache()
    return out


def bench_moe(q, hal):
    """The 35B-A3B-shaped sparse MoE block: 2048 tokens, 256 experts, top-8, hidden 2048, expert intermediate 512,
    HQ4_G32; router logits N(0, 1); the whole operator chain (route .. combine) per step."""
    import torch
    t, e, k, h, inter = 2048, 256, 8, 2048, 512
    cont = q.CONTAINERS["HQ4_G32"]
    gu = q.QWGemm.quantize(hal, torch.randn((e * 2 * inter, h), device="cuda") * 0.02, cont)
    dn = q.QWGemm.quantize(hal, torch.randn((e * h, inter), device="cuda") * 0.02, cont)
    op = q.QWMoEOperator(hal, q.QWWeightView(gu, e * 2 * inter, h, cont), q.QWWeightView(dn, e * h, inter, cont), e, inter, k)
    x = torch.randn((t, h), device="cuda").to(torch.float16)
    lg = torch.randn((t, e), device="cuda")
    outp = torch.empty((t, h), device="cuda")
    sc = torch.empty(op.scratchBytes(t), dtype=torch.uint8, device="cuda")
    ms = _time_call(lambda: op.encodeResident(x, lg, outp, sc), 20)
    flops = 2.0 * t * k * (2 * inter * h + h * inter)
    wbytes = e * (2 * inter * (h // 32) * 20 + h * (inter // 32) * 20)
    # the decode / verify size of the same block (8 tokens = 64 pairs, up to 64 experts touched): served by the grouped path
    # timed the way a decode loop runs it: CUDA-graph replay, weights declared static, router logits that change from
    # step to step (16 sets) so that the experts touched, and with them the weights read, differ between steps
    x8, out8 = x[:8].contiguous(), torch.empty((8, h), device="cuda")
    lg8 = [torch.randn((8, e), device="cuda") for _ in range(16)]
    torch.cuda.synchronize()
    hal.set_static_weights(True)
    for i in range(3):
        op.encodeResident(x8, lg8[i], out8, sc)
    ms8 = time_region(lambda i: op.encodeResident(x8, lg8[i % 16], out8, sc), 320, None, torch.cuda.current_stream(), graph=True) / 320
    torch.cuda.synchronize()
    hal.set_static_weights(False)
    return {"us": round(ms * 1e3, 1), "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1), "weight_GBps": round(wbytes / (ms * 1e-3) / 1e9, 1),
            "decode_T8_us": round(ms8 * 1e3, 1),
            "bound": "about 100 cycles per tcgen05.mma instruction whatever its N: 64-token expert tiles use a third of the tensor rate; neither the HBM roof (~80 us) nor the tensor roof binds yet"}


def bench_parallel(q, hal, rank, world, dist):
    """Tensor-parallel MLP of a 70B-class layer (hidden 8192, intermediate 28672, HQ4_G32; column-parallel gate||up with
    fused SwiGLU+FWHT, row-parallel down, one NCCL all-reduce) at M = 1, and the expert-parallel MoE block (2048
    tokens sharded over the ranks, 256 experts sharded over the ranks, NCCL all-to-all).  Max over ranks."""
    import torch
    from qwegn_b200 import parallel as par
    cont = q.CONTAINERS["HQ4_G32"]
    out = {}

    def tmax(ms):
        tt = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    hidden, inter = 8192, 28672
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)   # the same bank on every rank; each keeps its shard
    gu_plane = q.QWGemm.quantize(hal, torch.randn((2 * inter, hidden), generator=gen, device="cuda") * 0.02, cont)
    dn_plane = q.QWGemm.quantize(hal, torch.randn((hidden, inter), generator=gen, device="cuda") * 0.02, cont)
    x = torch.randn((1, hidden), generator=gen, device="cuda").to(torch.float16)
    y = torch.empty((1, hidden), dtype=torch.float32, device="cuda")
    wbytes = (2 * inter * (hidden // 32) + hidden * (inter // 32)) * 20
    # the all-reduce by NCCL after the down projection, and fused into the down projection's kernel (peer stores + flags)
    for label, fused in (("nccl_allreduce", False), ("fused_allreduce", True)):
        try:
            mlp = par.TPMlp(hal, gu_plane, dn_plane, hidden, inter, cont, rank, world, fused_allreduce=fused)
        except Exception as exc:   # symmetric memory unavailable on this box: report, keep the NCCL number
            out[f"tp{world}_mlp_decode_M1_H8192_I28672_{label}"] = {"unavailable": str(exc)[:120]}
            continue
        h_loc = torch.empty((1, mlp.inter_local), dtype=torch.float16, device="cuda")
        dist.barrier()
        ms = tmax(_time_call(lambda: mlp.forward(x, h_loc, y), 50, warm=5))
        entry = {"us": round(ms * 1e3, 1), "aggregate_weight_GBps": round(wbytes / (ms * 1e-3) / 1e9, 1)}
        try:   # the same step submitted as a CUDA graph of 20 MLPs (no Python between the kernels)
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            torch.cuda.synchronize()
            dist.barrier()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for _ in range(20):
                        mlp.forward(x, h_loc, y)
            torch.cuda.synchronize()
            dist.barrier()
            msg = tmax(_time_call(g.replay, 5, warm=2)) / 20
            entry["graph_us"] = round(msg * 1e3, 1)
            entry["graph_aggregate_weight_GBps"] = round(wbytes / (msg * 1e-3) / 1e9, 1)
            del g
        except Exception as exc:
            entry["graph_unavailable"] = str(exc)[:100]
        out[f"tp{world}_mlp_decode_M1_H8192_I28672_{label}"] = entry
        del mlp
        torch.cuda.empty_cache()
    del gu_plane, dn_plane
    torch.cuda.empty_cache()

    t, e, k, h, it = 2048, 256, 8, 2048, 512
    gu = q.QWGemm.quantize(hal, torch.randn((e * 2 * it, h), generator=gen, device="cuda") * 0.02, cont)
    dn = q.QWGemm.quantize(hal, torch.randn((e * h, it), generator=gen, device="cuda") * 0.02, cont)
    ep = par.EPMoE(hal, gu, dn, e, h, it, k, cont, rank, world)
    del gu, dn
    torch.cuda.empty_cache()
    t0, t1 = t * rank // world, t * (rank + 1) // world
    xs = torch.randn((t, h), generator=gen, device="cuda").to(torch.float16)[t0:t1].contiguous()
    lg = torch.randn((t, e), generator=gen, device="cuda")[t0:t1].contiguous()
    dist.barrier()
    ms = tmax(_time_call(lambda: ep.forward(xs, lg), 10, warm=3))
    flops = 2.0 * t * k * (2 * it * h + h * it)
    out[f"ep{world}_moe_T2048_E256_top8"] = {"us": round(ms * 1e3, 1), "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1)}
    return out


def cpu_baseline(q, hal, n, k, m):
    """The CPU restatement timed on this box's host cores on a bounded sample, and used as the checker of the
    device result at the timed shape."""
    import numpy as np
    import torch
    from oracle import qw_oracle as qo
    qo.build()
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
    return {"value": gemv_bytes(n, k, m) / dt / 1e9, "unit": UNIT, "cores": qo.num_threads(), "kind": "port",
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
    ap.add_argument("--sections", default="", help="comma list of extra sections at N=1: sweep,c1,cpu")
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
