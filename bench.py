#!/usr/bin/env python
"""Benchmark of the gated-GQA attention path.

    python bench.py --gpus N --steps K --warmup W [--workload decode_b8|decode_b1|decode_b64|decode_int8_b8|pp512|chunked_b1|...] [--extras all|none|a,b,...]
    python bench.py --impl reference ...      # the reference's scalar CPU math (oracle port) on the host cores

Default workload (the one the headline metric is quoted on): decode at 32K context across all 16 attention layers, fp16
KV cache, 8 independent sequences per GPU with context lengths uniform in [16K, 32K], one new token per step. A step is
one pass of the hot path over the batch: per layer, append the token's K/V row (norm, RoPE, fp16 store) and attend over
the whole cached context (split-KV decode with the merge and the output gate fused). With N GPUs each rank holds its own
8 sequences (batch sharding, no data-path collective): weak scaling; N=8 is the 64-sequence configuration.

Timing: CUDA events on the launching stream around exactly K steps after W warm-up steps, barrier and synchronize on both
sides, max over ranks. The KV working set per step (GBs) is far larger than L2, so no explicit flush is needed.

The printed line is that of the default workload. Its "extras" object carries the other configurations of the benchmark
statement, each measured in the same process right after it with fewer steps (pp512, decode at batch 1 and 64, int8 KV at
8K and 32K, chunked prefill at batch 1 and 16; with several ranks: one sequence split by keys across the ranks), each with
value, ms_per_step, clocks, e2e, roofline and a cpu_baseline of its own; "sustained" repeats the default step for two
seconds and gives the rate with the clock the GPU settles at.
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

import numpy as np

N_LAYERS = 16
NCU_TRAFFIC_RATIO = 1.028   # (dram__bytes_read + dram__bytes_write) / algorithmic bytes of decode_mma_kernel, profiles/decode_mma_kernel__decode_small.md
WORKLOADS = {
    # name: (kind, batch per GPU, kv mode, max length, min length)
    "decode_b8": ("decode", 8, "fp16", 32768, 16384),
    "decode_b1": ("decode", 1, "fp16", 32768, 32768),
    "decode_small": ("decode", 4, "fp16", 8192, 8192),        # ~2 GB of cache: the size used for ncu captures
    "decode_int8_small": ("decode", 4, "int8", 16384, 16384),
    "decode_int8v_small": ("decode", 4, "int8v", 8192, 8192),
    "decode_b64": ("decode", 64, "fp16", 32768, 16384),
    "decode_int8_b8": ("decode", 8, "int8", 32768, 16384),
    "decode_int8_b32": ("decode", 32, "int8", 32768, 16384),
    "decode_int8_8k_b1": ("decode", 1, "int8", 8192, 8192),      # benchmark config 4 at its short context
    "decode_int8_8k_b32": ("decode", 32, "int8", 8192, 8192),
    "decode_int8g_b8": ("decode", 8, "int8g", 32768, 16384),    # int8 keys with one scale per 64 dims (four per head row), int8 values
    "decode_int8v_b8": ("decode", 8, "int8v", 32768, 16384),    # keys fp16, values int8 (the reference's KATA_KV=int8v)
    "splitkv_b1": ("splitkv", 1, "fp16", 32768, 32768),       # one 32K sequence, keys split across the ranks, parts pushed to the peers and merged per layer
    "splitkv_b1_128k": ("splitkv", 1, "fp16", 131072, 131072),  # the same at 131,072 keys, where one GPU's HBM time dominates the exchange
    "pp512": ("prefill", 1, "fp16", 512, 512),
    # chunked: (kind, batch, kv mode, prompt length, restored prefix)
    "chunked_b1": ("chunked", 1, "fp16", 7300, 3600),
    "chunked_b16": ("chunked", 16, "fp16", 7300, 3600),
    "chunked_int8_b4": ("chunked", 4, "int8", 7300, 3600),    # the codes are expanded to fp16 per layer for the tcgen05 kernel
    "chunked_int8v_b4": ("chunked", 4, "int8v", 7300, 3600),
    "chunked_small": ("chunked", 4, "fp16", 3072, 1024),      # ~0.4 GB: the size used for ncu captures of the prefill kernel
    "draft_attn": ("draft", 8, "fp16", 2048, 4096),           # the block drafter's attention: 5 layers, block of 8 rows, window 2048 over a 4096 ring, 4 drafters in rotation (168 MB of rings read per step)
    "out_fwht": ("fwht", 32768, "fp32", 6144, 6144),          # the sign + Walsh-Hadamard transform that follows attention, on 32,768 output rows (805 MB in, 805 MB out)
}


EXTRAS_ONE_GPU = ["pp512", "decode_b1", "decode_b64", "decode_int8_b8", "decode_int8_b32", "decode_int8_8k_b1", "decode_int8_8k_b32", "decode_int8v_b8", "decode_int8g_b8", "chunked_b1", "chunked_b16"]
EXTRAS_MULTI_GPU = ["splitkv_b1", "splitkv_b1_128k"]      # strong scaling: one sequence, keys split across the ranks
EXTRAS_BUDGET_S = 400.0                                    # extras not started after this many seconds of the run are skipped (and say so)
METRIC = "gated-GQA attn tok/s (decode@32K, pp512); HBM GB/s & TC util vs peak"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons through NVML (read-only) on a background thread while
    the GPU is under load; falls back to polling nvidia-smi when the NVML binding is unavailable."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.samples, self.stop_flag, self.thread, self.max_mhz = index, [], False, None, None

    def _loop_nvml(self, nv, h):
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((time.perf_counter(), float(mhz), int(bits)))
            except Exception:
                break
            time.sleep(0.004)

    def _loop_smi(self):
        q = "clocks.sm,clocks.max.sm,clocks_throttle_reasons.active"
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                c = [x.strip() for x in out.strip().split(",")]
                self.max_mhz = float(c[1])
                self.samples.append((time.perf_counter(), float(c[0]), int(c[2], 16)))
            except Exception:
                break

    def start(self):
        try:
            import pynvml as nv
            import torch
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                h = nv.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._loop_nvml, args=(nv, h), daemon=True)
        except Exception:
            self.thread = threading.Thread(target=self._loop_smi, daemon=True)
        self.thread.start()

    def stop(self, t0=None, t1=None):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=6)
        inside = [x for x in self.samples if t0 is not None and t0 <= x[0] <= t1]
        use, window = (inside, "timed region") if len(inside) >= 2 else (self.samples, "warm-up + timed region (timed region shorter than the sampling period)")
        bits = 0
        for x in use:
            bits |= x[2]
        return {"sm_mhz": float(np.median([x[1] for x in use])) if use else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(v for k, v in self.REASONS.items() if bits & k), "samples": len(use), "window": window}


# ------------------------------------------------------------------------------------------------- the CUDA arm
def decode_workload_name(kv_mode, lmax, lmin, B):
    return f"decode, {N_LAYERS} layers, {kv_mode} KV, ctx {lmax}, batch {B}/GPU (lengths uniform [{lmin},{lmax}]), 1 new token/step, append+attend per layer"


def run_decode(args, rank, world, kind_cfg, steps=None, warmup=None, sustained_s=0.0, want_cpu=True):
    import torch
    import torch.distributed as dist
    from kata_b200 import capi, synth

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    _, B, kv_mode, lmax, lmin = kind_cfg
    dev = torch.device("cuda", torch.cuda.current_device())
    steps_total = warmup + steps + 2
    # Weak scaling: every rank holds B sequences with the SAME length draw, so the work per GPU is fixed as N grows (the contents differ per rank).
    lens = synth.seq_lengths(1234, B, lmin, lmax).astype(np.int64)
    lens = np.minimum(lens, lmax)
    ctx = capi.AttnContext(N_LAYERS, [int(l) + 2 * steps_total + 8 for l in lens], kv_mode=kv_mode)
    gen = torch.Generator(device=dev); gen.manual_seed(4321 + rank)
    seqs = list(range(B))
    qn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    kn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    # fill the caches through prep (K/V head slots only): contents are normed, rotated fp16 (or int8) rows, as in a real run
    CH = 1024
    for layer in range(N_LAYERS):
        for sq in seqs:
            for start in range(0, int(lens[sq]), CH):
                m = min(CH, int(lens[sq]) - start)
                kp = torch.randn(1, m, 1024, generator=gen, device=dev)
                vp = torch.randn(1, m, 1024, generator=gen, device=dev)
                ctx.prep(layer, [sq], [start], m, None, kp, vp, None, kn[layer], h0=24, nh=8)
    ctx.check()
    qfull = torch.randn(N_LAYERS, B, 1, 12288, generator=gen, device=dev)
    kproj = torch.randn(N_LAYERS, B, 1, 1024, generator=gen, device=dev)
    vproj = torch.randn(N_LAYERS, B, 1, 1024, generator=gen, device=dev)
    q16 = torch.empty(N_LAYERS, B, 1, 6144, dtype=torch.float16, device=dev)
    gate = torch.empty(N_LAYERS, B, 1, 6144, dtype=torch.float32, device=dev)
    out = torch.empty(N_LAYERS, B, 1, 6144, dtype=torch.float32, device=dev)
    pos = lens.copy()

    # per-layer views made once: slicing a tensor costs the host more than a microsecond, and at batch 1 a layer is 36 us of GPU time
    L_ = range(N_LAYERS)
    qfull_l, kproj_l, vproj_l, qn_l, kn_l = [qfull[l] for l in L_], [kproj[l] for l in L_], [vproj[l] for l in L_], [qn[l] for l in L_], [kn[l] for l in L_]
    q16_l, gate_l, out_l = [q16[l] for l in L_], [gate[l] for l in L_], [out[l] for l in L_]

    def step(p):   # the sixteen layers' prep + decode through one call of the C ABI (kata_attn_layers_step: the Engine's layer loop on the native side of the binding)
        ctx.layers_step(N_LAYERS, seqs, p.tolist() if isinstance(p, np.ndarray) else p, 1, qfull, kproj, vproj, qn, kn, q16, gate, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    for _ in range(warmup):
        step(pos); pos = pos + 1
        torch.cuda.current_stream().synchronize()   # as in serving, where every step ends with the host holding its result
    ctx.check()
    l0 = ctx.launches()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw0 = time.perf_counter()
    torch.cuda.profiler.start()   # lets `ncu --profile-from-start off` capture exactly the timed steps; a no-op otherwise
    e0.record()
    pos_timed0 = pos.copy()
    for _ in range(steps):
        step(pos); pos = pos + 1
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    tw1 = time.perf_counter()
    ms = e0.elapsed_time(e1)
    launches = ctx.launches() - l0
    clocks = sampler.stop(tw0, tw1)
    ctx.check()
    assert torch.isfinite(out).all()

    # the same step repeated for sustained_s seconds at a fixed position (the appended row is rewritten in place): where the clock settles
    sustained = None
    if sustained_s > 0:
        pos_s = (pos - 1).tolist()
        s2 = ClockSampler(torch.cuda.current_device()); s2.start()
        barrier()
        n_s, ts0 = 0, time.perf_counter()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        while time.perf_counter() - ts0 < sustained_s:
            for _ in range(16):
                step(pos_s)
            n_s += 16
            torch.cuda.current_stream().synchronize()
        g1.record(); torch.cuda.synchronize(); ts1 = time.perf_counter()
        ms_s = g0.elapsed_time(g1)
        sustained = {"seconds": ms_s * 1e-3, "steps": n_s, "value": B * n_s / (ms_s * 1e-3), "unit": "tok/s (this rank)", "ms_per_step": ms_s / n_s, "clocks": s2.stop(ts0, ts1)}

    # the dominant kernel alone: the decode launches of the same steps, timed on the same stream
    pos_k = pos_timed0.tolist()
    ctx.layers_decode(N_LAYERS, seqs, pos_k, 1, q16, gate, out)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    reps = max(2, steps)
    for _ in range(reps):   # one call of the C ABI per sixteen launches: a layer of the smallest workloads is shorter than a call through the Python binding
        ctx.layers_decode(N_LAYERS, seqs, pos_k, 1, q16, gate, out)
    k1.record(); torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / (reps * N_LAYERS)

    # end to end through the C ABI with HOST (pinned) buffers: kata_attn_host_step_run takes the step's projections of all layers from host memory,
    # appends and attends layer by layer and leaves the output rows in host memory (copies of the neighbouring layers under the layer that computes)
    hq = torch.randn(N_LAYERS, B, 1, 12288).pin_memory(); hk = torch.randn(N_LAYERS, B, 1, 1024).pin_memory(); hv = torch.randn(N_LAYERS, B, 1, 1024).pin_memory()
    hout = torch.empty(N_LAYERS, B, 1, 6144).pin_memory()
    hstep = capi.HostStep(ctx, max_n=B, max_T=1)

    def step_e2e(p):
        hstep.run(N_LAYERS, seqs, p.tolist() if isinstance(p, np.ndarray) else p, 1, hq, hk, hv, qn, kn, hout)
        torch.cuda.current_stream().synchronize()   # the caller holds the step's result on the host before the next step

    pos_e = pos_timed0.copy()
    step_e2e(pos_e)
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step_e2e(pos_e); pos_e = pos_e + 1
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    h2d = N_LAYERS * B * (12288 + 2048) * 4
    d2h = N_LAYERS * B * 6144 * 4

    row_bytes = {"fp16": 4096, "int8": 2064, "int8v": 3080, "int8g": 2088}[kv_mode]   # K+V bytes per key per layer (int8: codes + both fp16 scales; int8v: fp16 keys, value codes + their scales)
    bytes_per_launch = float(np.sum(pos_timed0 + 1)) * row_bytes
    per_rank = None
    if world > 1:
        mine = torch.tensor([ms / steps, e2e_ms / steps, kern_ms * 1e3, float(np.sum(pos_timed0 + 1))], device=dev, dtype=torch.float64)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        allr = torch.stack(allr).cpu().numpy()
        per_rank = {"ms_per_step": [round(float(x), 4) for x in allr[:, 0]], "e2e_ms_per_step": [round(float(x), 4) for x in allr[:, 1]],
                    "decode_us_per_launch": [round(float(x), 2) for x in allr[:, 2]], "keys_per_launch": [int(x) for x in allr[:, 3]],
                    "kv_gb_per_s_sum_over_ranks": float(np.sum(allr[:, 3] * row_bytes * N_LAYERS / (allr[:, 0] * 1e-3)) / 1e9)}
        ms, e2e_ms = float(allr[:, 0].max()) * steps, float(allr[:, 1].max()) * steps
    mean_len = float(np.mean([pos_timed0 + i + 1 for i in range(steps)]))   # keys attended per sequence per step (the new key included)
    pk = peaks()
    ach = bytes_per_launch / (kern_ms * 1e-3) / 1e9
    res = {
        "metric": METRIC, "value": world * B * steps / (ms * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16" if kv_mode == "fp16" else "int8", "data": "synthetic",
        "config": {"workload": decode_workload_name(kv_mode, lmax, lmin, B),
                   "batch_per_gpu": B, "global_batch": world * B, "mean_context": mean_len, "parallelism": f"batch-sharded x{world}",
                   "lengths": "the same length draw on every rank (per-GPU work fixed as N grows); cache contents differ per rank",
                   "l2": "inputs larger than L2 (no flush needed)" if bytes_per_launch * N_LAYERS > 2.5e8 else "all 16 layers' caches together are not much larger than L2: part of the reads may be L2 hits"},
        "clocks": clocks, "gpu_launches": int(launches),
        "e2e": {"value": world * B * steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "roofline": {"bound": "hbm", "kernel": "decode_mma_kernel" + (" (+ decode_combine_kernel: segments cut between more than 8 CTAs)" if B == 1 and lmax > 8192 else ""), "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "peak_src": pk["src"],
                     "frac_of_nominal_8TBs": ach / 8000.0, "us_per_launch": kern_ms * 1e3, "algorithmic_bytes_per_launch": bytes_per_launch,
                     "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO if kv_mode == "fp16" else None,
                     "traffic_note": "not measured in this run: algorithmic bytes x 1.028, a constant taken from the ncu capture of the decode_small workload (138.1 MB of dram read+write for 134.3 MB algorithmic, profiles/decode_mma_kernel__decode_small.md)"},
    }
    if per_rank:
        res["config"]["per_rank"] = per_rank
    if sustained:
        res["sustained"] = sustained
    if rank == 0 and want_cpu and not args.no_cpu_baseline:
        res["cpu_baseline"] = cpu_baseline_decode(ctx, pos_timed0, B, kv_mode, reps=4 if sustained_s > 0 else 1)   # the headline line: some 20 core-seconds of host work
    hstep.close(); ctx.close()
    del qfull, kproj, vproj, q16, gate, out
    torch.cuda.empty_cache()
    return res


def cpu_baseline_decode(ctx, pos, B, kv_mode, reps=1):
    """The oracle on the host cores, on a bounded sample: layer 0 of the same caches (copied back from the GPU) for up to 8 sequences at
    full length; tok/s extrapolated to 16 layers. fp16 cache: the reference's scalar decode (k_attn_decode restated). int8 caches: the
    oracle's fp32 evaluation of the formula on the dequantised planes (the reference has no scalar decode over int8 planes)."""
    from oracle import kata_oracle as orc
    nb = min(B, 8 if kv_mode == "fp16" else 4)
    rng = np.random.default_rng(1)
    q = rng.standard_normal((nb, 6144)).astype(np.float32); g = rng.standard_normal((nb, 6144)).astype(np.float32)
    cores = orc.hw_threads()
    if kv_mode == "fp16":
        ks = [ctx.plane_read(0, s, 0, 0, int(pos[s]) + 1).view(np.uint16) for s in range(nb)]
        vs = [ctx.plane_read(0, s, 1, 0, int(pos[s]) + 1).view(np.uint16) for s in range(nb)]
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.decode_batch(q, g, ks, vs, [int(p) for p in pos[:nb]], threads=cores)
        dt = (time.perf_counter() - t0) / reps
        what = "k_attn_decode restated"
    else:
        planes = []
        for s in range(nb):
            n = int(pos[s]) + 1
            pl = orc.KvPlanes(n, int8=(kv_mode == "int8"), int8v=(kv_mode == "int8v"), int8g=(kv_mode == "int8g"))
            pl.k[:] = ctx.plane_read(0, s, 0, 0, n).view(pl.k.dtype).reshape(n, 1024); pl.v[:] = ctx.plane_read(0, s, 1, 0, n).view(np.int8).reshape(n, 1024)
            if kv_mode in ("int8", "int8g"):
                pl.ksc[:] = ctx.plane_read(0, s, 2, 0, n).view(np.uint16).reshape(n, -1)
            pl.vsc[:] = ctx.plane_read(0, s, ctx.kv_planes() - 1, 0, n).view(np.uint16).reshape(n, 4)
            planes.append(pl)
        t0 = time.perf_counter()
        for _ in range(reps):
            for s in range(nb):
                orc.formula_f32(q[s:s + 1], g[s:s + 1], planes[s], int(pos[s]), threads=cores)
        dt = (time.perf_counter() - t0) / reps
        what = "fp32 formula over the dequantised planes"
    return {"value": nb / (dt * N_LAYERS), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{what}: 1 of {N_LAYERS} layers, {nb} sequences at full length, {reps} time(s) ({dt * reps:.2f} s on {cores} threads), tok/s extrapolated x{N_LAYERS} layers"}


def run_splitkv(args, rank, world, kind_cfg, steps=None, warmup=None):
    """Batch 1, context split by keys across the ranks: every rank holds keys [lo, hi) of all 16 layers and computes its (O, m, l) part per
    layer; the ranks push their parts into each other's exchange buffers over NVLink and merge in the same kernel (kata_attn_peer_*). The
    NCCL all-gather + merge per layer, and one batched all-gather for the 16 layers, are timed beside it. Strong scaling: total work fixed."""
    import torch
    import torch.distributed as dist
    from kata_b200 import capi, multi

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    _, _, kv_mode, L, _ = kind_cfg
    dev = torch.device("cuda", torch.cuda.current_device())
    steps_total = 3 * (warmup + steps) + 2   # three timed runs (peer exchange, NCCL per layer, one batched all-gather) at successive positions
    lo, hi = multi.split_keys(L, world)[rank]
    tail = rank == world - 1
    ctx = capi.AttnContext(N_LAYERS, [max(hi - lo, 1) + steps_total + 8], kv_mode=kv_mode)
    ctx.set_position_offset(0, lo)
    gen = torch.Generator(device=dev); gen.manual_seed(777)   # same projections on every rank
    qn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    kn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    qfull = torch.randn(N_LAYERS, 1, 1, 12288, generator=gen, device=dev)
    kproj = torch.randn(N_LAYERS, 1, 1, 1024, generator=gen, device=dev)
    vproj = torch.randn(N_LAYERS, 1, 1, 1024, generator=gen, device=dev)
    g2 = torch.Generator(device=dev); g2.manual_seed(1000 + rank)
    for layer in range(N_LAYERS):
        for st in range(lo, hi, 1024):
            m = min(1024, hi - st)
            ctx.prep(layer, [0], [st], m, None, torch.randn(1, m, 1024, generator=g2, device=dev), torch.randn(1, m, 1024, generator=g2, device=dev), None, kn[layer], h0=24, nh=8)
    ctx.check()
    q16 = torch.empty(N_LAYERS, 1, 1, 6144, dtype=torch.float16, device=dev); gate = torch.empty(N_LAYERS, 1, 1, 6144, device=dev)
    part = torch.empty(N_LAYERS, 24, 258, device=dev); parts = torch.empty(N_LAYERS, world, 24, 258, device=dev); out = torch.empty(N_LAYERS, 1, 6144, device=dev)
    big = 1 << 30
    px = capi.PeerExchange(rank, world)

    def step(pos, batched):
        if batched == "peer":   # the sixteen layers through one call of the C ABI (kata_attn_peer_layers_step)
            px.layers_step(ctx, N_LAYERS, 0, pos, 1, lo, big if tail else hi, tail, qfull, kproj, vproj, qn, kn, q16, gate, out)
            return
        for layer in range(N_LAYERS):
            ctx.prep(layer, [0], [pos], 1, qfull[layer], kproj[layer], vproj[layer], qn[layer], kn[layer], h0=0, nh=32 if tail else 24, q16=q16[layer], gate=gate[layer])
            if batched == "peer":
                px.decode(ctx, layer, 0, pos, 1, lo, big if tail else hi, q16[layer], gate[layer, 0], out=out[layer])
                continue
            ctx.decode_partial(layer, 0, pos, 1, lo, big if tail else hi, q16[layer], part=part[layer])
            if not batched:
                if world > 1:
                    dist.all_gather_into_tensor(parts[layer], part[layer])
                else:
                    parts[layer, 0].copy_(part[layer])
                ctx.merge_parts(parts[layer], 1, gate[layer, 0], out=out[layer])
        if batched is True:   # legal only because the 16 layers of this synthetic harness are independent
            if world > 1:
                gathered = torch.empty(world, N_LAYERS, 24, 258, device=dev); dist.all_gather_into_tensor(gathered, part)
                parts.copy_(gathered.transpose(0, 1))
            else:
                parts[:, 0].copy_(part)
            for layer in range(N_LAYERS):
                ctx.merge_parts(parts[layer], 1, gate[layer, 0], out=out[layer])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(batched, pos):
        for i in range(warmup):
            step(pos, batched); pos += 1
        ctx.check(); barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter(); e0.record()
        for i in range(steps):
            step(pos, batched); pos += 1
        e1.record(); barrier(); t1 = time.perf_counter()
        return e0.elapsed_time(e1), t0, t1

    # the same sequence whole on one GPU, in the same harness (every rank on its own GPU, no communication; rank 0's figure is reported)
    one = capi.AttnContext(N_LAYERS, [L + warmup + steps + 8], kv_mode=kv_mode)
    g3 = torch.Generator(device=dev); g3.manual_seed(2000 + rank)
    for layer in range(N_LAYERS):
        for st in range(0, L, 1024):
            m = min(1024, L - st)
            one.prep(layer, [0], [st], m, None, torch.randn(1, m, 1024, generator=g3, device=dev), torch.randn(1, m, 1024, generator=g3, device=dev), None, kn[layer], h0=24, nh=8)
    out1 = torch.empty(N_LAYERS, 1, 1, 6144, device=dev)

    def step_one(pos):
        one.layers_step(N_LAYERS, [0], [pos], 1, qfull, kproj, vproj, qn, kn, q16, gate, out1)
    for i in range(warmup):
        step_one(L + i)
    one.check(); barrier()
    o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    o0.record()
    for i in range(steps):
        step_one(L + warmup + i)
    o1.record(); torch.cuda.synchronize()
    ms_one = o0.elapsed_time(o1)
    one.close(); del out1
    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    l0 = ctx.launches()
    ms, tw0, tw1 = timed("peer", L)
    launches = (ctx.launches() - l0) * steps // (steps + warmup) + N_LAYERS * steps
    clocks = sampler.stop(tw0, tw1)
    px.check(); ref_out = out.clone()
    ms_n, _, _ = timed(False, L + warmup + steps)
    ms_b, _, _ = timed(True, L + 2 * (warmup + steps))
    ctx.check(); assert torch.isfinite(out).all() and torch.isfinite(ref_out).all()
    if world > 1:
        t = torch.tensor([ms, ms_n, ms_b], device=dev, dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms, ms_n, ms_b = t.tolist()
    pk = peaks(); bytes_step = N_LAYERS * (L + 1) * 4096.0
    ach = bytes_step / (ms / steps * 1e-3) / 1e9
    res = {"metric": METRIC, "value": steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": steps,
           "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
           "config": {"workload": f"decode, {N_LAYERS} layers, fp16 KV, ctx {L}, batch 1, keys split over {world} rank(s), parts pushed into the peers' buffers and merged in one kernel per layer", "global_batch": 1,
                      "parallelism": f"split-KV x{world}", "tok_s_one_gpu_same_harness": steps / (ms_one * 1e-3), "tok_s_with_nccl_all_gather_and_merge_per_layer": steps / (ms_n * 1e-3),
                      "tok_s_with_one_batched_all_gather_for_16_layers": steps / (ms_b * 1e-3), "l2": "inputs larger than L2"},
           "clocks": clocks, "gpu_launches": int(launches), "e2e": {"value": None, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0, "note": "not measured for this workload"},
           "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "achieved": ach, "peak": pk["hbm_gbs"] * world, "unit": "GB/s", "frac": ach / (pk["hbm_gbs"] * world), "peak_src": pk["src"],
                        "note": "fraction of N x the single-GPU copy rate: whole-step time (append, partial decode, exchange and merge per layer) against the bytes of the whole sequence", "us_per_launch": ms / steps / N_LAYERS * 1e3, "traffic": None}}
    if world > 1:
        dist.barrier()
    px.close(); ctx.close()
    return res


# ------------------------------------------------------------------------------------------------- the reference arm
def run_reference(args, kind_cfg):
    """The reference's own CPU implementation of the path: its scalar attention math (k_attn_decode restated in the
    oracle; the reference's kernels are Metal and cannot run here) on all host threads. Each step is a bounded sample:
    one of the 16 layers for the whole batch at full context. ms_per_step is the time a step (one layer) really took;
    value is tok/s for the 16 layers of the workload, i.e. that time x16 (labelled in cpu_baseline.sample)."""
    from oracle import kata_oracle as orc
    from kata_b200 import synth
    if kind_cfg[0] != "decode" or kind_cfg[2] != "fp16":   # the reference arm times the headline decode path
        kind_cfg = WORKLOADS["decode_b8"]
    _, B, kv_mode, lmax, lmin = kind_cfg
    world = max(1, args.gpus)
    B_s = min(B, 8)                    # bounded sample: at most 8 sequences per step; CPU tok/s does not depend on the batch size
    lens = synth.seq_lengths(1234, B, lmin, lmax)[:B_s]
    rng = np.random.default_rng(99)
    ks = [rng.standard_normal((int(l) + 1, 1024), dtype=np.float32).astype(np.float16).view(np.uint16) for l in lens]
    vs = [rng.standard_normal((int(l) + 1, 1024), dtype=np.float32).astype(np.float16).view(np.uint16) for l in lens]
    q = rng.standard_normal((B_s, 6144)).astype(np.float32); g = rng.standard_normal((B_s, 6144)).astype(np.float32)
    cores = orc.hw_threads()
    pos = [int(l) for l in lens]
    for _ in range(min(args.warmup, 1)):
        orc.decode_batch(q, g, ks, vs, pos, threads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.decode_batch(q, g, ks, vs, pos, threads=cores)
    dt = (time.perf_counter() - t0) / args.steps
    val = B_s / (dt * N_LAYERS)
    return {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": decode_workload_name(kv_mode, lmax, lmin, B), "batch_per_gpu": B, "global_batch": world * B,
                       "note": "host cores only: a CPU's tok/s does not grow with the GPU count, so the sample below stands for every N"},
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                             "sample": f"each timed step = 1 of the {N_LAYERS} layers for {B_s} sequences at full context (ms_per_step is that one layer); value = sequences / (ms_per_step x {N_LAYERS} layers)"},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def run_fwht(args, rank, world, cfg):
    """The engine's attention output transform (k_rms_fwht mode 3) over cfg[1] rows of 6144 floats: one step = one pass, HBM-bound."""
    import torch
    import torch.distributed as dist
    from kata_b200 import capi
    rows, width = cfg[1], cfg[3]
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev); gen.manual_seed(77 + rank)
    x = torch.randn(rows, width, generator=gen, device=dev); y = torch.empty_like(x)
    sign = torch.where(torch.rand(width, generator=gen, device=dev) < 0.5, -1.0, 1.0).to(torch.float32)
    hx = torch.randn(rows, width).pin_memory(); hy = torch.empty(rows, width).pin_memory()
    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    for _ in range(args.warmup):
        capi.out_fwht(x, sign, out=y)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw0 = time.perf_counter(); e0.record()
    for _ in range(args.steps):
        capi.out_fwht(x, sign, out=y)
    e1.record(); torch.cuda.synchronize(); tw1 = time.perf_counter()
    ms = e0.elapsed_time(e1); clocks = sampler.stop(tw0, tw1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        x.copy_(hx, non_blocking=True); capi.out_fwht(x, sign, out=y); hy.copy_(y, non_blocking=True); torch.cuda.current_stream().synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms, e2e_ms = t.tolist()
    pk = peaks(); nbytes = rows * width * 8.0; ach = nbytes / (ms / args.steps * 1e-3) / 1e9
    return {"metric": METRIC, "value": world * rows * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"attention output transform (sign, 1024-point Walsh-Hadamard per block, 1/32) over {rows} rows of {width} floats per GPU", "l2": "inputs larger than L2 (no flush needed)"},
            "clocks": clocks, "gpu_launches": int(args.steps),
            "e2e": {"value": world * rows * args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": rows * width * 4, "d2h_bytes_per_step": rows * width * 4},
            "roofline": {"bound": "hbm", "kernel": "out_fwht_kernel", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "peak_src": pk["src"],
                         "us_per_launch": ms / args.steps * 1e3, "algorithmic_bytes_per_launch": nbytes, "traffic": None}}


def run_draft(args, rank, world, cfg):
    """The block drafter's attention (k_draft_qk + k_draft_attn per layer, src/draft.cpp:196-209): one step = one drafter round (5 layers, a block
    of T rows over a full window) for each of 4 independent drafters, whose rings together exceed L2. HBM-bound: window x 4 KB per layer."""
    import torch
    import torch.distributed as dist
    from kata_b200 import capi
    T, win, ring, n_layers, n_ctx = cfg[1], cfg[3], cfg[4], 5, 4
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev); gen.manual_seed(99 + rank)
    ctxs = [capi.DraftContext(n_layers, ring, win) for _ in range(n_ctx)]
    qn = (1 + 0.05 * torch.randn(128, generator=gen, device=dev)).contiguous(); kn = (1 + 0.05 * torch.randn(128, generator=gen, device=dev)).contiguous()
    pos0 = 3 * win                                               # a full window behind the block, wrapped around the ring
    for c in ctxs:                                               # context rows through k_draft_ctx_kv, 64 at a time (Draft::kNMax)
        for il in range(n_layers):
            for st in range(pos0 - win, pos0, 64):
                c.qk(il, None, torch.randn(64, 1024, generator=gen, device=dev), torch.randn(64, 1024, generator=gen, device=dev), None, kn, st)
    qin = torch.randn(n_ctx, n_layers, T, 4096, generator=gen, device=dev); kin = torch.randn(n_ctx, n_layers, T, 1024, generator=gen, device=dev); vin = torch.randn(n_ctx, n_layers, T, 1024, generator=gen, device=dev)
    out = torch.empty(n_ctx, n_layers, T, 4096, device=dev)
    h_in = [torch.randn(n_ctx, n_layers, T, w).pin_memory() for w in (4096, 1024, 1024)]; h_out = torch.empty(n_ctx, n_layers, T, 4096).pin_memory()

    qbuf = torch.empty(n_ctx, n_layers, T, 4096, device=dev)

    def step(p, attn_only=False):
        for ci, c in enumerate(ctxs):
            for il in range(n_layers):
                if not attn_only:
                    c.qk(il, qin[ci, il], kin[ci, il], vin[ci, il], qn, kn, p, out=qbuf[ci, il])
                c.attn(il, qbuf[ci, il], p, out=out[ci, il])
    # The kernels take a few microseconds each, less than a launch through the Python binding costs: the device-resident figures replay a
    # CUDA graph of one step (a drafter round at one position), as a native caller's launch loop would run; e2e goes through the plain calls.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(args.warmup):
            step(pos0)
    torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize()
    l0 = sum(c.launches() for c in ctxs)
    g_step, g_attn = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_step):
        step(pos0)
    launches = (sum(c.launches() for c in ctxs) - l0) * args.steps
    with torch.cuda.graph(g_attn):
        step(pos0, attn_only=True)
    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    for _ in range(args.warmup):
        g_step.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw0 = time.perf_counter(); e0.record()
    for i in range(args.steps):
        g_step.replay()
    e1.record(); torch.cuda.synchronize(); tw1 = time.perf_counter()
    ms = e0.elapsed_time(e1); clocks = sampler.stop(tw0, tw1)
    # the attention kernels alone (attention + combine grid per launch), same rotation over drafters and layers
    pk_pos = pos0
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
        g_attn.replay()
    k1.record(); torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / (args.steps * n_ctx * n_layers)
    t0 = time.perf_counter()
    for i in range(args.steps):
        qin.copy_(h_in[0], non_blocking=True); kin.copy_(h_in[1], non_blocking=True); vin.copy_(h_in[2], non_blocking=True)
        step(pos0 + (1 + i) * T)
        h_out.copy_(out, non_blocking=True); torch.cuda.current_stream().synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms, e2e_ms = t.tolist()
    pk = peaks(); nbytes = float(win + T - 1) * 4096.0; ach = nbytes / (kern_ms * 1e-3) / 1e9
    res = {"metric": METRIC, "value": world * n_ctx * T * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
           "config": {"workload": f"block drafter attention: {n_ctx} drafters/GPU x {n_layers} layers, block of {T} rows, window {win} over a ring of {ring}; norm + RoPE + ring append, then attention, per layer",
                      "l2": f"{n_ctx} drafters in rotation: {n_ctx * n_layers * (win + T - 1) * 4096 / 1e6:.0f} MB of ring rows read per step (larger than L2)"},
           "clocks": clocks, "gpu_launches": int(launches),
           "e2e": {"value": world * n_ctx * T * args.steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": sum(h.numel() * 4 for h in h_in), "d2h_bytes_per_step": h_out.numel() * 4},
           "roofline": {"bound": "hbm", "kernel": "draft_attn_kernel", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"], "peak_src": pk["src"],
                        "us_per_launch": kern_ms * 1e3, "algorithmic_bytes_per_launch": nbytes, "traffic": None}}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import kata_oracle as orc
        rings = orc.DraftRing(ring, win)
        rings.k[:] = ctxs[0].ring_read(0, False); rings.v[:] = ctxs[0].ring_read(0, True)
        qh = qbuf[0, 0].cpu().numpy(); cores = orc.hw_threads(); reps = 20
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.draft_attn(qh, rings, pk_pos, threads=cores)
        dt = (time.perf_counter() - t0) / reps
        res["cpu_baseline"] = {"value": T / (dt * n_layers), "unit": "tok/s", "cores": cores, "kind": "port", "sample": f"k_draft_attn restated, 1 of {n_layers} layers of one drafter, mean of {reps} runs ({dt * 1e3:.1f} ms), tok/s extrapolated x{n_layers} layers"}
    for c in ctxs:
        c.close()
    return res


def compact(res):
    """The keys of a workload's result that go into the default line's "extras"."""
    keep = {k: res[k] for k in ("value", "unit", "ms_per_step", "steps", "warmup", "clocks", "e2e", "gpu_launches", "dtype", "scaling") if k in res}
    keep["workload"] = res["config"]["workload"]
    for k in ("l2", "kernel", "tok_s_with_nccl_all_gather_and_merge_per_layer", "tok_s_with_one_batched_all_gather_for_16_layers", "tok_s_one_gpu_same_harness"):
        if k in res["config"]:
            keep[k] = res["config"][k]
    r = res.get("roofline", {})
    keep["roofline"] = {k: r[k] for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "us_per_launch", "peak_src", "note") if k in r}
    if "cpu_baseline" in res:
        keep["cpu_baseline"] = res["cpu_baseline"]
    return keep


def run_workload(name, args, rank, world, steps=None, warmup=None, sustained_s=0.0):
    cfg = WORKLOADS[name]
    if cfg[0] == "decode":
        return run_decode(args, rank, world, cfg, steps=steps, warmup=warmup, sustained_s=sustained_s)
    if cfg[0] == "splitkv":
        return run_splitkv(args, rank, world, cfg, steps=steps, warmup=warmup)
    if cfg[0] == "fwht":
        return run_fwht(args, rank, world, cfg)
    if cfg[0] == "draft":
        return run_draft(args, rank, world, cfg)
    import bench_prefill
    return bench_prefill.run(args, rank, world, cfg, peaks(), ClockSampler, steps=steps, warmup=warmup)


def table(path):
    """Markdown table of a saved bench line (the default line with its extras): what profiles/bench_results.md holds."""
    d = json.loads([l for l in open(path).read().splitlines() if l.startswith("{")][-1])
    rows = [("decode_b8 (the headline line)", d)] + [(k, v) for k, v in d.get("extras", {}).items()]
    out = ["| workload | value (tok/s) | ms/step | e2e (tok/s) | dominant kernel, per launch | achieved | frac of measured peak | SM MHz, reasons | CPU baseline (tok/s, cores) |", "|---|---|---|---|---|---|---|---|---|"]
    for name, v in rows:
        if "roofline" not in v:
            out.append(f"| {name} | {v.get('skipped') or v.get('failed')} | | | | | | | |")
            continue
        r, c, e, cb = v["roofline"], v.get("clocks", {}), v.get("e2e", {}), v.get("cpu_baseline", {})
        ev = e.get("value")
        out.append(f"| {name} | {v['value']:,.0f} | {v['ms_per_step']:.3f} | {'-' if ev is None else format(ev, ',.0f')} | `{r.get('kernel', '')}` {r.get('us_per_launch', 0):.1f} us | {r['achieved']:,.0f} {r['unit']} | {r['frac']:.3f} | {c.get('sm_mhz')}, {','.join(c.get('reasons', [])) or 'none'} | {'-' if not cb or cb.get('value') is None else format(cb['value'], ',.2f')} ({cb.get('cores', '-')}) |")
    if "sustained" in d:
        sgl = d["sustained"]
        out.append("")
        out.append(f"Sustained: the headline step repeated for {sgl['seconds']:.1f} s: {sgl['value']:,.0f} tok/s, {sgl['ms_per_step']:.3f} ms/step, median SM clock {sgl['clocks'].get('sm_mhz')} MHz, reasons {sgl['clocks'].get('reasons')}.")
    return "\n".join(out)


def main():
    t_start = time.perf_counter()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="kata_b200", choices=["kata_b200", "reference"])
    ap.add_argument("--workload", default="decode_b8", choices=sorted(WORKLOADS))
    ap.add_argument("--extras", default=None, help="all | none | comma-separated workload names; default: all for the default workload, none otherwise")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--table", default=None, help="print the markdown table of a saved bench line (a file holding bench.py's output) and exit")
    args = ap.parse_args()
    if args.table:
        print(table(args.table))
        return
    args.warmup = max(args.warmup, 3) if args.impl == "kata_b200" else args.warmup
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, WORKLOADS[args.workload])), flush=True)
        return

    import torch
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback for the product path"
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    default = args.workload == "decode_b8"
    res = run_workload(args.workload, args, rank, world, sustained_s=2.0 if default else 0.0)
    want = args.extras if args.extras is not None else ("all" if default else "none")
    names = [] if want == "none" else (EXTRAS_ONE_GPU if world == 1 else EXTRAS_MULTI_GPU) if want == "all" else [n for n in want.split(",") if n]
    if names:
        extras = {}
        e_steps, e_warm = max(3, min(args.steps, 10)), 3
        for name in names:
            if name not in WORKLOADS:
                extras[name] = {"skipped": "unknown workload"}
                continue
            over = torch.tensor([1.0 if time.perf_counter() - t_start > EXTRAS_BUDGET_S else 0.0], device="cuda")
            if world > 1:
                import torch.distributed as dist
                dist.all_reduce(over, op=dist.ReduceOp.MAX)   # every rank takes the same decision
            if over.item() > 0:
                extras[name] = {"skipped": f"not started: the run had already taken more than {EXTRAS_BUDGET_S:.0f} s"}
                continue
            t0 = time.perf_counter()
            try:
                r = run_workload(name, args, rank, world, steps=e_steps, warmup=e_warm)
                extras[name] = compact(r); extras[name]["wall_s"] = round(time.perf_counter() - t0, 1)
            except Exception as ex:   # an extra that fails must not take the headline line with it; it says what happened
                if world > 1:
                    raise
                extras[name] = {"failed": f"{type(ex).__name__}: {ex}"[:300]}
                torch.cuda.empty_cache()
        res["extras"] = extras
    res["wall_s"] = round(time.perf_counter() - t_start, 1)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
