"""Prefill workloads of bench.py: pp512 (benchmark config 2) and chunked prefill + T=2 verify (config 5).

pp512: 512 prompt tokens, bf16 projections, all 16 layers; a step = per layer prep (norm, RoPE, append) + causal flash
prefill. chunked: a 7,300-token prompt whose first 3,600 positions are restored through the KV-plane API, then prefilled
in 512-token chunks (7 x 512 + 116) against the growing prefix, then one T=2 verify step; all 16 layers.
The roofline object is the prefill kernel alone: useful FLOPs = sum over query rows of keys attended x 24 x 256 x 4.
"""
from __future__ import annotations

import time

import numpy as np

N_LAYERS = 16


def _flops(pos0: int, m: int) -> float:
    return float(sum(range(pos0 + 1, pos0 + m + 1))) * 24 * 256 * 4


def run(args, rank, world, cfg, pk, ClockSampler, steps=None, warmup=None):
    import torch
    import torch.distributed as dist
    from kata_b200 import capi

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    kind, B, kv_mode, total, prefix = cfg
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev); gen.manual_seed(99 + rank)
    restore = prefix if kind == "chunked" else 0
    chunks, p = [], restore
    while p < total:
        m = min(512, total - p); chunks.append((p, m)); p += m
    ctx = capi.AttnContext(N_LAYERS, [total + 8] * B, kv_mode=kv_mode)
    seqs = list(range(B))
    qn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    kn = (1 + 0.05 * torch.randn(N_LAYERS, 256, generator=gen, device=dev)).contiguous()
    bf = torch.bfloat16
    if restore:   # build the prefix once, export its planes, reset, import them: the prefix-cache restore
        for layer in range(N_LAYERS):
            for s in seqs:
                for st in range(0, restore, 1024):
                    m = min(1024, restore - st)
                    ctx.prep(layer, [s], [st], m, None, torch.randn(1, m, 1024, generator=gen, device=dev).to(bf), torch.randn(1, m, 1024, generator=gen, device=dev).to(bf), None, kn[layer], h0=24, nh=8)
        ctx.check()
        saved = [[[ctx.plane_read(l, s, pl, 0, restore) for pl in range(ctx.kv_planes())] for s in seqs] for l in range(N_LAYERS)]
        ctx.reset()
        for l in range(N_LAYERS):
            for s in seqs:
                for pl in range(ctx.kv_planes()):
                    ctx.plane_write(l, s, pl, 0, saved[l][s][pl])
        del saved
    mmax = max(m for _, m in chunks)
    # one set of projections per chunk shape, reused across layers (values do not affect the timing)
    qfull = torch.randn(B, mmax, 12288, generator=gen, device=dev).to(bf)
    kproj = torch.randn(B, mmax, 1024, generator=gen, device=dev).to(bf)
    vproj = torch.randn(B, mmax, 1024, generator=gen, device=dev).to(bf)
    q16 = torch.empty(B, mmax, 6144, dtype=torch.float16, device=dev)
    gate = torch.empty(B, mmax, 6144, dtype=torch.float32, device=dev)
    out = torch.empty(B, mmax, 6144, dtype=torch.float32, device=dev)

    def sl(t, m):
        return t if m == mmax else t[:, :m].contiguous()

    # End to end (host is not None): the projections of a (chunk, layer) go up on one copy stream while the one before computes, its output rows come
    # down on another while the next one computes; device-side input and output buffers are doubled for that.
    cs_in, cs_out = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = {}

    def step(with_prep=True, host=None):
        cur = torch.cuda.current_stream()
        if host is not None and not bufs:
            bufs["in"] = [(qfull, kproj, vproj), (torch.empty_like(qfull), torch.empty_like(kproj), torch.empty_like(vproj))]; bufs["out"] = [out, torch.empty_like(out)]
        work = [(p0, m, layer) for (p0, m) in chunks for layer in range(N_LAYERS)]
        ev_in, ev_done, ev_down = {}, {}, {}
        if host is not None:
            cs_in.wait_stream(cur); cs_out.wait_stream(cur)
        for i, (p0, m, layer) in enumerate(work):
            qf_, kp_, vp_ = (qfull, kproj, vproj) if host is None else bufs["in"][i & 1]
            out_ = out if host is None else bufs["out"][i & 1]
            if host is not None:
                with torch.cuda.stream(cs_in):
                    if i >= 2: cs_in.wait_event(ev_done[i - 2])          # the item that used this input buffer has computed
                    qf_[:, :m].copy_(host[0][:, :m], non_blocking=True); kp_[:, :m].copy_(host[1][:, :m], non_blocking=True); vp_[:, :m].copy_(host[2][:, :m], non_blocking=True)
                    ev_in[i] = torch.cuda.Event(); ev_in[i].record(cs_in)
                cur.wait_event(ev_in[i])
                if i >= 2: cur.wait_event(ev_down[i - 2])                 # the rows that sat in this output buffer are on the host
            if m == mmax:
                if with_prep:
                    ctx.prep(layer, seqs, [p0] * B, m, qf_, kp_, vp_, qn[layer], kn[layer], q16=q16, gate=gate)
                ctx.prefill(layer, seqs, [p0] * B, m, q16, gate, out=out_)
            else:
                q_, g_ = (ctx.prep(layer, seqs, [p0] * B, m, sl(qf_, m), sl(kp_, m), sl(vp_, m), qn[layer], kn[layer])[0::2] if with_prep else (sl(q16, m), sl(gate, m)))
                o_ = ctx.prefill(layer, seqs, [p0] * B, m, q_, g_)
                out_[:, :m].copy_(o_)
            if host is not None:
                ev_done[i] = torch.cuda.Event(); ev_done[i].record(cur)
                with torch.cuda.stream(cs_out):
                    cs_out.wait_event(ev_done[i])
                    host[3][:, :m].copy_(out_[:, :m], non_blocking=True)
                    ev_down[i] = torch.cuda.Event(); ev_down[i].record(cs_out)
        if kind == "chunked":   # the T=2 verify that follows (target token plus one draft)
            for layer in range(N_LAYERS):
                q2, _, g2 = ctx.prep(layer, seqs, [total] * B, 2, sl(qfull, 2), sl(kproj, 2), sl(vproj, 2), qn[layer], kn[layer])
                ctx.decode(layer, seqs, [total] * B, 2, q2, g2)
        if host is not None:
            cs_out.synchronize(); cur.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # A pp512 layer is some 20 us of GPU work, less than two calls through the Python binding cost the host: the device-resident figures of
    # that workload replay a CUDA graph of one step (what a native caller's launch loop achieves); e2e goes through the plain calls.
    use_graph = kind == "prefill" and B * total <= 4096
    sampler = ClockSampler(torch.cuda.current_device()); sampler.start()
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(warmup):
            step()
    torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize()
    ctx.check()
    l0 = ctx.launches()
    run_step = step
    if use_graph:
        g_step = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_step):
            step()
        per_step = ctx.launches() - l0
        run_step = g_step.replay
        for _ in range(3):
            run_step()
    l0 = ctx.launches(); barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tw0 = time.perf_counter(); torch.cuda.profiler.start(); e0.record()
    for _ in range(steps):
        run_step()
    e1.record(); barrier(); torch.cuda.profiler.stop(); tw1 = time.perf_counter()
    ms = e0.elapsed_time(e1); launches = per_step * steps if use_graph else ctx.launches() - l0
    clocks = sampler.stop(tw0, tw1)
    ctx.check()
    assert torch.isfinite(out).all()
    # the prefill kernel alone (q16/gate of the last prep are reused)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    full = [(p0, m) for (p0, m) in chunks if m == mmax]
    for (p0, m) in full:
        ctx.prefill(0, seqs, [p0] * B, m, q16, gate, out=out)
    def kernel_only():
        for (p0, m) in full:
            for layer in range(N_LAYERS):
                ctx.prefill(layer, seqs, [p0] * B, m, q16, gate, out=out)
    run_k = kernel_only
    if use_graph:
        g_k = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_k):
            kernel_only()
        run_k = g_k.replay
        run_k()
    torch.cuda.synchronize(); k0.record()
    reps = max(2, steps)
    for _ in range(reps):
        run_k()
    k1.record(); torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / (reps * N_LAYERS * len(full))
    flops_launch = B * float(np.mean([_flops(p0, m) for (p0, m) in full]))
    # end to end with host buffers
    host = [torch.randn(B, mmax, 12288).to(bf).pin_memory(), torch.randn(B, mmax, 1024).to(bf).pin_memory(), torch.randn(B, mmax, 1024).to(bf).pin_memory(), torch.empty(B, mmax, 6144).pin_memory()]
    step(host=host); barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step(host=host)
    barrier(); e2e_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms, e2e_ms = t.tolist()
    toks = sum(m for _, m in chunks)
    ach = flops_launch / (kern_ms * 1e-3) / 1e12
    h2d = N_LAYERS * B * toks * (12288 + 2048) * 2; d2h = N_LAYERS * B * toks * 6144 * 4
    name = "pp512" if kind == "prefill" else f"chunked prefill {restore}->{total} in 512-token chunks after a plane restore at {restore}, then a T=2 verify"
    res = {"metric": "gated-GQA attn tok/s (decode@32K, pp512); HBM GB/s & TC util vs peak", "value": world * B * toks * steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
           "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
           "config": {"workload": f"{name}; {N_LAYERS} layers, {kv_mode} KV, bf16 projections, batch {B}/GPU, prep+prefill per layer", "batch_per_gpu": B, "global_batch": world * B,
                      "l2": ("each step streams the 16 layers' caches and activations, together larger than L2 (no flush needed)" if kind == "chunked" or B > 4 else
                             "NOT larger than L2: one layer's K/V for 512 tokens is 2 MB and the 16 layers' activations 450 MB are streamed once; the kernel is launch- and latency-bound at this size, not bandwidth-bound"),
                      "kernel": "prefill_tc5_kernel (tcgen05, cta_group::2)" + ("" if kv_mode == "fp16" else " after expand_codes_kernel") + " (items cut between CTA pairs are merged in the kernel)",
                      "launch": "CUDA graph replay of one step for value and roofline (a layer is shorter than two calls through the Python binding); plain calls for e2e" if use_graph else "plain calls"},
           "clocks": clocks, "gpu_launches": int(launches),
           "e2e": {"value": world * B * toks * steps / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "roofline": {"bound": "tensor", "kernel": "prefill_tc5_kernel", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": ach / pk["bf16_tflops"], "frac_of_sustained": ach / pk["bf16_tflops_sustained"], "peak_src": pk["src"],
                        "us_per_launch": kern_ms * 1e3, "algorithmic_flops_per_launch": flops_launch, "traffic": None}}
    if rank == 0 and not args.no_cpu_baseline and kv_mode == "fp16":
        res["cpu_baseline"] = cpu_baseline(ctx, full[-1], q16, gate, chunks)
    ctx.close()
    bufs.clear()
    del qfull, kproj, vproj, q16, gate, out, host
    torch.cuda.empty_cache()
    return res


def cpu_baseline(ctx, chunk, q16, gate, chunks):
    """The reference's own CPU check (tools/probe_flash.cpp:29-34: fp64 softmax(q k) v sigmoid(g) per token and head), as restated in
    the oracle's kor_formula_f64 (bit-equal to the reference's lines compiled in oracle/_ref on the reference's inputs), on all host
    threads, on a bounded sample: the last full chunk of sequence 0, layer 0, every 4th query row; extrapolated to all rows, chunks and
    layers by FLOPs."""
    from oracle import kata_oracle as orc
    p0, m = chunk
    n = p0 + m
    planes = orc.KvPlanes(n)
    planes.k[:] = ctx.plane_read(0, 0, 0, 0, n).view(np.uint16).reshape(n, 1024); planes.v[:] = ctx.plane_read(0, 0, 1, 0, n).view(np.uint16).reshape(n, 1024)
    q = q16[0, :m].cpu().numpy().view(np.uint16); g = gate[0, :m].cpu().numpy()
    cores = orc.hw_threads(); t_step = 4 if p0 == 0 else 16   # a bounded sample: a few seconds of host time
    t0 = time.perf_counter()
    orc.formula_f64(np.ascontiguousarray(q), np.ascontiguousarray(g), planes, p0, t_step=t_step, threads=cores)
    dt = time.perf_counter() - t0
    flops_sample = sum(p0 + r + 1 for r in range(0, m, t_step)) * 24 * 256 * 4.0
    rate = flops_sample / dt                                  # useful FLOP/s of the fp64 loop on these cores
    step_flops = N_LAYERS * sum(_flops(c0, cm) for c0, cm in chunks)   # one sequence, all chunks, all layers
    return {"value": sum(cm for _, cm in chunks) * rate / step_flops, "unit": "tok/s", "cores": cores, "kind": "port", "useful_gflops": rate / 1e9,
            "sample": f"fp64 check loop of tools/probe_flash.cpp restated (kor_formula_f64), layer 0, sequence 0, chunk at position {p0}, every {t_step}th of {m} rows ({dt:.2f} s); tok/s extrapolated by useful FLOPs to all rows, chunks and {N_LAYERS} layers"}
