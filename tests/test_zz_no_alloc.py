"""kata_attn_decode_static: the decode entry point for callers that cannot allocate device memory (engines that hand
all GPU memory to their own pools, loops that ban cudaMalloc because it synchronises the device). It works on
caller-owned K/V rows without a context, keeping its split-KV scratch in a fixed array inside the library.

This file is named so that pytest collects it last. The test calls the entry point through the C ABI twice in a row (the
second call reuses the scratch the first one left behind) and compares each result with kata_attn_decode on a context
holding the same rows. It passes alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decode_static_matches_context_decode_twice():
    from kata_b200 import capi
    assert torch.cuda.is_available()
    gen = torch.Generator(device="cuda"); gen.manual_seed(77)
    lens = [3000, 517, 1]
    ctx = capi.AttnContext(1, [4096, 1024, 64])
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    for s, L in enumerate(lens):
        for start in range(0, L + 2, 1024):
            m = min(1024, L + 2 - start)
            ctx.prep(0, [s], [start], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    ctx.check()
    # the caller-owned copy of the same rows: one [rows][1024] fp16 tensor for K and one for V, sequences back to back
    row0, ks, vs = [], [], []
    for s, cap in enumerate([4096, 1024, 64]):
        row0.append(sum(k.shape[0] for k in ks))
        ks.append(torch.from_numpy(ctx.plane_read(0, s, 0, 0, cap).view(np.float16).reshape(cap, 1024).copy()).cuda())
        vs.append(torch.from_numpy(ctx.plane_read(0, s, 1, 0, cap).view(np.float16).reshape(cap, 1024).copy()).cuda())
    k_rows, v_rows = torch.cat(ks).contiguous(), torch.cat(vs).contiguous()

    for T, first_pos in ((1, 0), (2, 1)):          # two calls in a row; the second also exercises T=2 and first_pos=1
        pos = [L - 1 if T == 1 else L for L in lens]   # T=2 reads the two extra rows appended above
        if first_pos:
            pos = [max(p, first_pos) for p in pos]
        qfull = torch.randn(3, T, 12288, generator=gen, device="cuda")
        q16 = (qfull.view(3, T, 24, 512)[..., :256].reshape(3, T, 6144) * 0.0625).to(torch.float16).contiguous()
        gate = qfull.view(3, T, 24, 512)[..., 256:].reshape(3, T, 6144).contiguous()
        want = ctx.decode(0, [0, 1, 2], pos, T, q16, gate, first_pos=first_pos)
        ctx.check()
        rc, got = capi.decode_static(k_rows, v_rows, row0, pos, T, q16, gate, first_pos=first_pos)
        torch.cuda.synchronize()
        assert rc == capi.OK
        d = (got - want).abs()
        assert torch.isfinite(got).all() and d.max().item() < 2e-3 and d.mean().item() < 2e-4, (d.max().item(), d.mean().item())
        assert d.max().item() < 1e-5   # same kernel, same work split: the two paths should agree far inside the tolerance

    # Eight sequences of 2-3K keys: every (sequence, KV head) segment is cut between a few CTAs, so the merge runs inside the decode kernel
    # on the tickets kept in the static array; the second call finds the tickets the first one left (re-armed by the kernel, cleared on
    # the stream before each launch).
    lens8 = [2100 + 113 * i for i in range(8)]
    ctx8 = capi.AttnContext(1, [3072] * 8)
    for s, L in enumerate(lens8):
        for start in range(0, L, 1024):
            m = min(1024, L - start)
            ctx8.prep(0, [s], [start], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    k8 = torch.cat([torch.from_numpy(ctx8.plane_read(0, s, 0, 0, 3072).view(np.float16).reshape(3072, 1024).copy()) for s in range(8)]).cuda().contiguous()
    v8 = torch.cat([torch.from_numpy(ctx8.plane_read(0, s, 1, 0, 3072).view(np.float16).reshape(3072, 1024).copy()) for s in range(8)]).cuda().contiguous()
    for rep in range(2):
        pos8 = [L - 1 - rep for L in lens8]
        qfull = torch.randn(8, 1, 12288, generator=gen, device="cuda")
        q16 = (qfull.view(8, 1, 24, 512)[..., :256].reshape(8, 1, 6144) * 0.0625).to(torch.float16).contiguous()
        gate = qfull.view(8, 1, 24, 512)[..., 256:].reshape(8, 1, 6144).contiguous()
        want = ctx8.decode(0, list(range(8)), pos8, 1, q16, gate)
        ctx8.check()
        rc, got = capi.decode_static(k8, v8, [3072 * s for s in range(8)], pos8, 1, q16, gate)
        torch.cuda.synchronize()
        assert rc == capi.OK and torch.isfinite(got).all() and (got - want).abs().max().item() < 1e-5
    ctx8.close()

    assert capi.lib().kata_attn_decode_static_check(None) == capi.OK   # no bounded wait ran out in the last call

    # sizes beyond the stated maximum are rejected with a range error before anything is launched
    n = 9
    rc, _ = capi.decode_static(k_rows, v_rows, [0] * n, [0] * n, 1, torch.zeros(n, 1, 6144, dtype=torch.float16, device="cuda"), torch.zeros(n, 1, 6144, device="cuda"))
    assert rc == 2
    ctx.close()
