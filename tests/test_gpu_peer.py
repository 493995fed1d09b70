"""The split-KV exchange between GPUs (kata_attn_peer_*): parts pushed into the peers' buffers and merged in one kernel.

One GPU: the single-rank path, and a wait that runs out (a peer that never calls) reported as a status with the context still usable.
Two GPUs (skipped otherwise): two processes, one per GPU, against the NCCL all-gather + merge and the oracle."""
import os
import socket

import numpy as np
import pytest
import torch

from kata_b200 import multi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from kata_b200 import capi as m
    m.lib()
    return m


@pytest.fixture(scope="module")
def orc():
    from oracle import kata_oracle as m
    m.lib()
    return m


def _parts(seed, n_ranks, T):
    rng = np.random.default_rng(seed)
    p = rng.standard_normal((n_ranks, T * 24, 258)).astype(np.float32)
    p[:, :, 256] = rng.uniform(-3, 3, (n_ranks, T * 24)); p[:, :, 257] = rng.uniform(0.5, 40, (n_ranks, T * 24))
    return p, rng.standard_normal((T, 6144)).astype(np.float32)


def test_single_rank_exchange_is_normalise_and_gate(capi):
    px = capi.PeerExchange(0, 1)
    for T in (1, 2, 1):
        p, gate = _parts(T, 1, T)
        out = px.exchange_merge(torch.from_numpy(p[0]).cuda(), T, torch.from_numpy(gate).cuda())
        px.check()
        want = multi.merge_parts_numpy(p, gate.reshape(T * 24, 256)).reshape(T, 6144)
        assert np.abs(out.cpu().numpy() - want).max() < 1e-5
    px.close()


def test_wait_that_runs_out_is_a_status_not_a_hang(capi):
    # two ranks' buffers in one process; rank 1 never calls, so rank 0's wait for its rows must give up and say so
    a = capi.PeerExchange(0, 2, group=False); b = capi.PeerExchange(1, 2, group=False)
    bufs = [a.buffer(), b.buffer()]
    a.open_pointers(bufs); b.open_pointers(bufs)
    a.set_wait_polls(20000)                                    # a few tens of milliseconds
    p, gate = _parts(3, 1, 2)
    out = torch.full((2, 6144), 7.0, device="cuda")
    a.exchange_merge(torch.from_numpy(p[0]).cuda(), 2, torch.from_numpy(gate).cuda(), out=out)
    with pytest.raises(capi.KataError) as e:
        a.check()
    assert e.value.code == 5 and "rank 1" in str(e.value)     # KATA_ERR_DEVICE_WAIT
    assert (out == 7.0).all()                                  # nothing was written for that call
    a.check()                                                  # the error word was cleared; the GPU still answers
    ctx = capi.AttnContext(1, [64])
    ctx.reset(); ctx.check()
    # The two exchanges are now out of step (a has counted one call, b none): without a resynchronisation every later exchange would time
    # out. After kata_attn_peer_resync with the same call number on both, b's rows reach a. (One GPU runs the two kernels one after the
    # other, so b, which goes first, cannot see a's rows and gives up after its short limit, as expected; a, second, finds b's rows.)
    a.resync(10); b.resync(10)
    b.set_wait_polls(2000)
    p2, gate2 = _parts(4, 2, 1)
    b.exchange_merge(torch.from_numpy(p2[1]).cuda(), 1, torch.from_numpy(gate2).cuda())
    out_a = a.exchange_merge(torch.from_numpy(p2[0]).cuda(), 1, torch.from_numpy(gate2).cuda())
    a.check()
    with pytest.raises(capi.KataError):
        b.check()
    want = multi.merge_parts_numpy(p2, gate2.reshape(24, 256)).reshape(1, 6144)
    assert np.abs(out_a.cpu().numpy() - want).max() < 1e-5
    a.close(); b.close()


def _rank_main(rank, world, port, Lk, k, v, q16, gate, ret):
    import torch.distributed as dist
    from kata_b200 import capi
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lo, hi = multi.split_keys(Lk, world)[rank]
    ctx = capi.AttnContext(1, [max(hi - lo, 1) + 8])
    if hi > lo:
        ctx.plane_write(0, 0, 0, 0, k[lo:hi]); ctx.plane_write(0, 0, 1, 0, v[lo:hi])
    px = capi.PeerExchange(rank, world)
    outs = []
    for T, pb in ((2, Lk - 2), (1, Lk - 1), (1, Lk - 700), (2, Lk - 2)):   # several calls: both buffer parities, changing T
        qd = torch.from_numpy(q16[pb:pb + T]).cuda().view(torch.float16); gd = torch.from_numpy(gate[pb:pb + T]).cuda()
        part = ctx.decode_partial(0, 0, pb, T, lo, hi, qd)
        fused = px.exchange_merge(part, T, gd) if pb != Lk - 1 else px.decode(ctx, 0, 0, pb, T, lo, hi, qd, gd)   # the one-call form once
        parts = torch.empty((world,) + tuple(part.shape), device="cuda")
        dist.all_gather_into_tensor(parts, part)
        nccl = ctx.merge_parts(parts, T, gd)
        ctx.check(); px.check()
        outs.append((fused.cpu().numpy(), nccl.cpu().numpy()))
    if rank == 0:
        ret.put(outs)
    dist.barrier(); px.close(); dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_push_and_merge_across_two_gpus(orc):
    import torch.multiprocessing as mp
    world, Lk = 2, 3000
    planes = orc.KvPlanes(Lk)
    qn, kn = synth.norm_weights(83); qf, kp, vp = synth.token_rows_fast(83, Lk)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn"); ret = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, Lk, planes.k, planes.v, orc.cvt_q_half(q), gate, ret)) for r in range(world)]
    for p in procs: p.start()
    outs = ret.get(timeout=240)
    for p in procs: p.join(timeout=60)
    assert all(p.exitcode == 0 for p in procs)
    for (fused, nccl), (T, pb) in zip(outs, ((2, Lk - 2), (1, Lk - 1), (1, Lk - 700), (2, Lk - 2))):
        assert np.array_equal(fused, nccl)                               # the same merge arithmetic, wherever the parts travelled
        ref = orc.formula_f32(q[pb:pb + T], gate[pb:pb + T], planes, pb)
        d = np.abs(fused - ref)
        assert d.max() < 2e-3 and d.mean() < 2e-4


def test_one_rank_peer_decode_equals_plain_decode_short_and_long(capi):
    # kata_attn_peer_decode on a group of one rank is a plain decode. When a sequence's keys are cut between more than 8 CTAs its rows leave
    # through the combine grid, which then does the exchange itself (no launch of its own); otherwise (here: one CTA per 1024 keys of a
    # 300-key sequence) the stand-alone exchange kernel follows the decode kernel. Both must equal kata_attn_decode.
    px = capi.PeerExchange(0, 1)
    gen = torch.Generator(device="cuda"); gen.manual_seed(51)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    for L, chunk in ((300, 1024), (300, 0), (20000, 0)):
        ctx = capi.AttnContext(1, [L + 8], dec_chunk=chunk)
        for st in range(0, L, 1024):
            m = min(1024, L - st)
            ctx.prep(0, [0], [st], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
        for T in (1, 2):
            qf = torch.randn(1, T, 12288, generator=gen, device="cuda"); kp = torch.randn(1, T, 1024, generator=gen, device="cuda"); vp = torch.randn(1, T, 1024, generator=gen, device="cuda")
            q16, _, g = ctx.prep(0, [0], [L], T, qf, kp, vp, qn, kn)
            want = ctx.decode(0, [0], [L], T, q16, g)
            l0 = ctx.launches()
            got = px.decode(ctx, 0, 0, L, T, 0, 1 << 30, q16, g[0])
            px.check(); ctx.check()
            assert ctx.launches() - l0 == (1 if chunk else 2)      # decode kernel (+ combine grid, which then carries the exchange)
            assert (got - want[0]).abs().max().item() < 1e-5
        ctx.close()
    px.close()


def test_one_rank_peer_layers_step_equals_the_plain_layer_loop(capi):
    # kata_attn_peer_layers_step (prep + split-KV decode, layer after layer, in one call) on a group of one rank against kata_attn_layers_step
    px = capi.PeerExchange(0, 1)
    gen = torch.Generator(device="cuda"); gen.manual_seed(52)
    NL, L = 3, 9000
    kn = (1 + 0.05 * torch.randn(NL, 256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(NL, 256, generator=gen, device="cuda")).contiguous()
    ctxs = [capi.AttnContext(NL, [L + 8]) for _ in range(2)]
    for layer in range(NL):
        for st in range(0, L, 1024):
            m = min(1024, L - st)
            k = torch.randn(1, m, 1024, generator=gen, device="cuda"); v = torch.randn(1, m, 1024, generator=gen, device="cuda")
            for ctx in ctxs:
                ctx.prep(layer, [0], [st], m, None, k, v, None, kn[layer], h0=24, nh=8)
    for T in (1, 2):
        qf = torch.randn(NL, 1, T, 12288, generator=gen, device="cuda"); kp = torch.randn(NL, 1, T, 1024, generator=gen, device="cuda"); vp = torch.randn(NL, 1, T, 1024, generator=gen, device="cuda")
        q16 = torch.empty(NL, 1, T, 6144, dtype=torch.float16, device="cuda"); g = torch.empty(NL, 1, T, 6144, device="cuda")
        want = torch.empty(NL, 1, T, 6144, device="cuda"); got = torch.empty(NL, T, 6144, device="cuda")
        pos = L + (0 if T == 1 else 1)
        ctxs[0].layers_step(NL, [0], [pos], T, qf, kp, vp, qn, kn, q16, g, want)
        px.layers_step(ctxs[1], NL, 0, pos, T, 0, 1 << 30, True, qf, kp, vp, qn, kn, q16.clone(), g.clone(), got)
        px.check(); ctxs[0].check(); ctxs[1].check()
        assert (got - want[:, 0]).abs().max().item() < 1e-5
    px.close()
