"""GPU tests of the C++ Engine mirror (csrc/attn_engine.hpp: the engine-named call sequences) and of the split-KV path
across GPUs with an NCCL all-gather of the (O, m, l) parts (needs two GPUs; skipped otherwise)."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch

from kata_b200 import multi, synth

pytestmark = pytest.mark.gpu


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_engine_mirror_prefill_step_verify(orc):
    from kata_b200 import capi
    L = capi.lib()
    L.kata_engine_create.restype = C.c_void_p
    n0 = 150
    qn, kn = synth.norm_weights(81)
    qf, kp, vp = synth.token_rows_fast(81, n0 + 3)
    planes = orc.KvPlanes(256)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    eng = C.c_void_p(L.kata_engine_create(torch.cuda.current_device(), 2, 256, 0))
    assert eng.value
    dq, dk, dv, dqn, dkn = _dev(qf), _dev(kp), _dev(vp), _dev(qn), _dev(kn)
    q16 = torch.empty(n0, 6144, dtype=torch.float16, device="cuda"); g = torch.empty(n0, 6144, device="cuda"); out = torch.empty(n0, 6144, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.kata_engine_prefill_attn(eng, 1, n0, 0, p(dq), p(dk), p(dv), p(dqn), p(dkn), p(q16), p(g), p(out), st) == 0
    o1 = torch.empty(1, 6144, device="cuda"); o2 = torch.empty(2, 6144, device="cuda")
    assert L.kata_engine_step_attn(eng, 1, n0, p(dq[n0:n0 + 1].contiguous()), p(dk[n0:n0 + 1].contiguous()), p(dv[n0:n0 + 1].contiguous()), p(dqn), p(dkn), p(q16), p(g), p(o1), st) == 0
    assert L.kata_engine_verify2_attn(eng, 1, n0 + 1, p(dq[n0 + 1:].contiguous()), p(dk[n0 + 1:].contiguous()), p(dv[n0 + 1:].contiguous()), p(dqn), p(dkn), p(q16), p(g), p(o2), st) == 0
    assert L.kata_engine_check(eng, st) == 0
    ref = orc.formula_f32(q, gate, planes, 0)
    for got, want in ((out.cpu().numpy(), ref[:n0]), (o1.cpu().numpy(), ref[n0:n0 + 1]), (o2.cpu().numpy(), ref[n0 + 1:])):
        d = np.abs(got - want)
        assert np.isfinite(got).all() and d.max() < 2e-3 and d.mean() < 2e-4
    L.kata_engine_destroy(eng)


def _rank_main(rank, world, port, Lk, T, k, v, q16, gate, ret):
    import torch.distributed as dist
    from kata_b200 import capi
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    lo, hi = multi.split_keys(Lk, world)[rank]
    ctx = capi.AttnContext(1, [max(hi - lo, 1) + 8])
    if hi > lo:
        ctx.plane_write(0, 0, 0, 0, k[lo:hi]); ctx.plane_write(0, 0, 1, 0, v[lo:hi])
    part = ctx.decode_partial(0, 0, Lk - T, T, lo, hi, torch.from_numpy(q16).cuda().view(torch.float16))
    parts = torch.empty((world,) + tuple(part.shape), device="cuda")
    dist.all_gather_into_tensor(parts, part)
    out = ctx.merge_parts(parts, T, torch.from_numpy(gate).cuda())
    ctx.check()
    if rank == 0:
        ret.put(out.cpu().numpy())
    dist.barrier(); dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_split_kv_across_gpus_nccl(orc):
    import torch.multiprocessing as mp
    world, Lk, T = 2, 3000, 2
    planes = orc.KvPlanes(Lk)
    qn, kn = synth.norm_weights(82); qf, kp, vp = synth.token_rows_fast(82, Lk)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    ref = orc.formula_f32(q[Lk - T:], gate[Lk - T:], planes, Lk - T)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn"); ret = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, Lk, T, planes.k, planes.v, orc.cvt_q_half(q[Lk - T:]), gate[Lk - T:], ret)) for r in range(world)]
    for p in procs: p.start()
    out = ret.get(timeout=240)
    for p in procs: p.join(timeout=60)
    assert all(p.exitcode == 0 for p in procs)
    d = np.abs(out - ref)
    assert d.max() < 2e-3 and d.mean() < 2e-4


@pytest.mark.parametrize("mode", ["fp16", "int8", "int8v", "int8g"])
def test_checkpoint_kv_segments_round_trip(tmp_path, mode):
    # save the KV segments of a prefilled context, restore them into a fresh one: planes identical (the reference's
    # test_cache.sh identity checks), another numerics mode refuses the file, a truncated file is refused and leaves zeros
    from kata_b200 import capi
    L = capi.lib()
    n, n_attn = 333, 3
    gen = torch.Generator(device="cuda"); gen.manual_seed(9)
    kn = torch.ones(256, device="cuda")
    a = capi.AttnContext(n_attn, [400], kv_mode=mode); m = capi.AttnContext(1, [400])
    for layer in range(n_attn):
        a.prep(layer, [0], [0], n, None, torch.randn(1, n, 1024, generator=gen, device="cuda"), torch.randn(1, n, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    m.prep(0, [0], [0], n, None, torch.randn(1, n, 1024, generator=gen, device="cuda"), torch.randn(1, n, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    a.check(); m.check()
    toks = np.arange(1000, 1000 + n + 20, dtype=np.int32); tp = toks.ctypes.data_as(C.c_void_p)
    path = str(tmp_path / "p.ckpt").encode()
    args = (C.c_uint64(42), n_attn, C.c_uint64(4096), C.c_uint64(8192))
    assert L.kata_ckpt_write_kv(a.h, m.h, 0, path, tp, n, *args, 5) == 0
    # not under its final name yet: the engine's own segments are still holes and the reference's restore would accept the file as it is
    b = capi.AttnContext(n_attn, [400], kv_mode=mode); mb = capi.AttnContext(1, [400]); got = C.c_uint32()
    assert not os.path.exists(path.decode()) and L.kata_ckpt_read_kv(b.h, mb.h, 0, path, tp, len(toks), *args, C.byref(got)) != 0
    assert L.kata_ckpt_publish(path) == 0
    assert L.kata_ckpt_read_kv(b.h, mb.h, 0, path, tp, len(toks), *args, C.byref(got)) == 0 and got.value == n
    for layer in range(n_attn):
        for pl in range(a.kv_planes()):
            assert np.array_equal(a.plane_read(layer, 0, pl, 0, 400), b.plane_read(layer, 0, pl, 0, 400))
    for pl in range(2):
        assert np.array_equal(m.plane_read(0, 0, pl, 0, 400), mb.plane_read(0, 0, pl, 0, 400))
    other = capi.AttnContext(n_attn, [400], kv_mode="int8" if mode == "fp16" else "fp16")
    assert L.kata_ckpt_read_kv(other.h, None, 0, path, tp, len(toks), *args, C.byref(got)) == 2
    with open(path, "r+b") as f:
        f.truncate(os.path.getsize(path) - 4096)
    c = capi.AttnContext(n_attn, [400], kv_mode=mode)
    assert L.kata_ckpt_read_kv(c.h, None, 0, path, tp, len(toks), *args, C.byref(got)) == 2
    assert (c.plane_read(0, 0, 0, 0, 400) == 0).all()


def test_engine_mirror_wide_verify_mtp_rows_quantiser_and_output_transform(orc):
    # the remaining Engine-named sequences: verifyWide (T = 5), encMtpKv + mtpRows on the MTP head's cache (first valid key at position 1),
    # dKvQuant on an int8 engine, dRmsFwht mode 3, resetState and the plane accessors
    from kata_b200 import capi
    L = capi.lib()
    L.kata_engine_create.restype = C.c_void_p; L.kata_engine_numerics_tag.restype = C.c_char_p; L.kata_engine_kv_plane_row.restype = C.c_size_t
    L.kata_engine_kv_plane_ptr.restype = C.c_void_p; L.kata_engine_mtp_kv_ptr.restype = C.c_void_p
    p = lambda t: C.c_void_p(t.data_ptr())
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    n0, T = 90, 5
    qn, kn = synth.norm_weights(83)
    qf, kp, vp = synth.token_rows_fast(83, n0 + T)
    planes = orc.KvPlanes(128)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    ref = orc.formula_f32(q, gate, planes, 0)
    eng = C.c_void_p(L.kata_engine_create(torch.cuda.current_device(), 1, 128, 0))
    assert eng.value and L.kata_engine_numerics_tag(eng) == b"fp16" and L.kata_engine_kv_planes(eng) == 2 and L.kata_engine_kv_plane_row(eng, 1) == 2048
    assert L.kata_engine_kv_plane_ptr(eng, 0, 0) and L.kata_engine_mtp_kv_ptr(eng, 1)
    dq, dk, dv, dqn, dkn = _dev(qf), _dev(kp), _dev(vp), _dev(qn), _dev(kn)
    q16 = torch.empty(n0, 6144, dtype=torch.float16, device="cuda"); g = torch.empty(n0, 6144, device="cuda"); out = torch.empty(n0, 6144, device="cuda")
    assert L.kata_engine_prefill_attn(eng, 0, n0, 0, p(dq), p(dk), p(dv), p(dqn), p(dkn), p(q16), p(g), p(out), st) == 0
    ow = torch.empty(T, 6144, device="cuda")
    assert L.kata_engine_verify_wide_attn(eng, 0, T, n0, p(dq[n0:].contiguous()), p(dk[n0:].contiguous()), p(dv[n0:].contiguous()), p(dqn), p(dkn), p(q16), p(g), p(ow), st) == 0
    assert L.kata_engine_check(eng, st) == 0
    d = np.abs(ow.cpu().numpy() - ref[n0:])
    assert d.max() < 2e-3 and d.mean() < 2e-4
    # MTP head: rows 0..n0-1 appended with encMtpKv (K/V slots only), then two rows through mtpRows; keys start at position 1
    assert L.kata_engine_enc_mtp_kv(eng, n0, 0, p(dk), p(dv), p(dkn), st) == 0
    om = torch.empty(2, 6144, device="cuda")
    assert L.kata_engine_mtp_rows_attn(eng, 2, n0, p(dq[n0:n0 + 2].contiguous()), p(dk[n0:n0 + 2].contiguous()), p(dv[n0:n0 + 2].contiguous()), p(dqn), p(dkn), p(q16), p(g), p(om), st) == 0
    assert L.kata_engine_check(eng, st) == 0
    ref1 = orc.formula_f32(q[n0:n0 + 2], gate[n0:n0 + 2], planes, n0, first_pos=1)
    d = np.abs(om.cpu().numpy() - ref1)
    assert d.max() < 2e-3 and d.mean() < 2e-4
    hk = np.empty((n0 + 2, 1024), np.uint16)
    assert L.kata_engine_mtp_plane_read(eng, 0, n0 + 2, hk.ctypes.data_as(C.c_void_p)) == 0
    assert (hk != planes.k[:n0 + 2]).mean() < 0.02            # the same rows as the trunk cached (sin/cos may differ by an ulp)
    # the transform after attention
    sign = np.where(np.random.default_rng(1).random(6144) < 0.5, -1.0, 1.0).astype(np.float32)
    xp = torch.empty_like(ow)
    assert L.kata_engine_attn_out_fwht(eng, p(ow), p(_dev(sign)), p(xp), T, st) == 0
    assert np.array_equal(xp.cpu().numpy().view(np.uint32), orc.out_fwht(ow.cpu().numpy(), sign).view(np.uint32))
    # resetState zeroes both caches
    assert L.kata_engine_reset_state(eng, st) == 0 and L.kata_engine_check(eng, st) == 0
    hz = np.ones((8, 1024), np.uint16)
    assert L.kata_engine_kv_plane_read(eng, 0, 0, 8, hz.ctypes.data_as(C.c_void_p)) == 0 and not hz.any()
    assert L.kata_engine_mtp_plane_read(eng, 1, 8, hz.ctypes.data_as(C.c_void_p)) == 0 and not hz.any()
    L.kata_engine_destroy(eng)
    # dKvQuant on an int8 engine: codes and scales equal to the oracle quantiser applied to the same fp16 rows
    e8 = C.c_void_p(L.kata_engine_create(torch.cuda.current_device(), 2, 64, 1))
    assert e8.value and L.kata_engine_numerics_tag(e8) == b"fp16+kv8" and L.kata_engine_kv_planes(e8) == 4
    rng = np.random.default_rng(2)
    ks = rng.standard_normal((7, 1024)).astype(np.float16); vs = (3 * rng.standard_normal((7, 1024))).astype(np.float16)
    assert L.kata_engine_kv_quant(e8, 7, 10, 1, p(_dev(ks)), p(_dev(vs)), st) == 0 and L.kata_engine_check(e8, st) == 0
    want = orc.KvPlanes(64, int8=True)
    orc.kv_quant(ks.view(np.uint16), vs.view(np.uint16), want, 10, 0)
    got = [np.empty((17, w), dt) for w, dt in ((1024, np.int8), (1024, np.int8), (4, np.uint16), (4, np.uint16))]
    for pl, a in enumerate(got):
        assert L.kata_engine_kv_plane_read(e8, 1, pl, 17, a.ctypes.data_as(C.c_void_p)) == 0
    for a, w in zip(got, (want.k, want.v, want.ksc, want.vsc)):
        assert np.array_equal(a[10:17], w[10:17]) and not a[:10].any()
    L.kata_engine_destroy(e8)


def _head_rank_main(rank, world, port, ret):
    import torch.distributed as dist
    from kata_b200 import capi
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    L, T = 3070, 2                                                    # 3072 keys: a whole multiple of the 512-key split
    gen = torch.Generator(device="cuda"); gen.manual_seed(41)          # the same inputs on every rank
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    lo, n = multi.shard_kv_heads(world)[rank]
    mine = capi.AttnContext(1, [L + 8], dec_chunk=512); mine.set_kv_heads(lo, n)
    whole = capi.AttnContext(1, [L + 8], dec_chunk=512) if rank == 0 else None
    for st in range(0, L, 1024):
        m = min(1024, L - st)
        kp = torch.randn(1, m, 1024, generator=gen, device="cuda"); vp = torch.randn(1, m, 1024, generator=gen, device="cuda")
        for c in (mine, whole):
            if c is not None:
                c.prep(0, [0], [st], m, None, kp, vp, None, kn, h0=24, nh=8)
    qf = torch.randn(1, T, 12288, generator=gen, device="cuda"); kp = torch.randn(1, T, 1024, generator=gen, device="cuda"); vp = torch.randn(1, T, 1024, generator=gen, device="cuda")
    q16, _, g = mine.prep(0, [0], [L], T, qf, kp, vp, qn, kn)
    out = torch.zeros(1, T, 6144, device="cuda")
    mine.decode(0, [0], [L], T, q16, g, out=out); mine.check()
    block = out[0, :, multi.head_columns(lo, n)].contiguous()          # this rank's column block: T x 6144 / world values
    blocks = [torch.empty_like(block) for _ in range(world)]
    dist.all_gather(blocks, block)                                     # the one exchange of the head-sharded group, after attention
    if rank == 0:
        q16w, _, gw = whole.prep(0, [0], [L], T, qf, kp, vp, qn, kn)
        want = whole.decode(0, [0], [L], T, q16w, gw); whole.check()
        ret.put(bool(torch.equal(torch.cat(blocks, dim=1), want[0])))
    dist.barrier(); dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_head_groups_across_two_gpus():
    # two ranks own two KV heads each; their column blocks, gathered over NCCL, are the single-GPU rows bit for bit
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn"); ret = ctx.Queue()
    procs = [ctx.Process(target=_head_rank_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    ok = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
    assert ok and all(p.exitcode == 0 for p in procs)


@pytest.mark.gpu
@pytest.mark.parametrize("kv_mode,T", [("fp16", 1), ("int8", 2), ("fp16", 5)])
def test_host_step_equals_the_device_calls(kv_mode, T):
    from kata_b200 import capi
    # a whole step (three layers, ragged batch) with projections and output rows in pinned host memory: same bits as prep + decode on device rows
    n_layers, lens = 3, [300, 1, 777]
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    ctxs = [capi.AttnContext(n_layers, [1024] * 3, kv_mode=kv_mode) for _ in range(2)]
    qn = (1 + 0.05 * torch.randn(n_layers, 256, generator=gen, device="cuda")).contiguous(); kn = (1 + 0.05 * torch.randn(n_layers, 256, generator=gen, device="cuda")).contiguous()
    seqs = [0, 1, 2]
    for layer in range(n_layers):
        for s, L in enumerate(lens):
            k = torch.randn(1, L, 1024, generator=gen, device="cuda"); v = torch.randn(1, L, 1024, generator=gen, device="cuda")
            for ctx in ctxs:
                ctx.prep(layer, [s], [0], L, None, k, v, None, kn[layer], h0=24, nh=8)
    hq = torch.randn(n_layers, 3, T, 12288).pin_memory(); hk = torch.randn(n_layers, 3, T, 1024).pin_memory(); hv = torch.randn(n_layers, 3, T, 1024).pin_memory()
    hout = torch.zeros(n_layers, 3, T, 6144).pin_memory()
    hs = capi.HostStep(ctxs[0], max_n=4, max_T=8)
    for rep in range(2):   # the second step appends at the next positions and reuses the doubled device rows
        pos = [L + rep * T for L in lens]
        hs.run(n_layers, seqs, pos, T, hq, hk, hv, qn, kn, hout)
        if rep == 0:   # the same layers through the one-call loop over device rows
            dq16 = torch.empty(n_layers, 3, T, 6144, dtype=torch.float16, device="cuda"); dg = torch.empty(n_layers, 3, T, 6144, device="cuda"); dout = torch.empty(n_layers, 3, T, 6144, device="cuda")
            third = capi.AttnContext(n_layers, [1024] * 3, kv_mode=kv_mode)
            for layer in range(n_layers):
                for pl in range(third.kv_planes()):
                    for s_, L_ in enumerate(lens):
                        third.plane_write(layer, s_, pl, 0, ctxs[1].plane_read(layer, s_, pl, 0, L_))
            third.layers_step(n_layers, seqs, pos, T, hq.cuda(), hk.cuda(), hv.cuda(), qn, kn, dq16, dg, dout)
            third.check(); third.close()
        torch.cuda.current_stream().synchronize()
        ctxs[0].check()
        for layer in range(n_layers):
            q16, _, g = ctxs[1].prep(layer, seqs, pos, T, hq[layer].cuda(), hk[layer].cuda(), hv[layer].cuda(), qn[layer], kn[layer])
            ref = ctxs[1].decode(layer, seqs, pos, T, q16, g)
            assert torch.equal(ref.cpu(), hout[layer])
            if rep == 0:
                assert torch.equal(ref, dout[layer])
        ctxs[1].check()
    hs.close()
