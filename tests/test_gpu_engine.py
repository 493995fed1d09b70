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


@pytest.mark.parametrize("mode", ["fp16", "int8", "int8v"])
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
    b = capi.AttnContext(n_attn, [400], kv_mode=mode); mb = capi.AttnContext(1, [400]); got = C.c_uint32()
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
