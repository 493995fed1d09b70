"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Bars: int8 codes and fp16 scales bit-exact; floating-point outputs within max-abs 2e-3 and mean-abs 2e-4 of the fp32
evaluation of the same formula (the tolerance the benchmark statement gives). Shapes follow the reference's own check
(tools/probe_flash.cpp: a prefix, a ragged tail tile, NaN beyond the valid keys) and its cross-path equalities.
"""
import numpy as np
import pytest
import torch

from kata_b200 import synth

pytestmark = pytest.mark.gpu

TOL_MAX, TOL_MEAN = 2e-3, 2e-4
NAN16 = 0x7E00


def _close(got, ref, tmax=TOL_MAX, tmean=TOL_MEAN):
    got = np.asarray(got, np.float32)
    d = np.abs(got - ref)
    assert np.isfinite(got).all(), "non-finite output"
    assert d.max() < tmax and d.mean() < tmean, (float(d.max()), float(d.mean()))


@pytest.fixture(scope="module")
def capi():
    from kata_b200 import capi as m
    assert torch.cuda.is_available()
    m.lib()
    return m


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _upload_planes(ctx, planes, layer=0, seq=0, n=None):
    n = planes.max_ctx if n is None else n
    ctx.plane_write(layer, seq, 0, 0, planes.k[:n])
    ctx.plane_write(layer, seq, 1, 0, planes.v[:n])
    if planes.int8 or planes.mode == 3:
        ctx.plane_write(layer, seq, 2, 0, planes.ksc[:n])
        ctx.plane_write(layer, seq, 3, 0, planes.vsc[:n])
    elif planes.mode == 2:   # int8v: {K fp16, V int8, V scales}
        ctx.plane_write(layer, seq, 2, 0, planes.vsc[:n])


def _oracle_fill(orc, seed, L, max_ctx, int8=False, poison=False, fast=False, layer=0, seq=0, int8v=False, int8g=False):
    planes = orc.KvPlanes(max_ctx, int8=int8, poison=poison, int8v=int8v, int8g=int8g)
    qn, kn = synth.norm_weights(seed, layer)
    qf, kp, vp = (synth.token_rows_fast if fast else synth.token_rows)(seed, L, layer=layer, seq=seq)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    return planes, q, gate, (qf, kp, vp, qn, kn)


# ------------------------------------------------------------------------------------------------ prep and quantiser
def test_prep_fp16_matches_oracle(capi, orc):
    L, pos0 = 70, 300
    planes = orc.KvPlanes(512)
    qn, kn = synth.norm_weights(21)
    qf, kp, vp = synth.token_rows(21, L, start=pos0)
    q_ref, gate_ref = orc.prep(qf, kp, vp, qn, kn, planes, pos0)
    ctx = capi.AttnContext(2, [512])
    q16, q32, gate = ctx.prep(1, [0], [pos0], L, _dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn), want_q32=True)
    ctx.check()
    assert np.array_equal(gate.cpu().numpy()[0], gate_ref)
    assert np.abs(q32.cpu().numpy()[0] - q_ref).max() < 2e-6
    assert np.abs(q16.cpu().numpy()[0].astype(np.float32) * 16 - q_ref).max() < 6e-3
    v = ctx.plane_read(1, 0, 1, 0, 512).view(np.uint16).reshape(512, 1024)
    assert np.array_equal(v, planes.v)                                    # V is a pure fp16 rounding: bit-exact
    k = ctx.plane_read(1, 0, 0, 0, 512).view(np.uint16).reshape(512, 1024)
    assert (k[:pos0] == 0).all() and (k[pos0 + L:] == 0).all()            # zero-initialised, only rows pos0.. written
    kd = np.abs(k.view(np.float16).astype(np.float32) - planes.k.view(np.float16).astype(np.float32))
    assert kd.max() < 4e-3 and (k != planes.k).mean() < 0.02              # sin/cos differ from libm by an ulp at most
    assert (ctx.plane_read(0, 0, 0, 0, 512) == 0).all()                   # the other layer is untouched


def test_prep_kv_only_and_bf16(capi, orc):
    L = 33
    qn, kn = synth.norm_weights(22)
    qf, kp, vp = synth.token_rows(22, L)
    kb, vb = synth.to_bf16_bits(kp), synth.to_bf16_bits(vp)
    planes = orc.KvPlanes(64)
    orc.prep(None, synth.bf16_bits_to_f32(kb), synth.bf16_bits_to_f32(vb), qn, kn, planes, 5, h0=24, nh=8)
    ctx = capi.AttnContext(1, [64])
    ctx.prep(0, [0], [5], L, None, _dev(kb[None]).view(torch.bfloat16), _dev(vb[None]).view(torch.bfloat16), None, _dev(kn), h0=24, nh=8)
    ctx.check()
    v = ctx.plane_read(0, 0, 1, 0, 64).view(np.uint16).reshape(64, 1024)
    k = ctx.plane_read(0, 0, 0, 0, 64).view(np.float16).reshape(64, 1024).astype(np.float32)
    assert np.array_equal(v, planes.v)
    assert np.abs(k - planes.k.view(np.float16).astype(np.float32)).max() < 4e-3


@pytest.mark.parametrize("mode", ["rint", "half_away"])
def test_kv_quant_bit_exact(capi, orc, mode):
    rng = np.random.default_rng(31)
    T = 40
    rows = (rng.standard_normal((T, 1024)) * rng.uniform(0.01, 30, (T, 1))).astype(np.float16)
    rows[1] = 0
    rows[2, :8] = [127, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]
    rows[2, 8:256] = 0
    rows[3, :2] = [1001.0, -1001.0]
    rows[3, 2:256] = 0
    rows[4, :4] = [6e-6, -3e-6, 1e-6, 6e-8]
    rows[4, 4:256] = 0
    vrows = rows[::-1].copy()
    ref = orc.KvPlanes(64, int8=True)
    orc.kv_quant(rows.view(np.uint16), vrows.view(np.uint16), ref, 7, 1 if mode == "half_away" else 0)
    ctx = capi.AttnContext(1, [64], kv_mode="int8", quant_round=mode)
    ctx.kv_quant(0, 0, _dev(rows.view(np.uint16)).view(torch.float16), _dev(vrows.view(np.uint16)).view(torch.float16), 7)
    ctx.check()
    assert ctx.tag() == "fp16+kv8" and ctx.kv_planes() == 4 and [ctx.plane_row_bytes(p) for p in range(5)] == [1024, 1024, 8, 8, 0]
    assert np.array_equal(ctx.plane_read(0, 0, 0, 0, 64).view(np.int8).reshape(64, 1024), ref.k)
    assert np.array_equal(ctx.plane_read(0, 0, 1, 0, 64).view(np.int8).reshape(64, 1024), ref.v)
    assert np.array_equal(ctx.plane_read(0, 0, 2, 0, 64).view(np.uint16).reshape(64, 4), ref.ksc)
    assert np.array_equal(ctx.plane_read(0, 0, 3, 0, 64).view(np.uint16).reshape(64, 4), ref.vsc)
    want = [127, 0, 2, 2, 0, -2, -2, 4] if mode == "rint" else [127, 1, 2, 3, -1, -2, -3, 4]
    assert ref.k[9, :8].tolist() == want


def test_prep_int8_quantise_on_append_bit_exact(capi, orc):
    # the fused path must equal: fp16 rows as the fp16 path caches them -> the reference quantiser
    L = 50
    qn, kn = synth.norm_weights(23)
    qf, kp, vp = synth.token_rows(23, L)
    c16 = capi.AttnContext(1, [64])
    c8 = capi.AttnContext(1, [64], kv_mode="int8")
    args = (_dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn))
    c16.prep(0, [0], [3], L, *args)
    c8.prep(0, [0], [3], L, *args)
    c16.check(); c8.check()
    k16 = c16.plane_read(0, 0, 0, 3, L).view(np.uint16).reshape(L, 1024)
    v16 = c16.plane_read(0, 0, 1, 3, L).view(np.uint16).reshape(L, 1024)
    ref = orc.KvPlanes(64, int8=True)
    orc.kv_quant(k16, v16, ref, 3, 0)
    assert np.array_equal(c8.plane_read(0, 0, 0, 0, 64).view(np.int8).reshape(64, 1024), ref.k)
    assert np.array_equal(c8.plane_read(0, 0, 1, 0, 64).view(np.int8).reshape(64, 1024), ref.v)
    assert np.array_equal(c8.plane_read(0, 0, 2, 0, 64).view(np.uint16).reshape(64, 4), ref.ksc)
    assert np.array_equal(c8.plane_read(0, 0, 3, 0, 64).view(np.uint16).reshape(64, 4), ref.vsc)


# ------------------------------------------------------------------------------------------------ decode
@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("T", [1, 2])
def test_decode_lengths(capi, orc, int8, T):
    Lmax = 700
    planes, q, gate, _ = _oracle_fill(orc, 41, Lmax, 1024, int8=int8, poison=not int8)
    ctx = capi.AttnContext(1, [1024], kv_mode="int8" if int8 else "fp16")
    for L in (T, 15, 16, 17, 63, 64, 65, 127, 128, 129, 300, 700):
        if L < T:
            continue
        # the cache holds exactly L rows; everything beyond is NaN (fp16) or garbage codes with NaN scales (int8)
        cut = orc.KvPlanes(1024, int8=int8, poison=True) if not int8 else orc.KvPlanes(1024, int8=True)
        cut.k[:L], cut.v[:L] = planes.k[:L], planes.v[:L]
        if int8:
            cut.ksc[:L], cut.vsc[:L] = planes.ksc[:L], planes.vsc[:L]
            cut.k[L:], cut.v[L:] = 77, -77
            cut.ksc[L:], cut.vsc[L:] = NAN16, NAN16
        _upload_planes(ctx, cut)
        pb = L - T
        out = ctx.decode(0, [0], [pb], T, _dev(orc.cvt_q_half(q[pb:L])[None]).view(torch.float16), _dev(gate[pb:L][None]))
        ctx.check()
        got = out.cpu().numpy()[0]
        _close(got, orc.formula_f32(q[pb:L], gate[pb:L], cut, pb))
        assert np.abs(got - orc.dec_attn(q[pb:L], gate[pb:L], cut, pb, T=T)).max() < 3e-4   # same rounding points as the restated kernel


def test_decode_first_pos_one(capi, orc):
    planes, q, gate, _ = _oracle_fill(orc, 42, 90, 128)
    planes.k[0] = NAN16
    planes.v[0] = NAN16
    ctx = capi.AttnContext(1, [128])
    _upload_planes(ctx, planes)
    out = ctx.decode(0, [0], [88], 2, _dev(orc.cvt_q_half(q[88:90])[None]).view(torch.float16), _dev(gate[88:90][None]), first_pos=1)
    ctx.check()
    _close(out.cpu().numpy()[0], orc.formula_f32(q[88:90], gate[88:90], planes, 88, first_pos=1))


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("dec_chunk", [0, 64, 1024])
def test_decode_ragged_batch_and_split_merge(capi, orc, int8, dec_chunk):
    lens = [1, 2000, 37, 513, 1200]
    ctx = capi.AttnContext(3, [2048, 2048, 64, 1024, 2048], kv_mode="int8" if int8 else "fp16", dec_chunk=dec_chunk)
    layer, T = 2, 1
    refs, q16s, gates = [], [], []
    for s, L in enumerate(lens):
        planes, q, gate, _ = _oracle_fill(orc, 50 + s, L, int(ctx.max_ctx[s]), int8=int8, fast=True, seq=s)
        _upload_planes(ctx, planes, layer=layer, seq=s)
        refs.append(orc.formula_f32(q[L - 1:], gate[L - 1:], planes, L - 1)[0])
        q16s.append(orc.cvt_q_half(q[L - 1:]))
        gates.append(gate[L - 1:])
    order = [4, 0, 3, 1, 2]                                    # the batch lists sequences in any order
    out = ctx.decode(layer, order, [lens[s] - 1 for s in order], T, _dev(np.stack([q16s[s] for s in order])).view(torch.float16), _dev(np.stack([gates[s] for s in order])))
    ctx.check()
    got = out.cpu().numpy()
    for i, s in enumerate(order):
        _close(got[i, 0], refs[s])


def test_decode_scalar_path_and_cross_path(capi, orc):
    planes, q, gate, _ = _oracle_fill(orc, 43, 1500, 2048, fast=True)
    ctx = capi.AttnContext(1, [2048])
    _upload_planes(ctx, planes)
    for T, pb in ((1, 1499), (2, 1498), (8, 100)):
        qs, gs = q[pb:pb + T], gate[pb:pb + T]
        out = ctx.decode_scalar(0, [0], [pb], T, _dev(qs[None]), _dev(gs[None]))
        ctx.check()
        ref = orc.attn_split_combine(qs, gs, planes, pb, T=T, S=min(32, max(1, (pb + T) // 64)))
        assert np.abs(out.cpu().numpy()[0] - ref).max() < 2e-5
        # the matrix path agrees with the scalar path on the same cache (the reference's KATA_SCALAR_DEC cross-check); T = 8 is the wide verify
        m = ctx.decode(0, [0], [pb], T, _dev(orc.cvt_q_half(qs)[None]).view(torch.float16), _dev(gs[None]))
        _close(m.cpu().numpy()[0], out.cpu().numpy()[0])


@pytest.mark.parametrize("int8", [False, True])
def test_wide_verify_matches_single_token_decodes(capi, orc, int8):
    # T = 5 and 8 query tokens per sequence (Engine::verifyWide) on the matrix path, two ragged sequences: every token must equal its own T = 1 decode
    lens = (700, 333)
    ctx = capi.AttnContext(1, [1024, 512], kv_mode="int8" if int8 else "fp16")
    fills = []
    for s, n in enumerate(lens):
        planes, q, gate, _ = _oracle_fill(orc, 90 + s, n, int(ctx.max_ctx[s]), int8=int8, fast=True, seq=s)
        _upload_planes(ctx, planes, seq=s); fills.append((planes, q, gate))
    for T in (5, 8):
        pbs = [n - T for n in lens]
        q16 = np.stack([orc.cvt_q_half(fills[s][1][pbs[s]:pbs[s] + T]) for s in range(2)]); g = np.stack([fills[s][2][pbs[s]:pbs[s] + T] for s in range(2)])
        wide = ctx.decode(0, [0, 1], pbs, T, _dev(q16).view(torch.float16), _dev(g)).cpu().numpy()
        ctx.check()
        for s in range(2):
            _close(wide[s], orc.formula_f32(fills[s][1][pbs[s]:pbs[s] + T], fills[s][2][pbs[s]:pbs[s] + T], fills[s][0], pbs[s]))
            for t in range(T):
                one = ctx.decode(0, [s], [pbs[s] + t], 1, _dev(q16[s:s + 1, t:t + 1]).view(torch.float16), _dev(g[s:s + 1, t:t + 1])).cpu().numpy()[0, 0]
                assert np.abs(one - wide[s, t]).max() < 1e-4


def test_verify_t2_equals_two_decodes(capi, orc):
    planes, q, gate, _ = _oracle_fill(orc, 44, 400, 512)
    ctx = capi.AttnContext(1, [512])
    _upload_planes(ctx, planes)
    q16 = _dev(orc.cvt_q_half(q)).view(torch.float16)
    g = _dev(gate)
    v = ctx.decode(0, [0], [398], 2, q16[398:400][None].contiguous(), g[398:400][None].contiguous()).cpu().numpy()[0]
    d0 = ctx.decode(0, [0], [398], 1, q16[398:399][None].contiguous(), g[398:399][None].contiguous()).cpu().numpy()[0, 0]
    d1 = ctx.decode(0, [0], [399], 1, q16[399:400][None].contiguous(), g[399:400][None].contiguous()).cpu().numpy()[0, 0]
    ctx.check()
    assert np.abs(v[0] - d0).max() < 1e-5 and np.abs(v[1] - d1).max() < 1e-5


def test_config1_golden_decode(capi, orc):
    # benchmark config 1: one layer, 512 keys, one token; GPU prep builds the cache, then the committed golden output
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))
    seed, L = 1001, 512
    qn, kn = synth.norm_weights(seed)
    qf, kp, vp = synth.token_rows(seed, L)
    ctx = capi.AttnContext(1, [L])
    q16, _, gate = ctx.prep(0, [0], [0], L, _dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn))
    out = ctx.decode(0, [0], [L - 1], 1, q16[:, L - 1:].contiguous(), gate[:, L - 1:].contiguous())
    ver = ctx.decode(0, [0], [L - 2], 2, q16[:, L - 2:].contiguous(), gate[:, L - 2:].contiguous())
    ctx.check()
    _close(out.cpu().numpy()[0, 0], g["c1_decode_f32"])
    assert np.abs(out.cpu().numpy()[0, 0] - g["c1_decode"]).max() < 3e-4
    assert np.abs(ver.cpu().numpy()[0] - g["c1_verify_t2"]).max() < 3e-4
    v = ctx.plane_read(0, 0, 1, 0, L).view(np.uint16).reshape(L, 1024)
    assert np.array_equal(v[[0, 1, 255, 511]], g["c1_v_rows"])
    c8 = capi.AttnContext(1, [L], kv_mode="int8")
    q16b, _, gateb = c8.prep(0, [0], [0], L, _dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn))
    ver8 = c8.decode(0, [0], [L - 2], 2, q16b[:, L - 2:].contiguous(), gateb[:, L - 2:].contiguous())
    c8.check()
    assert np.array_equal(c8.plane_read(0, 0, 1, 0, L).view(np.int8).reshape(L, 1024)[[0, 1, 255, 511]], g["q8_v_codes"])
    assert np.array_equal(c8.plane_read(0, 0, 3, 0, L).view(np.uint16).reshape(L, 4), g["q8_v_scales"])
    assert (c8.plane_read(0, 0, 2, 0, L).view(np.uint16).reshape(L, 4) != g["q8_k_scales"]).mean() < 0.02
    assert np.abs(ver8.cpu().numpy()[0] - g["q8_verify_t2"]).max() < 2e-3


def test_split_kv_partials_merge(capi, orc):
    # three "ranks" hold contiguous key slices (as three sequences of one context); merged partials == single-context decode
    L, T = 1000, 2
    planes, q, gate, _ = _oracle_fill(orc, 45, L, 1024, fast=True)
    bounds = [(0, 400), (400, 401), (401, 1000), (1000, 1300)]   # the last rank holds no key yet
    ctx = capi.AttnContext(1, [1024] * 4)
    for s, (lo, hi) in enumerate(bounds):
        n = max(0, min(hi, L) - lo)
        if n:
            ctx.plane_write(0, s, 0, 0, planes.k[lo:lo + n])
            ctx.plane_write(0, s, 1, 0, planes.v[lo:lo + n])
    pb = L - T
    q16 = _dev(orc.cvt_q_half(q[pb:L])).view(torch.float16)
    parts = torch.stack([ctx.decode_partial(0, s, pb, T, lo, hi, q16) for s, (lo, hi) in enumerate(bounds)])
    out = ctx.merge_parts(parts, T, _dev(gate[pb:L]))
    ctx.check()
    assert parts[3, :, 257].abs().max().item() == 0 and torch.isinf(parts[3, :, 256]).all()
    _close(out.cpu().numpy(), orc.formula_f32(q[pb:L], gate[pb:L], planes, pb))


# ------------------------------------------------------------------------------------------------ int8v: keys fp16, values int8
def _cut_v8(orc, planes, n, max_ctx):
    """The first n rows of an int8v cache; beyond them NaN keys, garbage value codes and NaN value scales."""
    cut = orc.KvPlanes(max_ctx, int8v=True, poison=True)
    cut.k[:n], cut.v[:n], cut.vsc[:n] = planes.k[:n], planes.v[:n], planes.vsc[:n]
    cut.v[n:], cut.vsc[n:] = -77, NAN16
    return cut


def test_int8v_planes_tag_and_append(capi, orc):
    # KATA_KV=int8v (src/engine.cpp:54-59, src/engine.h:71-81): planes {K fp16, V int8, V scales}, tag suffix "+kv8v"
    L, pos0 = 50, 3
    qn, kn = synth.norm_weights(24)
    qf, kp, vp = synth.token_rows(24, L)
    c16, cv = capi.AttnContext(1, [64]), capi.AttnContext(1, [64], kv_mode="int8v")
    assert cv.kv_planes() == 3 and [cv.plane_row_bytes(i) for i in range(4)] == [2048, 1024, 8, 0] and cv.tag() == "fp16+kv8v"
    args = (_dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn))
    q16a, _, ga = c16.prep(0, [0], [pos0], L, *args)
    q16b, _, gb = cv.prep(0, [0], [pos0], L, *args)
    c16.check(); cv.check()
    assert torch.equal(q16a, q16b) and torch.equal(ga, gb)
    assert np.array_equal(cv.plane_read(0, 0, 0, 0, 64), c16.plane_read(0, 0, 0, 0, 64))          # keys: the fp16 path's rows, bit for bit
    ref = orc.KvPlanes(64, int8v=True)
    orc.prep(qf, kp, vp, qn, kn, ref, pos0)
    assert np.array_equal(cv.plane_read(0, 0, 1, 0, 64).view(np.int8).reshape(64, 1024), ref.v)   # values: the reference quantiser, bit for bit
    assert np.array_equal(cv.plane_read(0, 0, 2, 0, 64).view(np.uint16).reshape(64, 4), ref.vsc)
    # stand-alone quantise call: value rows only
    v16 = c16.plane_read(0, 0, 1, pos0, L).view(np.float16).reshape(L, 1024)
    cv.reset()
    cv.kv_quant(0, 0, None, _dev(v16), pos0)
    cv.check()
    assert np.array_equal(cv.plane_read(0, 0, 1, 0, 64).view(np.int8).reshape(64, 1024), ref.v)
    assert np.array_equal(cv.plane_read(0, 0, 2, 0, 64).view(np.uint16).reshape(64, 4), ref.vsc)
    assert (cv.plane_read(0, 0, 0, 0, 64) == 0).all()


@pytest.mark.parametrize("T", [1, 2])
def test_int8v_decode_lengths(capi, orc, T):
    planes, q, gate, _ = _oracle_fill(orc, 45, 700, 1024, int8v=True, fast=True)
    ctx = capi.AttnContext(1, [1024], kv_mode="int8v")
    for L in (T, 15, 16, 17, 31, 33, 64, 65, 129, 300, 700):
        if L < T:
            continue
        cut = _cut_v8(orc, planes, L, 1024)
        _upload_planes(ctx, cut)
        pb = L - T
        out = ctx.decode(0, [0], [pb], T, _dev(orc.cvt_q_half(q[pb:L])[None]).view(torch.float16), _dev(gate[pb:L][None]))
        ctx.check()
        got = out.cpu().numpy()[0]
        _close(got, orc.formula_f32(q[pb:L], gate[pb:L], cut, pb))
        assert np.abs(got - orc.dec_attn(q[pb:L], gate[pb:L], cut, pb, T=T)).max() < 3e-4   # k_attn_dec_split_k16v8 restated: same rounding points


@pytest.mark.parametrize("dec_chunk", [0, 64])
def test_int8v_ragged_batch_split_merge_and_wide_verify(capi, orc, dec_chunk):
    lens = [9, 2000, 37, 513, 1200]
    ctx = capi.AttnContext(2, [2048, 2048, 64, 1024, 2048], kv_mode="int8v", dec_chunk=dec_chunk)
    fills = []
    for s, L in enumerate(lens):
        planes, q, gate, _ = _oracle_fill(orc, 55 + s, L, int(ctx.max_ctx[s]), int8v=True, fast=True, seq=s)
        _upload_planes(ctx, planes, layer=1, seq=s); fills.append((planes, q, gate))
    order = [4, 0, 3, 1, 2]
    for T in (1, 5):
        pbs = [lens[s] - T for s in order]
        q16 = np.stack([orc.cvt_q_half(fills[s][1][lens[s] - T:]) for s in order]); g = np.stack([fills[s][2][lens[s] - T:] for s in order])
        got = ctx.decode(1, order, pbs, T, _dev(q16).view(torch.float16), _dev(g)).cpu().numpy()
        ctx.check()
        for i, s in enumerate(order):
            _close(got[i], orc.formula_f32(fills[s][1][lens[s] - T:], fills[s][2][lens[s] - T:], fills[s][0], lens[s] - T))


@pytest.mark.parametrize("legacy", [False, True], ids=["tcgen05", "mma"])
def test_int8v_prefill(capi, orc, legacy):
    planes, q, gate, _ = _oracle_fill(orc, 62, 700, 1024, int8v=True, fast=True)
    ctx = capi.AttnContext(1, [1024], kv_mode="int8v", legacy_prefill=legacy)
    _upload_planes(ctx, _cut_v8(orc, planes, 700, 1024))
    for pb, M in ((300, 70), (0, 1), (0, 17), (0, 130), (353, 17), (190, 510)):
        n = pb + M
        sub = _cut_v8(orc, planes, n, 1024)
        out = ctx.prefill(0, [0], [pb], M, _dev(orc.cvt_q_half(q[pb:n])[None]).view(torch.float16), _dev(gate[pb:n][None]))
        ctx.check()
        got = out.cpu().numpy()[0]
        _close(got, orc.formula_f32(q[pb:n], gate[pb:n], sub, pb))
        if M <= 130:
            assert np.abs(got - orc.flash_prefill(orc.cvt_q_half(q[pb:n]), gate[pb:n], sub, pb)).max() < 3e-4   # k_flash_prefill_k16v8 restated


# ------------------------------------------------------------------------------------------------ prefill
@pytest.mark.parametrize("int8,legacy", [(False, False), (False, True), (True, False), (True, True)], ids=["fp16-tcgen05", "fp16-mma", "int8-tcgen05", "int8-mma"])
def test_prefill_probe_shape(capi, orc, int8, legacy):
    # the reference's probe: 70 rows (ragged tail) at position 300, NaN beyond the valid keys; plus M = 1, 15, 16, 17 and pos 0
    planes, q, gate, _ = _oracle_fill(orc, 61, 370, 512, int8=int8, poison=not int8, fast=True)
    if int8:
        planes.ksc[370:], planes.vsc[370:] = NAN16, NAN16
    ctx = capi.AttnContext(1, [512], kv_mode="int8" if int8 else "fp16", legacy_prefill=legacy)
    _upload_planes(ctx, planes)
    for pb, M in ((300, 70), (0, 1), (0, 15), (0, 16), (0, 17), (0, 70), (353, 17), (0, 370)):
        sub = orc.KvPlanes(512, int8=int8, poison=not int8)
        n = pb + M
        sub.k[:n], sub.v[:n] = planes.k[:n], planes.v[:n]
        if int8:
            sub.ksc[:n], sub.vsc[:n] = planes.ksc[:n], planes.vsc[:n]
        out = ctx.prefill(0, [0], [pb], M, _dev(orc.cvt_q_half(q[pb:n])[None]).view(torch.float16), _dev(gate[pb:n][None]))
        ctx.check()
        got = out.cpu().numpy()[0]
        _close(got, orc.formula_f32(q[pb:n], gate[pb:n], sub, pb))
        assert np.abs(got - orc.flash_prefill(orc.cvt_q_half(q[pb:n]), gate[pb:n], sub, pb)).max() < 3e-4


def test_prefill_long_tcgen05_vs_oracle_and_mma(capi, orc):
    # several 128-row query tiles over many 128-key tiles (running-maximum rescales, diagonal and tail tiles), two sequences
    pb, M = 700, 600
    ctx = capi.AttnContext(1, [2048, 2048])
    leg = capi.AttnContext(1, [2048, 2048], legacy_prefill=True)
    q16s, gates, refs = [], [], []
    for s, scale in enumerate((1.0, 3.0)):   # the second sequence has sharper scores: more maximum updates
        planes, q, gate, _ = _oracle_fill(orc, 70 + s, pb + M, 2048, poison=True, fast=True, seq=s)
        q = (q * scale).astype(np.float32)
        _upload_planes(ctx, planes, seq=s); _upload_planes(leg, planes, seq=s)
        q16s.append(orc.cvt_q_half(q[pb:])); gates.append(gate[pb:])
        refs.append(orc.formula_f32(q[pb:], gate[pb:], planes, pb))
    dq, dg = _dev(np.stack(q16s)).view(torch.float16), _dev(np.stack(gates))
    out = ctx.prefill(0, [0, 1], [pb, pb], M, dq, dg)
    ref2 = leg.prefill(0, [0, 1], [pb, pb], M, dq, dg)
    ctx.check(); leg.check()
    for s in range(2):
        _close(out.cpu().numpy()[s], refs[s])
        assert np.abs(out.cpu().numpy()[s] - ref2.cpu().numpy()[s]).max() < TOL_MAX   # the two kernels round P against different running maxima


def test_chunked_prefill_restore_equals_one_shot(capi, orc):
    # prefill 0..150, export the planes, reset, import them (the prefix-cache restore), continue in chunks, compare with one shot
    n, cut = 420, 150
    qn, kn = synth.norm_weights(62)
    qf, kp, vp = synth.token_rows_fast(62, n)
    dq, dk, dv, dqn, dkn = _dev(qf), _dev(kp), _dev(vp), _dev(qn), _dev(kn)
    one = capi.AttnContext(1, [512])
    q16, _, g = one.prep(0, [0], [0], n, dq[None], dk[None], dv[None], dqn, dkn)
    o1 = one.prefill(0, [0], [0], n, q16, g).cpu().numpy()[0]
    ch = capi.AttnContext(1, [512])
    q16a, _, ga = ch.prep(0, [0], [0], cut, dq[None, :cut].contiguous(), dk[None, :cut].contiguous(), dv[None, :cut].contiguous(), dqn, dkn)
    oa = ch.prefill(0, [0], [0], cut, q16a, ga).cpu().numpy()[0]
    saved = [ch.plane_read(0, 0, p, 0, cut) for p in range(ch.kv_planes())]
    ch.reset()
    assert (ch.plane_read(0, 0, 0, 0, 512) == 0).all()
    for p, data in enumerate(saved):
        ch.plane_write(0, 0, p, 0, data)
    outs = [oa]
    for start, m in ((150, 128), (278, 100), (378, 42)):
        sl = slice(start, start + m)
        q16c, _, gc = ch.prep(0, [0], [start], m, dq[None, sl].contiguous(), dk[None, sl].contiguous(), dv[None, sl].contiguous(), dqn, dkn)
        outs.append(ch.prefill(0, [0], [start], m, q16c, gc).cpu().numpy()[0])
    ch.check(); one.check()
    for p in range(2):
        assert np.array_equal(ch.plane_read(0, 0, p, 0, n), one.plane_read(0, 0, p, 0, n))
    assert np.abs(np.concatenate(outs) - o1).max() < 2e-4
    # and the T=2 verify that follows a chunked prefill
    v = ch.decode(0, [0], [n - 2], 2, q16[:, n - 2:].contiguous(), g[:, n - 2:].contiguous()).cpu().numpy()[0]
    assert np.abs(v - o1[n - 2:]).max() < 3e-4


def test_prefill_batch_bf16_out(capi, orc):
    M = 96
    ctx = capi.AttnContext(2, [128, 256])
    refs, q16s, gates = [], [], []
    for s, pb in enumerate((0, 100)):
        planes, q, gate, _ = _oracle_fill(orc, 63 + s, pb + M, int(ctx.max_ctx[s]), fast=True, seq=s)
        _upload_planes(ctx, planes, layer=1, seq=s)
        refs.append(orc.formula_f32(q[pb:], gate[pb:], planes, pb))
        q16s.append(orc.cvt_q_half(q[pb:]))
        gates.append(gate[pb:])
    out = ctx.prefill(1, [0, 1], [0, 100], M, _dev(np.stack(q16s)).view(torch.float16), _dev(np.stack(gates)), out_dtype=torch.bfloat16)
    ctx.check()
    got = out.float().cpu().numpy()
    for s in range(2):
        d = np.abs(got[s] - refs[s])
        assert (d <= TOL_MAX + np.abs(refs[s]) * 2.0 ** -8).all() and d.mean() < 2 * TOL_MEAN   # one bf16 rounding on top of the tolerance


# ------------------------------------------------------------------------------------------------ errors
def test_errors_are_codes_not_faults(capi):
    ctx = capi.AttnContext(2, [64, 32])
    z16 = torch.zeros((1, 1, 6144), dtype=torch.float16, device="cuda")
    z32 = torch.zeros((1, 1, 6144), dtype=torch.float32, device="cuda")
    for fn, code in (
        (lambda: ctx.decode(2, [0], [0], 1, z16, z32), 2),          # layer out of range
        (lambda: ctx.decode(0, [2], [0], 1, z16, z32), 2),          # sequence out of range
        (lambda: ctx.decode(0, [1], [32], 1, z16, z32), 2),         # position beyond max_ctx
        (lambda: ctx.decode(0, [0], [5], 9, z16, z32), 2),          # T > 8
        (lambda: ctx.decode(0, [0], [5], 1, z16, z32, first_pos=6), 2),
        (lambda: ctx.prefill(0, [0], [0], 2000, z16, z32), 2),      # chunk too long
        (lambda: ctx.kv_quant(0, 0, z16, z16, 0), 3),               # fp16 context has no quantiser
        (lambda: ctx.plane_read(0, 0, 2, 0, 1), 1),                 # no scale planes in fp16 mode
    ):
        with pytest.raises(capi.KataError) as e:
            fn()
        assert e.value.code == code
    ctx.check()
    assert ctx.tag() == "fp16" and ctx.kv_planes() == 2 and ctx.plane_row_bytes(0) == 2048


# ------------------------------------------------------------------------------------------------ benchmark sizes
def test_full_size_decode_32k_properties(capi, orc):
    # one layer at the benchmark's context length: against the fp32 formula, and the size-independent properties the
    # reference relies on (matrix path == scalar path, T=2 verify == two T=1 decodes, result independent of the split)
    L = 32768
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    # split sizes: from the SM count (0), 2048 keys, and the reference's own 128 keys (src/engine.cpp:120: 256 splits per KV head here) and 256
    ctxs = [capi.AttnContext(1, [L + 8], dec_chunk=c) for c in (0, 2048, 128, 256)]
    for st in range(0, L, 1024):
        kp = torch.randn(1, 1024, 1024, generator=gen, device="cuda"); vp = torch.randn(1, 1024, 1024, generator=gen, device="cuda")
        for c in ctxs:
            c.prep(0, [0], [st], 1024, None, kp, vp, None, kn, h0=24, nh=8)
    qf = torch.randn(1, 2, 12288, generator=gen, device="cuda"); kp = torch.randn(1, 2, 1024, generator=gen, device="cuda"); vp = torch.randn(1, 2, 1024, generator=gen, device="cuda")
    outs, outs1 = [], []
    for c in ctxs:
        q16, q32, g = c.prep(0, [0], [L - 2], 2, qf, kp, vp, qn, kn, want_q32=True)
        outs.append(c.decode(0, [0], [L - 2], 2, q16, g))
        outs1.append(c.decode(0, [0], [L - 1], 1, q16[:, 1:].contiguous(), g[:, 1:].contiguous()))
        c.check()
    c = ctxs[0]
    sc = c.decode_scalar(0, [0], [L - 2], 2, q32, g)
    d0 = c.decode(0, [0], [L - 2], 1, q16[:, :1].contiguous(), g[:, :1].contiguous()); d1 = c.decode(0, [0], [L - 1], 1, q16[:, 1:].contiguous(), g[:, 1:].contiguous())
    c.check()
    a = outs[0].cpu().numpy()[0]
    for o, o1 in zip(outs[1:], outs1[1:]):                                          # split invariance, T = 2 and T = 1
        assert np.abs(a - o.cpu().numpy()[0]).max() < 2e-5 and np.abs(a[1] - o1.cpu().numpy()[0, 0]).max() < 2e-5
    assert np.abs(a[0] - d0.cpu().numpy()[0, 0]).max() < 2e-5 and np.abs(a[1] - d1.cpu().numpy()[0, 0]).max() < 2e-5
    _close(a, sc.cpu().numpy()[0])                                                  # matrix path vs scalar path
    planes = orc.KvPlanes(L)
    planes.k[:] = c.plane_read(0, 0, 0, 0, L).view(np.uint16).reshape(L, 1024); planes.v[:] = c.plane_read(0, 0, 1, 0, L).view(np.uint16).reshape(L, 1024)
    ref = orc.formula_f32(q32.cpu().numpy()[0], g.cpu().numpy()[0], planes, L - 2)
    for o in outs:
        _close(o.cpu().numpy()[0], ref)


@pytest.mark.parametrize("mode", ["int8", "int8v"])
def test_full_size_quantised_decode_32k_properties(capi, orc, mode):
    # the int8 caches at the benchmark's context length: against the fp32 formula on the dequantised planes, T=2 verify == two T=1
    # decodes, result independent of the split, and the value codes / scales equal to the quantiser applied to the fp16 cache's rows
    L = 32768
    gen = torch.Generator(device="cuda"); gen.manual_seed(8)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    ctxs = [capi.AttnContext(1, [L + 8], kv_mode=mode, dec_chunk=c) for c in (0, 2048, 128, 256)]   # 128: the reference's split size (src/engine.cpp:120)
    c16 = capi.AttnContext(1, [L + 8])
    for st in range(0, L, 1024):
        kp = torch.randn(1, 1024, 1024, generator=gen, device="cuda"); vp = torch.randn(1, 1024, 1024, generator=gen, device="cuda")
        for c in ctxs + [c16]:
            c.prep(0, [0], [st], 1024, None, kp, vp, None, kn, h0=24, nh=8)
    qf = torch.randn(1, 2, 12288, generator=gen, device="cuda"); kp = torch.randn(1, 2, 1024, generator=gen, device="cuda"); vp = torch.randn(1, 2, 1024, generator=gen, device="cuda")
    outs, outs1 = [], []
    for c in ctxs:
        q16, q32, g = c.prep(0, [0], [L - 2], 2, qf, kp, vp, qn, kn, want_q32=True)
        outs.append(c.decode(0, [0], [L - 2], 2, q16, g))
        outs1.append(c.decode(0, [0], [L - 1], 1, q16[:, 1:].contiguous(), g[:, 1:].contiguous()))
        c.check()
    c16.prep(0, [0], [L - 2], 2, qf, kp, vp, qn, kn); c16.check()
    c = ctxs[0]
    d0 = c.decode(0, [0], [L - 2], 1, q16[:, :1].contiguous(), g[:, :1].contiguous()); d1 = c.decode(0, [0], [L - 1], 1, q16[:, 1:].contiguous(), g[:, 1:].contiguous())
    c.check()
    a = outs[0].cpu().numpy()[0]
    # looser than the fp16 cache's 2e-5: the int8 fragments enter the MMAs as code + 1152 and the bias comes out of the fp32 accumulators
    # afterwards, so accumulation-order noise is that of sums some hundred times larger than the result
    for o, o1 in zip(outs[1:], outs1[1:]):                                          # split invariance, T = 2 and T = 1
        assert np.abs(a - o.cpu().numpy()[0]).max() < 1e-4 and np.abs(a[1] - o1.cpu().numpy()[0, 0]).max() < 1e-4
    assert np.abs(a[0] - d0.cpu().numpy()[0, 0]).max() < 1e-4 and np.abs(a[1] - d1.cpu().numpy()[0, 0]).max() < 1e-4
    planes = orc.KvPlanes(L, int8=(mode == "int8"), int8v=(mode == "int8v"))
    planes.k[:] = c.plane_read(0, 0, 0, 0, L).view(planes.k.dtype).reshape(L, 1024); planes.v[:] = c.plane_read(0, 0, 1, 0, L).view(np.int8).reshape(L, 1024)
    if mode == "int8":
        planes.ksc[:] = c.plane_read(0, 0, 2, 0, L).view(np.uint16).reshape(L, 4)
    planes.vsc[:] = c.plane_read(0, 0, c.kv_planes() - 1, 0, L).view(np.uint16).reshape(L, 4)
    ref_f = orc.formula_f32(q32.cpu().numpy()[0], g.cpu().numpy()[0], planes, L - 2)
    for o in outs:
        _close(o.cpu().numpy()[0], ref_f)
    # quantise-on-append == the reference quantiser over the rows the fp16 path caches (bit for bit, all 32K rows)
    ref = orc.KvPlanes(L, int8=True)
    orc.kv_quant(np.ascontiguousarray(c16.plane_read(0, 0, 0, 0, L).view(np.uint16).reshape(L, 1024)), np.ascontiguousarray(c16.plane_read(0, 0, 1, 0, L).view(np.uint16).reshape(L, 1024)), ref, 0, 0)
    assert np.array_equal(planes.v, ref.v) and np.array_equal(planes.vsc, ref.vsc)
    if mode == "int8":
        assert np.array_equal(planes.k, ref.k) and np.array_equal(planes.ksc, ref.ksc)
    else:
        assert np.array_equal(planes.k, c16.plane_read(0, 0, 0, 0, L).view(np.uint16).reshape(L, 1024))


def test_full_size_prefill_chunk_over_7k_prefix(capi, orc):
    # the last full chunk of the 7,300-token prompt: 512 rows at position 6,672, tcgen05 kernel vs the fp32 formula (sampled rows)
    pb, M = 6672, 512
    gen = torch.Generator(device="cuda"); gen.manual_seed(6)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    ctx = capi.AttnContext(1, [pb + M])
    for st in range(0, pb, 1024):
        m = min(1024, pb - st)
        ctx.prep(0, [0], [st], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    qf = torch.randn(1, M, 12288, generator=gen, device="cuda").to(torch.bfloat16); kp = torch.randn(1, M, 1024, generator=gen, device="cuda").to(torch.bfloat16); vp = torch.randn(1, M, 1024, generator=gen, device="cuda").to(torch.bfloat16)
    q16, q32, g = ctx.prep(0, [0], [pb], M, qf, kp, vp, qn, kn, want_q32=True)
    out = ctx.prefill(0, [0], [pb], M, q16, g).cpu().numpy()[0]
    ctx.check()
    planes = orc.KvPlanes(pb + M)
    planes.k[:] = ctx.plane_read(0, 0, 0, 0, pb + M).view(np.uint16).reshape(-1, 1024); planes.v[:] = ctx.plane_read(0, 0, 1, 0, pb + M).view(np.uint16).reshape(-1, 1024)
    rows = [0, 1, 127, 128, 300, 511]
    for r in rows:
        ref = orc.formula_f32(q32.cpu().numpy()[0, r:r + 1], g.cpu().numpy()[0, r:r + 1], planes, pb + r)
        _close(out[r:r + 1], ref)


def _prefill_both_kernels(capi, positions, M, seed):
    """Rows of a batch at the given positions through the tcgen05 kernel and through the mma.sync kernel of a second context holding the same caches."""
    gen = torch.Generator(device="cuda"); gen.manual_seed(seed)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    n = len(positions); ctxs = [capi.AttnContext(1, [p + M for p in positions]), capi.AttnContext(1, [p + M for p in positions], legacy_prefill=True)]
    seqs = list(range(n)); outs = []
    top = max(positions)
    pre_k = torch.randn(n, max(top, 1), 1024, generator=gen, device="cuda"); pre_v = torch.randn(n, max(top, 1), 1024, generator=gen, device="cuda")
    qf = torch.randn(n, M, 12288, generator=gen, device="cuda"); kp = torch.randn(n, M, 1024, generator=gen, device="cuda"); vp = torch.randn(n, M, 1024, generator=gen, device="cuda")
    for ctx in ctxs:
        for s, pb in enumerate(positions):
            for st in range(0, pb, 1024):
                m = min(1024, pb - st)
                ctx.prep(0, [s], [st], m, None, pre_k[s:s + 1, st:st + m].contiguous(), pre_v[s:s + 1, st:st + m].contiguous(), None, kn, h0=24, nh=8)
        q16, _, g = ctx.prep(0, seqs, list(positions), M, qf, kp, vp, qn, kn)
        outs.append((ctx, q16, g, ctx.prefill(0, seqs, list(positions), M, q16, g)))
        ctx.check()
    return outs


@pytest.mark.gpu
@pytest.mark.parametrize("positions,M", [((900,) * 8, 256), ((40, 3000, 700, 12, 1500), 200), ((2500,), 128), ((5000, 5000), 512)],
                         ids=["rounds-then-ranges", "ragged-batch", "one-query-tile-cut-many-ways", "two-long-sequences"])
def test_prefill_work_split_variants(capi, orc, positions, M):
    # whole items in rounds plus a cut last round (equal sequences), equal ranges of the whole list (a ragged batch), items cut into many parts
    # (one sequence, one query tile, 74 pairs): whatever the split, the rows equal the mma.sync kernel's within the tolerance, and a second
    # launch (the flags of the cut items' parts have gone down again) gives the same bits as the first
    (ctx, q16, g, out), (_, _, _, ref) = _prefill_both_kernels(capi, positions, M, 71)
    a, b = out.cpu().numpy(), ref.cpu().numpy()
    assert np.isfinite(a).all()
    assert np.abs(a - b).max() < TOL_MAX and np.abs(a - b).mean() < TOL_MEAN
    again = ctx.prefill(0, list(range(len(positions))), list(positions), M, q16, g); ctx.check()
    assert torch.equal(again, out)


@pytest.mark.gpu
def test_prefill_cut_items_in_a_replayed_cuda_graph(capi, orc):
    # one sequence: 48 items for 74 pairs, every item cut; the launch is captured once and replayed: each replay must find the part flags down
    (ctx, q16, g, out), _ = _prefill_both_kernels(capi, (3000,), 512, 72)
    st = torch.cuda.Stream()
    buf = torch.empty_like(out)
    with torch.cuda.stream(st):
        ctx.prefill(0, [0], [3000], 512, q16, g, out=buf)   # warm-up on the capture stream
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            ctx.prefill(0, [0], [3000], 512, q16, g, out=buf)
        for _ in range(3):
            buf.zero_()
            graph.replay()
            st.synchronize()
            assert torch.equal(buf, out)
    ctx.check()


@pytest.mark.gpu
def test_out_fwht_bit_exact(capi, orc):
    # the transform between attention and the output projection (k_rms_fwht mode 3): same butterflies in the same order -> same bits
    rng = np.random.default_rng(11)
    sign = np.where(rng.random(6144) < 0.5, -1.0, 1.0).astype(np.float32)
    for rows, width in ((1, 6144), (7, 6144), (300, 6144), (5, 1024)):
        x = (rng.standard_normal((rows, width)) * rng.choice([1e-3, 1.0, 50.0], size=(rows, 1))).astype(np.float32)
        got = capi.out_fwht(_dev(x), _dev(sign[:width])).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), orc.out_fwht(x, sign[:width]).view(np.uint32))
    d = _dev(x.copy())
    capi.out_fwht(d, _dev(sign[:1024]), out=d)   # in place
    assert np.array_equal(d.cpu().numpy().view(np.uint32), orc.out_fwht(x, sign[:1024]).view(np.uint32))
    with pytest.raises(capi.KataError):
        capi.out_fwht(torch.zeros(2, 1000, device="cuda"), _dev(sign[:1000]))


@pytest.mark.parametrize("mode", ["fp16", "int8", "int8v"])
def test_decode_right_after_append_matches_a_synchronised_run(capi, orc, mode):
    # Long enough ranges per CTA (4 sequences x ~24K keys) for the decode kernel to request tiles before it has waited for the append that
    # precedes it on the stream. The step append -> decode must give what append, synchronise, decode gives, also for the newest key, for
    # T = 1 and T = 2, and the same as a context whose work split is fixed (no early requests there: ranges are short).
    lens = [24001, 23057, 24576, 20000]
    gen = torch.Generator(device="cuda"); gen.manual_seed(17)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    ctxs = [capi.AttnContext(1, [l + 16 for l in lens], kv_mode=mode, dec_chunk=c) for c in (0, 1024)]
    for s, l in enumerate(lens):
        for st in range(0, l, 1024):
            m = min(1024, l - st)
            kp = torch.randn(1, m, 1024, generator=gen, device="cuda"); vp = torch.randn(1, m, 1024, generator=gen, device="cuda")
            for c in ctxs:
                c.prep(0, [s], [st], m, None, kp, vp, None, kn, h0=24, nh=8)
    seqs = [0, 1, 2, 3]
    pos = list(lens)
    for T in (1, 2, 1):
        qf = torch.randn(4, T, 12288, generator=gen, device="cuda"); kp = torch.randn(4, T, 1024, generator=gen, device="cuda"); vp = torch.randn(4, T, 1024, generator=gen, device="cuda")
        outs = []
        for c, sync in ((ctxs[0], False), (ctxs[1], True)):
            q16, _, g = c.prep(0, seqs, pos, T, qf, kp, vp, qn, kn)
            if sync:
                torch.cuda.synchronize()
            outs.append(c.decode(0, seqs, pos, T, q16, g))
            c.check()
        a, b = outs[0].cpu().numpy(), outs[1].cpu().numpy()
        assert np.isfinite(a).all() and np.abs(a - b).max() < 1e-4
        # a decode that missed the newest key differs by more than the agreement asked for above (one key in 24K still shows): drop it and compare
        q16, _, g = ctxs[1].prep(0, seqs, pos, T, qf, kp, vp, qn, kn)
        miss = ctxs[1].decode(0, seqs, [p - 1 for p in pos], 1, q16[:, :1].contiguous(), g[:, :1].contiguous()).cpu().numpy()
        assert np.abs(miss[:, 0] - a[:, 0]).max() > 3e-4
        pos = [p + T for p in pos]


def test_append_and_decode_replay_in_a_cuda_graph(capi, orc):
    # the calls only enqueue work (no allocation, no synchronisation, metadata by value): a captured step replays with the same result
    lens = [5000, 3000]
    ctx = capi.AttnContext(2, [l + 8 for l in lens])
    gen = torch.Generator(device="cuda"); gen.manual_seed(3)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    for layer in range(2):
        for s, l in enumerate(lens):
            for st in range(0, l, 1024):
                m = min(1024, l - st)
                ctx.prep(layer, [s], [st], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    qf = torch.randn(2, 2, 1, 12288, generator=gen, device="cuda"); kp = torch.randn(2, 2, 1, 1024, generator=gen, device="cuda"); vp = torch.randn(2, 2, 1, 1024, generator=gen, device="cuda")
    q16 = torch.empty(2, 2, 1, 6144, dtype=torch.float16, device="cuda"); gate = torch.empty(2, 2, 1, 6144, device="cuda"); out = torch.empty(2, 2, 1, 6144, device="cuda")

    def step():
        for layer in range(2):
            ctx.prep(layer, [0, 1], lens, 1, qf[layer], kp[layer], vp[layer], qn, kn, q16=q16[layer], gate=gate[layer])
            ctx.decode(layer, [0, 1], lens, 1, q16[layer], gate[layer], out=out[layer])
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side); torch.cuda.synchronize()
    ctx.check()
    eager = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(2):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    ctx.check()


def test_partial_decode_right_after_append_on_another_sequence(capi, orc):
    # The split-KV step of a rank: append the new row, then at once the partial decode of the same sequence (not sequence 0), with ranges
    # long enough (one CTA per 4096 keys) for the kernel to request tiles before it has waited for the append. The merged part must
    # contain the newest key: equal to the plain decode of the same rows, and to the fp32 formula.
    lens = [40, 9000]
    ctx = capi.AttnContext(1, [64, 9100], dec_chunk=4096)
    gen = torch.Generator(device="cuda"); gen.manual_seed(23)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    for s, l in enumerate(lens):
        for st in range(0, l, 1024):
            m = min(1024, l - st)
            ctx.prep(0, [s], [st], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    pos = lens[1]
    for T in (1, 2):
        qf = torch.randn(1, T, 12288, generator=gen, device="cuda"); kp = 3.0 * torch.randn(1, T, 1024, generator=gen, device="cuda"); vp = 3.0 * torch.randn(1, T, 1024, generator=gen, device="cuda")
        torch.cuda.synchronize()
        q16, q32, g = ctx.prep(0, [1], [pos], T, qf, kp, vp, qn, kn, want_q32=True)
        part = ctx.decode_partial(0, 1, pos, T, 0, 1 << 30, q16)
        got = ctx.merge_parts(part[None], T, g[0]).cpu().numpy()
        ctx.check()
        want = ctx.decode(0, [1], [pos], T, q16, g).cpu().numpy()[0]
        assert np.abs(got - want).max() < 1e-5
        planes = orc.KvPlanes(pos + T)
        planes.k[:] = ctx.plane_read(0, 1, 0, 0, pos + T).view(np.uint16).reshape(-1, 1024); planes.v[:] = ctx.plane_read(0, 1, 1, 0, pos + T).view(np.uint16).reshape(-1, 1024)
        _close(got, orc.formula_f32(q32.cpu().numpy()[0], g.cpu().numpy()[0], planes, pos))
        pos += T


@pytest.mark.parametrize("declare", [False, True], ids=["undeclared", "declared"])
def test_decode_right_after_rows_written_through_the_plane_pointer(capi, orc, declare):
    # A device-side restore (the counterpart of the reference's plane-wise restore, src/ckpt.cpp:98): a caller's copy kernel writes every
    # row of a sequence through kata_attn_kv_plane_ptr and the decode follows on the same stream without a synchronisation. Without a
    # declaration the library stops requesting rows early; with kata_attn_mark_rows_written it holds back the declared rows. Either way
    # the result must equal that of the context the rows came from.
    lens = [24001, 23057, 24576, 20000]
    gen = torch.Generator(device="cuda"); gen.manual_seed(29)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    src = capi.AttnContext(1, [l + 16 for l in lens]); dst = capi.AttnContext(1, [l + 16 for l in lens])
    for s, l in enumerate(lens):
        for st in range(0, l, 1024):
            m = min(1024, l - st)
            src.prep(0, [s], [st], m, None, torch.randn(1, m, 1024, generator=gen, device="cuda"), torch.randn(1, m, 1024, generator=gen, device="cuda"), None, kn, h0=24, nh=8)
    seqs = [0, 1, 2, 3]; pos = [l - 1 for l in lens]
    qf = torch.randn(4, 1, 12288, generator=gen, device="cuda")
    q16, _, g = src.prep(0, seqs, pos, 1, qf, None, None, qn, None, h0=0, nh=24)
    want = src.decode(0, seqs, pos, 1, q16, g)
    src.check()
    views = [(src.plane_tensor(0, s, pl, lens[s]), dst.plane_tensor(0, s, pl, lens[s])) for s in seqs for pl in (0, 1)]
    for rep in range(3):
        dst.reset()
        torch.cuda.synchronize()
        for a, b in views:
            b.copy_(a)                      # the caller's kernels: 375 MB of rows, still in flight when the decode is enqueued
        if declare:
            dst.mark_rows_written(-1, 0)
        got = dst.decode(0, seqs, pos, 1, q16, g)
        dst.check()
        assert torch.equal(got, want)


@pytest.mark.parametrize("path", ["prefill-tcgen05", "prefill-mma", "decode-T2"])
def test_references_own_check_judges_the_cuda_kernels(capi, path):
    # The reference's CPU check compiled from its own lines (tools/probe_flash.cpp:16-19, 26-34; oracle/_ref): its generator makes K, V, Q
    # and the gate, the cache beyond the 370 valid keys is NaN, and its fp64 loop judges what the CUDA kernel wrote for the 70 rows at
    # position 300. The reference reports 6.6e-5 for its own Metal kernel on this procedure.
    from oracle import probe_ref
    if probe_ref.build() is None:
        pytest.skip("no prebuilt oracle/_ref/libprobe_ref.so on this machine")

    def kernel(q16, k, v, g, pb, m):
        rows = 512                                                   # 370 valid rows, NaN rows behind them
        ctx = capi.AttnContext(1, [rows], legacy_prefill=(path == "prefill-mma"))
        ctx.plane_write(0, 0, 0, 0, k[:rows]); ctx.plane_write(0, 0, 1, 0, v[:rows])
        dq = _dev(q16[:m]).view(torch.float16).reshape(1, m, 6144); dg = _dev(g[:m]).reshape(1, m, 6144)
        if path.startswith("prefill"):
            out = ctx.prefill(0, [0], [pb], m, dq, dg)
        else:
            out = torch.cat([ctx.decode(0, [0], [pb + t], 2, dq[:, t:t + 2].contiguous(), dg[:, t:t + 2].contiguous()) for t in range(0, m, 2)], dim=1)
        ctx.check()
        res = out.cpu().numpy()[0]
        ctx.close()
        return res

    res = probe_ref.run(kernel)
    assert res.non_finite == 0 and res.worst < 2e-4, res.worst


def test_fp32_decode_path_ragged_batch_first_pos_and_token_groups(capi, orc):
    # the CUDA-core path on a ragged batch: lengths around the 32-key tile and the 128-key chunk, T across the 4-token groups, first_pos = 1
    lens = [1, 31, 33, 130, 700, 4500]
    ctx = capi.AttnContext(1, [l + 16 for l in lens])
    planes, qs, gs = [], [], []
    for s, L in enumerate(lens):
        pl, q, g, _ = _oracle_fill(orc, 300 + s, L + 8, L + 16, fast=True, seq=s)
        _upload_planes(ctx, pl, seq=s); planes.append(pl); qs.append(q); gs.append(g)
    seqs = list(range(len(lens)))
    for T, first_pos in ((1, 0), (3, 0), (5, 1), (8, 0)):
        pos = [max(L - 1, first_pos) for L in lens]   # rows up to pos + T - 1 exist (8 spare rows were filled)
        dq = _dev(np.stack([qs[s][pos[s]:pos[s] + T] for s in seqs])); dg = _dev(np.stack([gs[s][pos[s]:pos[s] + T] for s in seqs]))
        out = ctx.decode_scalar(0, seqs, pos, T, dq, dg, first_pos=first_pos).cpu().numpy()
        ctx.check()
        for s in seqs:
            ref = orc.formula_f32(qs[s][pos[s]:pos[s] + T], gs[s][pos[s]:pos[s] + T], planes[s], pos[s], first_pos=first_pos)
            assert np.isfinite(out[s]).all() and np.abs(out[s] - ref).max() < 2e-5, (T, first_pos, s)


@pytest.mark.parametrize("mode", ["fp16", "int8"])
def test_kv_head_shards_equal_the_whole_context(capi, orc, mode):
    # Sharding by KV-head group: two contexts, each owning two KV heads (as two ranks would, here on one GPU), against one context that owns
    # all four, on the same inputs: append, T = 2 decode of a ragged batch, and a prefill chunk over a prefix. Each shard must write
    # exactly its own 12 query heads' columns (the rest untouched), equal to the whole context's; with a split that cuts every head's keys
    # at the same places (dec_chunk dividing the head's tiles) the decode is bit-identical.
    from kata_b200 import multi
    lens = [1024, 2560]
    gen = torch.Generator(device="cuda"); gen.manual_seed(31)
    kn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous(); qn = (1 + 0.05 * torch.randn(256, generator=gen, device="cuda")).contiguous()
    whole = capi.AttnContext(1, [l + 600 for l in lens], kv_mode=mode, dec_chunk=256)
    shards = []
    for lo, n in multi.shard_kv_heads(2):
        c = capi.AttnContext(1, [l + 600 for l in lens], kv_mode=mode, dec_chunk=256); c.set_kv_heads(lo, n); shards.append((c, lo, n))
    for s, l in enumerate(lens):
        for st in range(0, l, 512):
            kp = torch.randn(1, 512, 1024, generator=gen, device="cuda"); vp = torch.randn(1, 512, 1024, generator=gen, device="cuda")
            for c in [whole] + [x[0] for x in shards]:
                c.prep(0, [s], [st], 512, None, kp, vp, None, kn, h0=24, nh=8)
    # a shard's planes hold its own heads' columns and zeros elsewhere
    for c, lo, n in shards:
        for pl in (0, 1):
            a = whole.plane_read(0, 1, pl, 0, 64).reshape(64, 4, -1); b_ = c.plane_read(0, 1, pl, 0, 64).reshape(64, 4, -1)
            assert np.array_equal(a[:, lo:lo + n], b_[:, lo:lo + n]) and not np.delete(b_, np.s_[lo:lo + n], axis=1).any()
    SENT = 777.0
    # decode, T = 2, over the last two rows (rewritten by the prep of the same call): 1024 and 2560 keys are whole multiples of the 256-key
    # split, so every head's keys are cut at the same places whether a launch holds two heads or four
    dpos = [l - 2 for l in lens]
    qf = torch.randn(2, 2, 12288, generator=gen, device="cuda"); kp = torch.randn(2, 2, 1024, generator=gen, device="cuda"); vp = torch.randn(2, 2, 1024, generator=gen, device="cuda")
    q16, _, g = whole.prep(0, [0, 1], dpos, 2, qf, kp, vp, qn, kn)
    want = whole.decode(0, [0, 1], dpos, 2, q16, g); whole.check()
    for c, lo, n in shards:
        cols = multi.head_columns(lo, n)
        q16s = torch.full_like(q16, SENT); gs = torch.full_like(g, SENT)
        c.prep(0, [0, 1], dpos, 2, qf, kp, vp, qn, kn, q16=q16s, gate=gs)
        assert torch.equal(q16s[..., cols], q16[..., cols]) and torch.equal(gs[..., cols], g[..., cols])
        rest = torch.ones(6144, dtype=torch.bool, device="cuda"); rest[cols] = False
        assert (q16s[..., rest] == SENT).all() and (gs[..., rest] == SENT).all()
        out = torch.full_like(want, SENT)
        c.decode(0, [0, 1], dpos, 2, q16s, gs, out=out); c.check()
        assert torch.equal(out[..., cols], want[..., cols]) and (out[..., rest] == SENT).all()
    # prefill of a 300-row chunk behind the decoded rows (sequence 1 only), tcgen05 kernel
    M, p0 = 300, lens[1]
    qf = torch.randn(1, M, 12288, generator=gen, device="cuda"); kp = torch.randn(1, M, 1024, generator=gen, device="cuda"); vp = torch.randn(1, M, 1024, generator=gen, device="cuda")
    q16, _, g = whole.prep(0, [1], [p0], M, qf, kp, vp, qn, kn)
    want = whole.prefill(0, [1], [p0], M, q16, g); whole.check()
    for c, lo, n in shards:
        cols = multi.head_columns(lo, n)
        q16s, _, gs = c.prep(0, [1], [p0], M, qf, kp, vp, qn, kn)
        out = torch.full_like(want, SENT)
        c.prefill(0, [1], [p0], M, q16s, gs, out=out); c.check()
        rest = torch.ones(6144, dtype=torch.bool, device="cuda"); rest[cols] = False
        # (a shard's items are cut between CTA pairs at other places than the whole context's: P is rounded to fp16 against other running maxima)
        assert (out[..., cols] - want[..., cols]).abs().max().item() < 3e-4 and (out[..., rest] == SENT).all()
        # what a shard cannot do says so
        with pytest.raises(capi.KataError) as e:
            c.decode_scalar(0, [1], [p0], 1, torch.zeros(1, 1, 6144, device="cuda"), torch.zeros(1, 1, 6144, device="cuda"))
        assert e.value.code == 3


# ------------------------------------------------------------------------------------------------ int8g: int8 keys with one scale per 64 dims
def test_int8g_planes_quantiser_and_append(capi, orc):
    # planes {K int8, V int8, K scales [head][group] (32 B), V scales (8 B)}, tag, and the quantiser: stand-alone on arbitrary fp16 rows bit for
    # bit (codes and all four group scales per head; edge rows: zero groups, ties, clamp), and fused into the append against the oracle
    ctx = capi.AttnContext(1, [128], kv_mode="int8g")
    assert ctx.tag() == "fp16+kv8g" and ctx.kv_planes() == 4 and [ctx.plane_row_bytes(i) for i in range(4)] == [1024, 1024, 32, 8]
    rng = np.random.default_rng(61)
    ks = (rng.standard_normal((20, 1024)) * rng.choice([1e-4, 1.0, 30.0], size=(20, 16)).repeat(64, axis=1)).astype(np.float16)
    ks[3, 64:128] = 0; ks[4, :64] = np.float16(0.5) * np.arange(-32, 32).astype(np.float16); ks[5] = 0
    vs = rng.standard_normal((20, 1024)).astype(np.float16)
    ctx.kv_quant(0, 0, _dev(ks), _dev(vs), 7); ctx.check()
    want = orc.KvPlanes(64, int8g=True)
    orc.kv_quant(ks.view(np.uint16), vs.view(np.uint16), want, 7, 3)
    got = [ctx.plane_read(0, 0, i, 7, 20) for i in range(4)]
    assert np.array_equal(got[0].view(np.int8).reshape(20, 1024), want.k[7:27]) and np.array_equal(got[1].view(np.int8).reshape(20, 1024), want.v[7:27])
    assert np.array_equal(got[2].view(np.uint16).reshape(20, 16), want.ksc[7:27]) and np.array_equal(got[3].view(np.uint16).reshape(20, 4), want.vsc[7:27])
    codes, sc = orc.kv_quant_rows_np(ks.reshape(20, 16, 64))   # the independent numpy quantiser, group by group
    assert np.array_equal(codes.reshape(20, 1024), want.k[7:27]) and np.array_equal(sc.view(np.uint16), want.ksc[7:27])
    # quantise-on-append: V bit-exact; K groups equal except where sin/cos of the rotation differ by an ulp from the host's
    L = 90
    planes, q, gate, (qf, kp, vp, qn, kn) = _oracle_fill(orc, 62, L, 128, int8g=True)
    c2 = capi.AttnContext(1, [128], kv_mode="int8g")
    c2.prep(0, [0], [0], L, _dev(qf[None]), _dev(kp[None]), _dev(vp[None]), _dev(qn), _dev(kn)); c2.check()
    assert np.array_equal(c2.plane_read(0, 0, 1, 0, L).view(np.int8).reshape(L, 1024), planes.v[:L]) and np.array_equal(c2.plane_read(0, 0, 3, 0, L).view(np.uint16).reshape(L, 4), planes.vsc[:L])
    assert (c2.plane_read(0, 0, 2, 0, L).view(np.uint16).reshape(L, 16) != planes.ksc[:L]).mean() < 0.02
    assert (c2.plane_read(0, 0, 0, 0, L).view(np.int8).reshape(L, 1024) != planes.k[:L]).mean() < 0.02
    with pytest.raises(capi.KataError):
        capi.AttnContext(1, [64], kv_mode="int8g", quant_round="half_away")   # the grouped quantiser rounds to even only


@pytest.mark.parametrize("T", [1, 2])
def test_int8g_decode_lengths_and_batch(capi, orc, T):
    # decode over the grouped-scale cache (planes from the oracle's quantiser) against the fp32 formula on the dequantised planes: lengths
    # around the 32-key tile, a long one, first_pos = 1, and a ragged batch with a split that cuts segments
    for L in (1 + T, 31, 33, 64, 700):
        planes, q, gate, _ = _oracle_fill(orc, 63 + L, L, 1024, int8g=True, fast=True)
        ctx = capi.AttnContext(1, [1024], kv_mode="int8g")
        _upload_planes(ctx, planes)
        pb = L - T
        out = ctx.decode(0, [0], [pb], T, _dev(orc.cvt_q_half(q[pb:L])[None]).view(torch.float16), _dev(gate[pb:L][None]))
        ctx.check()
        _close(out.cpu().numpy()[0], orc.formula_f32(q[pb:L], gate[pb:L], planes, pb))
        if L > 2:
            o1 = ctx.decode(0, [0], [pb], T, _dev(orc.cvt_q_half(q[pb:L])[None]).view(torch.float16), _dev(gate[pb:L][None]), first_pos=1)
            _close(o1.cpu().numpy()[0], orc.formula_f32(q[pb:L], gate[pb:L], planes, pb, first_pos=1))
        ctx.close()
    lens = [900, 130, 2048]
    ctx = capi.AttnContext(1, [l + 8 for l in lens], kv_mode="int8g", dec_chunk=64)
    ps, qs, gs = [], [], []
    for s, L in enumerate(lens):
        pl, q, g, _ = _oracle_fill(orc, 90 + s, L, L + 8, int8g=True, fast=True, seq=s)
        _upload_planes(ctx, pl, seq=s); ps.append(pl); qs.append(q); gs.append(g)
    pos = [l - T for l in lens]
    dq = _dev(np.stack([orc.cvt_q_half(qs[s][pos[s]:lens[s]]) for s in range(3)])).view(torch.float16); dg = _dev(np.stack([gs[s][pos[s]:lens[s]] for s in range(3)]))
    out = ctx.decode(0, [0, 1, 2], pos, T, dq, dg).cpu().numpy(); ctx.check()
    for s in range(3):
        _close(out[s], orc.formula_f32(qs[s][pos[s]:lens[s]], gs[s][pos[s]:lens[s]], ps[s], pos[s]))


def test_int8g_prefill_and_full_step(capi, orc):
    # a ragged chunk over a prefix through the tcgen05 kernel (keys expanded to code x group scale), then append + decode on the same context
    pb, M = 300, 200
    planes, q, gate, (qf, kp, vp, qn, kn) = _oracle_fill(orc, 95, pb + M + 2, 640, int8g=True, fast=True)
    ctx = capi.AttnContext(1, [640], kv_mode="int8g")
    _upload_planes(ctx, planes, n=pb + M)
    out = ctx.prefill(0, [0], [pb], M, _dev(orc.cvt_q_half(q[pb:pb + M])[None]).view(torch.float16), _dev(gate[pb:pb + M][None]))
    ctx.check()
    _close(out.cpu().numpy()[0], orc.formula_f32(q[pb:pb + M], gate[pb:pb + M], planes, pb))
    p2 = pb + M
    q16, q32, g = ctx.prep(0, [0], [p2], 2, _dev(qf[p2:p2 + 2][None]), _dev(kp[p2:p2 + 2][None]), _dev(vp[p2:p2 + 2][None]), _dev(qn), _dev(kn), want_q32=True)
    dec = ctx.decode(0, [0], [p2], 2, q16, g); ctx.check()
    _close(dec.cpu().numpy()[0], orc.formula_f32(q[p2:p2 + 2], gate[p2:p2 + 2], planes, p2))
