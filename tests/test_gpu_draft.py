"""GPU parity of the block drafter's attention (include/kata_draft.h) against the CPU oracle's restatement of k_draft_qk,
k_draft_ctx_kv and k_draft_attn (shaders/draft.metal:203-281), through the C ABI.

Bars: V ring rows bit-exact (a pure fp16 rounding); K ring rows and the query within an fp16 / fp32 ulp or two of the oracle (the RoPE
sine and cosine come from different math libraries); attention outputs within 2e-5 of the oracle on the same ring contents (the kernel
carries ~22 bits of q and p through the tensor cores, the reference 24)."""
import numpy as np
import pytest
import torch

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


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _norms(rng):
    return (1 + 0.05 * rng.standard_normal(128)).astype(np.float32), (1 + 0.05 * rng.standard_normal(128)).astype(np.float32)


def test_qk_and_ctx_kv_match_oracle(capi, orc):
    rng = np.random.default_rng(5)
    ring, win = 256, 128
    ctx = capi.DraftContext(2, ring, win)
    ref = orc.DraftRing(ring, win)
    qn, kn = _norms(rng)
    # context rows through k_draft_ctx_kv (wrapping past the ring end), then a block through k_draft_qk
    n, pos0 = 60, 230
    ck, cv = rng.standard_normal((n, 1024)).astype(np.float32), rng.standard_normal((n, 1024)).astype(np.float32)
    orc.draft_qk(None, ck, cv, None, kn, ref, pos0)
    assert ctx.qk(1, None, _dev(ck), _dev(cv), None, _dev(kn), pos0) is None
    T, bpos = 8, pos0 + n
    qin, kin, vin = rng.standard_normal((T, 4096)).astype(np.float32), rng.standard_normal((T, 1024)).astype(np.float32), rng.standard_normal((T, 1024)).astype(np.float32)
    q_ref = orc.draft_qk(qin, kin, vin, qn, kn, ref, bpos)
    q = ctx.qk(1, _dev(qin), _dev(kin), _dev(vin), _dev(qn), _dev(kn), bpos).cpu().numpy()
    assert np.abs(q - q_ref).max() < 4e-6
    v = ctx.ring_read(1, True); k = ctx.ring_read(1, False)
    assert np.array_equal(v, ref.v)                                             # bit-exact, rows outside the written ones still zero
    written = np.zeros(ring, bool); written[np.arange(pos0, bpos + T) % ring] = True
    assert (k[~written] == 0).all() and (ctx.ring_read(0, False) == 0).all()    # other rows and the other layer untouched
    kd = np.abs(k.view(np.float16).astype(np.float32) - ref.k.view(np.float16).astype(np.float32))
    assert kd.max() < 4e-3 and (k != ref.k).mean() < 0.02


@pytest.mark.parametrize("T", [1, 3, 8, 12, 16])
def test_attention_matches_oracle(capi, orc, T):
    # window 2048 over a 4096 ring (Draft::kWindow / kRing): short history, full window, wrap-around; rows of the block see each other
    rng = np.random.default_rng(100 + T)
    ctx = capi.DraftContext(1, 4096, 2048)
    for pos0 in (0, 5, 130, 2047, 2048, 4090, 9000):
        ref = orc.DraftRing(4096, 2048)
        lo = max(0, pos0 + 1 - 2048)
        keys = np.arange(lo, pos0 + T)
        ref.k[:] = 0x7E00; ref.v[:] = 0x7E00                                   # NaN everywhere but the visible rows
        ref.k[keys % 4096] = rng.standard_normal((len(keys), 1024)).astype(np.float16).view(np.uint16)
        ref.v[keys % 4096] = rng.standard_normal((len(keys), 1024)).astype(np.float16).view(np.uint16)
        ctx.ring_write(0, False, 0, ref.k); ctx.ring_write(0, True, 0, ref.v)
        q = (rng.standard_normal((T, 4096)) * 1.5).astype(np.float32)
        got = ctx.attn(0, _dev(q), pos0).cpu().numpy()
        want = orc.draft_attn(q, ref, pos0)
        assert np.isfinite(got).all() and np.abs(got - want).max() < 2e-5, (pos0, float(np.abs(got - want).max()))


def test_small_window_masks_per_row(capi, orc):
    # a window shorter than the block: every row has its own first visible key
    rng = np.random.default_rng(9)
    ctx = capi.DraftContext(1, 64, 5)
    ref = orc.DraftRing(64, 5)
    ref.k[:] = rng.standard_normal((64, 1024)).astype(np.float16).view(np.uint16); ref.v[:] = rng.standard_normal((64, 1024)).astype(np.float16).view(np.uint16)
    ctx.ring_write(0, False, 0, ref.k); ctx.ring_write(0, True, 0, ref.v)
    for T, pos0 in ((16, 40), (7, 2), (16, 0)):
        q = rng.standard_normal((T, 4096)).astype(np.float32)
        got = ctx.attn(0, _dev(q), pos0).cpu().numpy()
        assert np.abs(got - orc.draft_attn(q, ref, pos0)).max() < 2e-5


def test_block_forward_sequence_and_errors(capi, orc):
    # Draft::materialise + forwardBlockToks, attention part (src/draft.cpp:112-123, 196-209): context rows, then qk + attn per layer
    rng = np.random.default_rng(12)
    ctx = capi.DraftContext(5, 4096, 2048)
    refs = [orc.DraftRing(4096, 2048) for _ in range(5)]
    qn, kn = _norms(rng)
    frontier = 0
    for n in (64, 64, 30):
        for il in range(5):
            ck, cv = rng.standard_normal((n, 1024)).astype(np.float32), rng.standard_normal((n, 1024)).astype(np.float32)
            orc.draft_qk(None, ck, cv, None, kn, refs[il], frontier); ctx.qk(il, None, _dev(ck), _dev(cv), None, _dev(kn), frontier)
        frontier += n
    T = 8
    for il in range(5):
        qin, kin, vin = rng.standard_normal((T, 4096)).astype(np.float32), rng.standard_normal((T, 1024)).astype(np.float32), rng.standard_normal((T, 1024)).astype(np.float32)
        q_ref = orc.draft_qk(qin, kin, vin, qn, kn, refs[il], frontier)
        q = ctx.qk(il, _dev(qin), _dev(kin), _dev(vin), _dev(qn), _dev(kn), frontier)
        out = ctx.attn(il, q, frontier).cpu().numpy()                            # straight after the append on the same stream
        assert np.abs(out - orc.draft_attn(q_ref, refs[il], frontier)).max() < 2e-4   # K rows differ by an fp16 ulp here and there
    assert ctx.launches() == 3 * 5 + 5 * 3
    z = torch.zeros(17, 4096, device="cuda")
    with pytest.raises(capi.KataError):
        ctx.attn(0, z, 0)                                                        # more than KATA_DRAFT_MAX_BLOCK rows
    with pytest.raises(capi.KataError):
        ctx.attn(5, z[:8].contiguous(), 0)                                       # layer out of range
    with pytest.raises(capi.KataError):
        capi.DraftContext(1, 1000, 100)                                          # ring not a power of two
