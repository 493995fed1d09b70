"""Generates tests/golden/attn_golden.npz: known-answer vectors of the attention path computed by the CPU oracle on
seeded synthetic inputs (kata_b200.synth). The reference stores no vectors for this path, so these are produced here;
the inputs are regenerated from the seeds at test time and only outputs (plus input checksums) are stored.

    python -m tests.golden.make_golden        # rewrites the .npz
"""
import os

import numpy as np

from kata_b200 import synth

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")


def compute(orc):
    g = {}
    # -- config 1 of the benchmark statement: one layer, decode of 1 token, KV length 512, fp16 cache
    seed, L = 1001, 512
    qn, kn = synth.norm_weights(seed)
    qf, kp, vp = synth.token_rows(seed, L)
    g["c1_input_sums"] = np.array([qf.sum(dtype=np.float64), kp.sum(dtype=np.float64), vp.sum(dtype=np.float64), qn.sum(dtype=np.float64), kn.sum(dtype=np.float64)])
    p16 = orc.KvPlanes(L)
    q, gate = orc.prep(qf, kp, vp, qn, kn, p16, 0)
    g["c1_k_rows"] = p16.k[[0, 1, 255, 511]].copy()          # fp16 bit patterns of cached (normed, rotated) K rows
    g["c1_v_rows"] = p16.v[[0, 1, 255, 511]].copy()
    g["c1_q_last"] = q[L - 1].copy()
    g["c1_decode"] = orc.dec_attn(q[L - 1 :], gate[L - 1 :], p16, L - 1, T=1)[0]
    g["c1_decode_f32"] = orc.formula_f32(q[L - 1 :], gate[L - 1 :], p16, L - 1)[0]
    g["c1_verify_t2"] = orc.dec_attn(q[L - 2 :], gate[L - 2 :], p16, L - 2, T=2)
    # -- causal prefill with a ragged tail, over a prefix (the shape of the reference's probe: posBase 300, M 70)
    pf = orc.flash_prefill(orc.cvt_q_half(q[300:370]), gate[300:370], p16, 300)
    g["pf_rows_0_33_69"] = pf[[0, 33, 69]].copy()
    # -- int8 cache: quantise-on-append codes/scales (bit-exact class) and a T=2 verify over it
    p8 = orc.KvPlanes(L, int8=True)
    orc.prep(qf, kp, vp, qn, kn, p8, 0)
    g["q8_k_codes"] = p8.k[[0, 1, 255, 511]].copy()
    g["q8_v_codes"] = p8.v[[0, 1, 255, 511]].copy()
    g["q8_k_scales"] = p8.ksc.copy()
    g["q8_v_scales"] = p8.vsc.copy()
    g["q8_verify_t2"] = orc.dec_attn(q[L - 2 :], gate[L - 2 :], p8, L - 2, T=2)
    # -- quantiser edge rows (ties, clamp, zero row, subnormal scale), both rounding modes
    rows = np.zeros((4, 1024), np.float16)
    rows[1, :8] = [127, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]
    rows[2, :2] = [1001.0, -1001.0]
    rows[3, :4] = [6e-6, -3e-6, 1e-6, 6e-8]
    for mode in (0, 1):
        pe = orc.KvPlanes(4, int8=True)
        orc.kv_quant(rows.view(np.uint16), rows.view(np.uint16), pe, 0, mode)
        g[f"edge_codes_mode{mode}"] = pe.k[:, :8].copy()
        g[f"edge_scales_mode{mode}"] = pe.ksc.copy()
    return g


if __name__ == "__main__":
    from oracle import kata_oracle
    kata_oracle.build()
    np.savez_compressed(OUT, **compute(kata_oracle))
    print("wrote", OUT, os.path.getsize(OUT), "bytes")
