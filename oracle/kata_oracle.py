"""ctypes front end of the CPU oracle (``kata_oracle.cpp``) plus an independent numpy restatement of the quantiser.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline / reference arm
of ``bench.py``. The ``kata_b200`` package never imports it. Parity status of the oracle itself is described in the
header of ``kata_oracle.cpp``: the fp64 formula is pinned bit for bit to the reference's own check compiled here
(``oracle/_ref``, ``probe_ref.py``); the restated shader kernels' accumulation order and the prep/quantiser kernels remain
"parity unpinned" (the reference stores no golden vectors and its kernels are Metal).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkata_oracle.so")

H, KVH, D, G, QD, KVD, QFULL = 24, 4, 256, 6, 6144, 1024, 12288


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (g++ only, no reference sources are compiled)."""
    src = os.path.join(_HERE, "kata_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.kor_hw_threads.restype = C.c_uint32
    return _lib


def _p(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def hw_threads() -> int:
    return int(lib().kor_hw_threads())


def inv_freq() -> np.ndarray:
    out = np.empty(32, np.float32)
    lib().kor_inv_freq(_p(out))
    return out


class KvPlanes:
    """One attention layer's cache planes on the host, in the reference layout (src/engine.h:73-83):
    K, V: [max_ctx][1024] fp16 (stored as uint16 bit patterns) or int8; scales/mean: [max_ctx][4] fp16.
    ``mode`` 0: fp16; 1 (``int8=True``): K and V int8; 2 (``int8v=True``): K fp16, V int8 (KATA_KV=int8v, src/engine.cpp:54-59);
    3 (``int8g=True``): K int8 with one scale per 64 dims (ksc [max_ctx][16] = [head][group]), V int8 per row."""

    def __init__(self, max_ctx: int, int8: bool = False, poison: bool = False, int8v: bool = False, int8g: bool = False):
        self.max_ctx, self.int8 = max_ctx, int8
        self.mode = 1 if int8 else 2 if int8v else 3 if int8g else 0
        fill = 0x7E00 if poison else 0  # fp16 quiet NaN
        self.ksc = self.vsc = self.kmn = None
        if self.mode == 1:
            self.k = np.zeros((max_ctx, KVD), np.int8)
            self.ksc = np.zeros((max_ctx, 4), np.uint16)
            self.kmn = np.zeros((max_ctx, 4), np.uint16)
        elif self.mode == 3:
            self.k = np.zeros((max_ctx, KVD), np.int8)
            self.ksc = np.zeros((max_ctx, 16), np.uint16)
        else:
            self.k = np.full((max_ctx, KVD), fill, np.uint16)
        if self.mode:
            self.v = np.zeros((max_ctx, KVD), np.int8)
            self.vsc = np.zeros((max_ctx, 4), np.uint16)
        else:
            self.v = np.full((max_ctx, KVD), fill, np.uint16)

    def k_f32(self):
        return self.k.astype(np.float32) if self.mode in (1, 3) else self.k.view(np.float16).astype(np.float32)

    def v_f32(self):
        return self.v.astype(np.float32) if self.mode else self.v.view(np.float16).astype(np.float32)


def prep(qfull, kproj, vproj, qnorm, knorm, planes: KvPlanes, pos0: int, h0: int = 0, nh: int = 32, quant_mode: int = 0):
    """k_attn_prep(_b) (+ k_kv_quant_sym in int8 mode, as src/engine.cpp:167-168 chains them). Returns (q, gate) fp32 [M][6144]."""
    M = kproj.shape[0]
    q = np.zeros((M, QD), np.float32)
    gate = np.zeros((M, QD), np.float32)
    invf = inv_freq()
    qf = qfull if qfull is not None else np.zeros((M, QFULL), np.float32)
    if planes.mode == 2:   # keys straight into the fp16 plane, values through the scratch rows and the quantiser
        vs = np.zeros((M, KVD), np.uint16)
        lib().kor_prep(_p(qf), _p(kproj), _p(vproj), _p(qnorm), _p(knorm), _p(invf), _p(q), _p(gate), _p(planes.k), _p(vs),
                       C.c_uint32(pos0), C.c_uint32(M), C.c_uint32(h0), C.c_uint32(nh), C.c_uint32(0), C.c_uint32(pos0))
        if h0 + nh > 28:
            kv_quant(None, vs, planes, pos0, quant_mode)
    elif planes.int8 or planes.mode == 3:
        ks = np.zeros((M, KVD), np.uint16)
        vs = np.zeros((M, KVD), np.uint16)
        lib().kor_prep(_p(qf), _p(kproj), _p(vproj), _p(qnorm), _p(knorm), _p(invf), _p(q), _p(gate), _p(ks), _p(vs),
                       C.c_uint32(pos0), C.c_uint32(M), C.c_uint32(h0), C.c_uint32(nh), C.c_uint32(pos0), C.c_uint32(pos0))
        kv_quant(ks, vs, planes, pos0, 3 if planes.mode == 3 else quant_mode)
    else:
        lib().kor_prep(_p(qf), _p(kproj), _p(vproj), _p(qnorm), _p(knorm), _p(invf), _p(q), _p(gate), _p(planes.k), _p(planes.v),
                       C.c_uint32(pos0), C.c_uint32(M), C.c_uint32(h0), C.c_uint32(nh), C.c_uint32(0), C.c_uint32(0))
    return q, gate


def kv_quant(ks, vs, planes: KvPlanes, pos0: int, mode: int = 0):
    """k_kv_quant_sym (mode 0, rint), half-away variant (mode 1), reference asymmetric-K (mode 2), one K scale per 64 dims (mode 3, planes of mode 3)."""
    assert planes.mode and vs.dtype == np.uint16 and (ks is None) == (planes.mode == 2) and (mode == 3) == (planes.mode == 3)
    T = vs.shape[0]
    lib().kor_kv_quant(_p(ks), _p(vs), _p(planes.k) if planes.mode in (1, 3) else None, _p(planes.v), _p(planes.ksc), _p(planes.vsc), _p(planes.kmn), C.c_uint32(pos0), C.c_uint32(T), C.c_int(mode))


def attn_decode(q, gate, planes: KvPlanes, pos: int, threads: int = 1):
    """k_attn_decode: q, gate fp32 [6144] -> out fp32 [6144]."""
    assert planes.mode == 0
    out = np.zeros(QD, np.float32)
    lib().kor_attn_decode(_p(q), _p(gate), _p(planes.k), _p(planes.v), _p(out), C.c_uint32(pos), C.c_uint32(threads))
    return out


def attn_split_combine(q, gate, planes: KvPlanes, pos_base: int, T: int = 1, first_pos: int = 0, S: int | None = None):
    """k_attn_split(_b) + k_attn_combine(_b); S defaults to the engine's choice (src/engine.cpp:171)."""
    assert planes.mode == 0
    if S is None:
        S = min(32, max(1, (pos_base + 1) // 64))
    pm = np.zeros((T * 24, S), np.float32)
    pl = np.zeros((T * 24, S), np.float32)
    pacc = np.zeros((T * 24, S, D), np.float32)
    out = np.zeros((T, QD), np.float32)
    lib().kor_attn_split(_p(q), _p(planes.k), _p(planes.v), _p(pm), _p(pl), _p(pacc), C.c_uint32(pos_base), C.c_uint32(first_pos), C.c_uint32(S), C.c_uint32(T))
    lib().kor_attn_combine(_p(pm), _p(pl), _p(pacc), _p(gate), _p(out), C.c_uint32(S), C.c_uint32(T))
    return out


def cvt_q_half(q):
    out = np.zeros(q.shape, np.uint16)
    lib().kor_cvt_q_half(_p(q), _p(out), C.c_uint64(q.size))
    return out


def flash_prefill(q16, gate, planes: KvPlanes, pos_base: int, threads: int = 0):
    """k_flash_prefill / _q8: q16 fp16 bits [M][6144] prescaled -> out fp32 [M][6144]."""
    M = q16.shape[0]
    out = np.zeros((M, QD), np.float32)
    lib().kor_flash_prefill(_p(q16), _p(planes.k), _p(planes.v), _p(gate), _p(out), C.c_uint32(pos_base), C.c_uint32(M),
                            _p(planes.ksc), _p(planes.vsc), _p(planes.kmn), C.c_int(planes.mode), C.c_uint32(threads or hw_threads()))
    return out


def dec_attn(q, gate, planes: KvPlanes, pos_base: int, T: int = 1, first_pos: int = 0, chunk: int = 128, threads: int = 0):
    """Engine::dDecAttn (src/engine.cpp:119-127): k_dec_q_pack -> k_attn_dec_split[_q8] -> k_attn_dec_combine."""
    qp = np.zeros((4, 16, D), np.uint16)
    lib().kor_dec_q_pack(_p(q), _p(qp), C.c_uint32(T))
    ns = (pos_base + T - first_pos + chunk - 1) // chunk
    pacc = np.zeros((4 * ns * 16, D), np.float32)
    pm = np.zeros(4 * ns * 16, np.float32)
    pl = np.zeros(4 * ns * 16, np.float32)
    lib().kor_attn_dec_split(_p(qp), _p(planes.k), _p(planes.v), _p(pacc), _p(pm), _p(pl), C.c_uint32(pos_base), C.c_uint32(T), C.c_uint32(first_pos), C.c_uint32(chunk),
                             _p(planes.ksc), _p(planes.vsc), _p(planes.kmn), C.c_int(planes.mode), C.c_uint32(threads or hw_threads()))
    out = np.zeros((T, QD), np.float32)
    lib().kor_attn_dec_combine(_p(pacc), _p(pm), _p(pl), _p(gate), _p(out), C.c_uint32(pos_base), C.c_uint32(T), C.c_uint32(first_pos), C.c_uint32(chunk))
    return out


def formula_f64(q16, gate, planes: KvPlanes, pos_base: int, first_pos: int = 0, t_step: int = 1, h_step: int = 1, threads: int = 0):
    """The reference's own fp64 check (tools/probe_flash.cpp:29-34). Entries not visited stay NaN."""
    M = q16.shape[0]
    out = np.full((M, QD), np.nan, np.float64)
    lib().kor_formula_f64(_p(q16), _p(planes.k), _p(planes.v), _p(gate), _p(out), C.c_uint32(pos_base), C.c_uint32(M), C.c_uint32(first_pos), C.c_uint32(t_step), C.c_uint32(h_step),
                          _p(planes.ksc), _p(planes.vsc), _p(planes.kmn), C.c_int(planes.mode), C.c_uint32(threads or hw_threads()))
    return out


def formula_f32(q, gate, planes: KvPlanes, pos_base: int, first_pos: int = 0, threads: int = 0):
    """fp32 evaluation of softmax(q k^T / 16) v * sigmoid(gate) on the cache contents: the tolerance reference."""
    M = q.shape[0]
    out = np.zeros((M, QD), np.float32)
    lib().kor_formula_f32(_p(q), _p(planes.k), _p(planes.v), _p(gate), _p(out), C.c_uint32(pos_base), C.c_uint32(M), C.c_uint32(first_pos),
                          _p(planes.ksc), _p(planes.vsc), _p(planes.kmn), C.c_int(planes.mode), C.c_uint32(threads or hw_threads()))
    return out


def out_fwht(x, sign):
    """sign (.) x through the normalised 1024-point Walsh-Hadamard transform per block (k_rms_fwht mode 3), fp32, the shader's stage order."""
    x = np.ascontiguousarray(x, np.float32); sign = np.ascontiguousarray(sign, np.float32)
    out = np.empty_like(x)
    lib().kor_out_fwht(_p(x), _p(sign), _p(out), C.c_uint32(x.shape[0]), C.c_uint32(x.shape[1]))
    return out


def decode_batch(q, gate, k_planes, v_planes, pos, threads: int = 0):
    """CPU baseline: one layer's decode step for a batch (k_attn_decode per (sequence, head)) on `threads` host threads."""
    B = q.shape[0]
    out = np.zeros((B, QD), np.float32)
    kp = (C.c_void_p * B)(*[k.ctypes.data for k in k_planes])
    vp = (C.c_void_p * B)(*[v.ctypes.data for v in v_planes])
    posa = np.asarray(pos, np.uint32)
    lib().kor_decode_batch(_p(q), _p(gate), kp, vp, _p(out), _p(posa), C.c_uint32(B), C.c_uint32(threads or hw_threads()))
    return out


# ---- independent numpy restatement of the symmetric quantiser (shaders/flash.metal:165-178) ----
def kv_quant_rows_np(rows_f16: np.ndarray, half_away: bool = False):
    """rows_f16: float16 [..., 256]. Returns (int8 codes, float16 scales). Written without reference to the C++ oracle
    so the two can be compared bit for bit."""
    v = rows_f16.astype(np.float32)
    amax = np.max(np.abs(v), axis=-1, keepdims=True).astype(np.float32)
    sc = np.where(amax > 0, (amax / np.float32(127.0)).astype(np.float32).astype(np.float16), np.float16(1.0)).astype(np.float16)
    inv = (np.float32(1.0) / sc.astype(np.float32)).astype(np.float32)
    x = (v * inv).astype(np.float32)
    x64 = x.astype(np.float64)  # x + 0.5 is exact in fp64 for every fp32 x in range, so floor/ceil see the true value
    r = np.where(x64 >= 0, np.floor(x64 + 0.5), np.ceil(x64 - 0.5)) if half_away else np.rint(x)
    return np.clip(r, -127, 127).astype(np.int8), sc[..., 0]


# ---- the block drafter's attention (shaders/draft.metal:203-281) ----
DRAFT_H, DRAFT_KVH, DRAFT_D = 32, 8, 128


class DraftRing:
    """One drafter layer's K and V rings on the host: [ring][8 * 128] fp16 bit patterns, position p at row p % ring (src/draft.h:36)."""

    def __init__(self, ring: int = 4096, window: int = 2048):
        self.ring, self.window = ring, window
        self.k = np.zeros((ring, DRAFT_KVH * DRAFT_D), np.uint16)
        self.v = np.zeros((ring, DRAFT_KVH * DRAFT_D), np.uint16)


def draft_inv_freq() -> np.ndarray:
    out = np.empty(64, np.float32)
    lib().kor_draft_inv_freq(_p(out))
    return out


def draft_qk(qin, kin, vin, qnorm, knorm, rings: DraftRing, pos0: int):
    """k_draft_qk (qin given; returns the fp32 query rows) or k_draft_ctx_kv (qin None): K and V rows of positions pos0.. into the rings."""
    T = kin.shape[0]
    qout = np.zeros((T, DRAFT_H * DRAFT_D), np.float32) if qin is not None else None
    lib().kor_draft_qk(_p(qin), _p(kin), _p(vin), _p(qnorm), _p(knorm), _p(draft_inv_freq()), _p(qout), _p(rings.k), _p(rings.v), C.c_uint32(pos0), C.c_uint32(T), C.c_uint32(rings.ring))
    return qout


def draft_attn(q, rings: DraftRing, pos0: int, threads: int = 0):
    """k_draft_attn: q fp32 [T][4096] -> out fp32 [T][4096]; non-causal inside the block, sliding window behind it."""
    T = q.shape[0]
    out = np.zeros((T, DRAFT_H * DRAFT_D), np.float32)
    lib().kor_draft_attn(_p(q), _p(rings.k), _p(rings.v), _p(out), C.c_uint32(pos0), C.c_uint32(T), C.c_uint32(rings.window), C.c_uint32(rings.ring), C.c_uint32(threads or hw_threads()))
    return out
