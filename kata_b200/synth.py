"""Seeded synthetic inputs for the attention path, with the distributions the benchmark statement gives:
pre-norm q, k, v ~ N(0,1); QK-norm weights 1 + N(0, 0.05); gate logits ~ N(0,1). One Philox stream per tensor
(key = seed, counter offset by a tensor id), so tensors can be regenerated independently and in any order.
No dataset or benchmark suite is involved anywhere in this repository; every input is produced here."""
from __future__ import annotations

import numpy as np

H, KVH, D, QD, KVD, QFULL = 24, 4, 256, 6144, 1024, 12288

_T_QFULL, _T_K, _T_V, _T_QNORM, _T_KNORM, _T_LEN = range(6)


def _rng(seed: int, tensor_id: int, layer: int = 0, seq: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, (tensor_id << 40) | (layer << 24) | seq]))


def norm_weights(seed: int, layer: int = 0):
    """(qnorm, knorm) effective RMSNorm weights, fp32 [256] each."""
    qn = (1.0 + 0.05 * _rng(seed, _T_QNORM, layer).standard_normal(D)).astype(np.float32)
    kn = (1.0 + 0.05 * _rng(seed, _T_KNORM, layer).standard_normal(D)).astype(np.float32)
    return qn, kn


def token_rows(seed: int, M: int, layer: int = 0, seq: int = 0, start: int = 0):
    """Projection outputs for tokens [start, start+M) of one sequence and layer:
    qfull [M][12288] (per head [query 256 | gate 256]), kproj [M][1024], vproj [M][1024], fp32.
    Row t depends only on (seed, layer, seq, start+t), so chunked and one-shot generation agree."""
    qf = np.empty((M, QFULL), np.float32)
    kp = np.empty((M, KVD), np.float32)
    vp = np.empty((M, KVD), np.float32)
    for tid, arr, w in ((_T_QFULL, qf, QFULL), (_T_K, kp, KVD), (_T_V, vp, KVD)):
        base = (tid << 40) | (layer << 24) | seq
        for t in range(M):  # one stream per row: standard_normal consumes a data-dependent number of draws
            g = np.random.Generator(np.random.Philox(key=[seed ^ 0x5DEECE66D, base + ((start + t) << 44)]))
            arr[t] = g.standard_normal(w, dtype=np.float32)
    return qf, kp, vp


def seq_lengths(seed: int, batch: int, lo: int = 16384, hi: int = 32768):
    """Context lengths for a decode batch: uniform integers in [lo, hi]; a batch of 1 gets hi."""
    if batch == 1:
        return np.array([hi], np.int64)
    return _rng(seed, _T_LEN).integers(lo, hi + 1, size=batch, dtype=np.int64)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def token_rows_fast(seed: int, M: int, layer: int = 0, seq: int = 0):
    """Same distributions as token_rows from ONE stream per tensor (fast for tens of thousands of rows; rows are not
    position-independent, so use it only where a cache is filled in one go)."""
    qf = _rng(seed, _T_QFULL, layer, seq).standard_normal((M, QFULL), dtype=np.float32)
    kp = _rng(seed, _T_K, layer, seq).standard_normal((M, KVD), dtype=np.float32)
    vp = _rng(seed, _T_V, layer, seq).standard_normal((M, KVD), dtype=np.float32)
    return qf, kp, vp
