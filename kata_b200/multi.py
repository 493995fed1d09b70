"""Host-side sharding of the attention path across the GPUs of one box (one process per GPU).

Two plans, neither of which has a reference counterpart (the reference is single-device):
  * independent sequences of a batch -> ranks, balanced by context length (no data-path collective);
  * one long sequence -> contiguous key ranges per rank; every rank computes the unnormalised partial {O, m, l} of its
    keys (kata_attn_decode_partial), the parts are all-gathered and merged with the reference's split-merge rule
    (k_attn_dec_combine, shaders/flash.metal:147-151, with "split" = rank).
"""
from __future__ import annotations

import numpy as np


def shard_sequences(lengths, world: int):
    """Greedy longest-first bin packing of sequences onto ranks. Returns a list (per rank) of sequence indices."""
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]))
    load, out = [0] * world, [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i); load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def split_keys(n_keys: int, world: int, align: int = 16):
    """Contiguous key ranges [lo, hi) per rank, boundaries aligned to the decode tile; the last rank takes the tail
    (and is the one that appends new rows)."""
    per = -(-n_keys // world)
    per = -(-per // align) * align
    return [(min(r * per, n_keys), min((r + 1) * per, n_keys)) if r < world - 1 else (min(r * per, n_keys), max(n_keys, min(r * per, n_keys))) for r in range(world)]


def merge_parts_numpy(parts: np.ndarray, gate: np.ndarray) -> np.ndarray:
    """Reference merge on the host (tests only): parts [ranks][rows][258] = {O[256], m (natural log units), l};
    gate [rows][256]. Returns [rows][256]."""
    m = parts[:, :, 256]
    M = m.max(axis=0)
    w = np.where(np.isneginf(m), 0.0, np.exp(m - M[None, :])).astype(np.float32)
    L = (parts[:, :, 257] * w).sum(axis=0)
    A = (parts[:, :, :256] * w[:, :, None]).sum(axis=0)
    return (A / L[:, None]) * (1.0 / (1.0 + np.exp(-gate)))
