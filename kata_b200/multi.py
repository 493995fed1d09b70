"""Host-side sharding of the attention path across the GPUs of one box (one process per GPU).

Three plans, none of which has a reference counterpart (the reference is single-device):
  * KV-head groups -> ranks (up to 4): a rank owns whole KV heads and their 6 query heads each; attention needs no exchange, the output
    rows are disjoint 256-wide column blocks which the consumer gathers if it wants whole rows;
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


def shard_kv_heads(world: int):
    """(first KV head, number of KV heads) per rank for a head-sharded group of 1, 2 or 4 ranks."""
    if world not in (1, 2, 4):
        raise ValueError("the 4 KV heads shard over 1, 2 or 4 ranks")
    per = 4 // world
    return [(r * per, per) for r in range(world)]


def head_columns(kv_head_lo: int, kv_head_n: int):
    """Column slice of a [.., 6144] query / gate / output row that belongs to KV heads [lo, lo + n): 6 query heads of 256 dims per KV head."""
    return slice(kv_head_lo * 6 * 256, (kv_head_lo + kv_head_n) * 6 * 256)


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
