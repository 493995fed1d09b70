"""Host logic of the decode kernel's work split (kata_attn_decode_plan: no GPU involved): the CTA ranges cut the list of key tiles exactly, the map
from a tile to its CTA agrees with the ranges (checked inside the library for every tile), segments of equal length get CTAs of their own when
that uses nearly all SMs, the reference's split size gives the reference's number of splits, and the count of contributors that decides where the
partials are merged is what the ranges say."""
import ctypes as C
import random

from kata_b200 import capi


def _plan(kend, first_row=0, kvh_n=4, tile_keys=16, sm=148, dec_chunk=0, max_items=None):
    L = C.CDLL(capi.LIB_PATH)
    n = len(kend); max_items = max_items or sm * 8 + 4 * 64
    arr = (C.c_int32 * n)(*kend); nt = (C.c_int32 * n)(); cap = sm * 8 + 2; ft = (C.c_int32 * cap)()
    cps, mik, mc = C.c_int32(), C.c_int32(), C.c_int32()
    n_ctas = L.kata_attn_decode_plan(n, arr, first_row, kvh_n, tile_keys, sm, dec_chunk, max_items, nt, ft, cap, C.byref(cps), C.byref(mik), C.byref(mc))
    assert n_ctas >= 1, n_ctas
    return n_ctas, list(nt), list(ft)[:n_ctas + 1], cps.value, mik.value, mc.value


def _check(kend, **kw):
    n_ctas, nt, ft, cps, mik, mc = _plan(kend, **kw)
    tile_keys, kvh_n, first_row = kw.get("tile_keys", 16), kw.get("kvh_n", 4), kw.get("first_row", 0)
    assert nt == [max(1, (max(0, k - first_row) + tile_keys - 1) // tile_keys) for k in kend]
    total = kvh_n * sum(nt)
    assert ft[0] == 0 and ft[-1] == total and all(a < b for a, b in zip(ft, ft[1:]))       # every CTA has work, every tile one CTA
    # contributors per segment, counted from the ranges
    worst, start = 1, 0
    for b in range(len(kend)):
        for kv in range(kvh_n):
            lo, hi = start, start + nt[b]; start = hi
            worst = max(worst, sum(1 for c in range(n_ctas) if ft[c] < hi and ft[c + 1] > lo))
    assert worst == mc and mik == (1 if mc <= 8 else 0)
    if cps:
        assert len(set(nt)) == 1 and n_ctas == cps * kvh_n * len(kend)
        assert all(ft[c] % nt[0] == 0 for c in range(0, n_ctas, cps))                       # no CTA crosses into another segment
    return n_ctas, cps, mc


def test_headline_and_single_sequence_shapes():
    rng = random.Random(1234)
    n_ctas, cps, mc = _check([rng.randint(16384, 32768) for _ in range(8)])
    assert n_ctas == 148 and cps == 0 and mc <= 8
    n_ctas, cps, mc = _check([32769])                       # one 32K sequence: 4 segments of equal length, 37 CTAs each
    assert (n_ctas, cps, mc) == (148, 37, 37)
    n_ctas, cps, mc = _check([8193], tile_keys=32)          # int8 keys, 8K
    assert cps == 37 and n_ctas == 148
    n_ctas, cps, mc = _check([1])                           # one key: one tile per segment
    assert n_ctas == 4


def test_reference_split_size():
    for L in (512, 7302, 32768):
        n_ctas, cps, mc = _check([L], dec_chunk=128, max_items=148 * 8 + 4 * 64)
        assert n_ctas == min(148 * 8, -(-(4 * -(-L // 16)) // 8))      # ranges of 128 keys = 8 tiles over the four segments' tiles, capped at 8 CTAs per SM


def test_random_batches():
    rng = random.Random(7)
    for _ in range(300):
        n = rng.choice([1, 1, 2, 3, 8, 17, 64]); tk = rng.choice([16, 32]); kv = rng.choice([4, 4, 1, 2])
        kend = [rng.choice([1, 15, 16, 17, 300, 4096, 8192, 20000, 32768]) + rng.randint(0, 40) for _ in range(n)] if rng.random() < 0.7 else [rng.choice([512, 8192, 32768])] * n
        _check(kend, kvh_n=kv, tile_keys=tk, dec_chunk=rng.choice([0, 0, 64, 128, 256, 1024]), first_row=rng.choice([0, 0, 1]), sm=rng.choice([148, 148, 132, 16]))
