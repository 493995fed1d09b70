"""Host logic of the tcgen05 prefill's work split (kata_attn_prefill_plan: no GPU involved): whatever the batch, every key tile of every
work item is computed exactly once, the head of a cut item is the last thing its pair computes and every other
part the first thing after its pair's rounds (the order the in-kernel merge of cut items relies on), and the heaviest pair stays close to the mean."""
import ctypes as C
import random

import pytest

from kata_b200 import capi

E = 2   # the planner's per-part allowance, in key tiles


def _plan(M, pos, kvh_lo=0, kvh_n=4, pairs=74):
    L = C.CDLL(capi.LIB_PATH)
    n = len(pos)
    n_q = (M + 127) // 128
    n_items = 3 * n_q * kvh_n * n
    arr = (C.c_int32 * n)(*pos); scratch = (C.c_int32 * max(n_items, 1))(); rounds = C.c_int32()
    i0 = (C.c_int32 * 75)(); t0 = (C.c_int32 * 75)(); order = (C.c_uint8 * n)()
    P = L.kata_attn_prefill_plan(M, n, arr, kvh_lo, kvh_n, pairs, scratch, C.byref(rounds), i0, t0, order)
    assert 1 <= P <= min(74, pairs)
    order = list(order)
    assert sorted(order) == list(range(n)) and [pos[i] for i in order] == sorted(pos)
    tiles = []
    for idx in range(n_items):
        grp, mem = divmod(idx, 3 * n_q); qt = n_q - 1 - mem // 3; bi = order[grp // kvh_n]; q0 = qt * 128
        tiles.append((pos[bi] + q0 + min(128, M - q0) + 127) // 128)
    assert list(scratch)[:n_items] == tiles
    return P, rounds.value, list(i0)[:P + 1], list(t0)[:P + 1], tiles


def _check(M, pos, **kw):
    P, R, i0, t0, tiles = _plan(M, pos, **kw)
    n_items, rem0 = len(tiles), R * P
    assert rem0 <= n_items and i0[0] == 0 and t0[0] == 0 and i0[P] == n_items - rem0 and t0[P] == 0
    parts, loads = {}, []
    for p in range(P):
        lo, hi = (i0[p], t0[p]), (i0[p + 1], t0[p + 1])
        assert lo <= hi
        my_parts = 0 if (lo[0] == hi[0] and lo[1] >= hi[1]) else hi[0] - lo[0] + (1 if hi[1] > 0 else 0)
        load = 0
        for it in range(R + my_parts):
            k = it - R
            idx = P * it + (P - 1 - p if it & 1 else p) if k < 0 else rem0 + lo[0] + k
            assert 0 <= idx < n_items
            j0 = lo[1] if k == 0 else 0
            j1 = hi[1] if (k >= 0 and lo[0] + k == hi[0]) else tiles[idx]
            assert 0 <= j0 < j1 <= tiles[idx]
            parts.setdefault(idx, []).append((j0, j1, p, it, R + my_parts))
            load += j1 - j0 + E
        loads.append(load)
    assert sorted(parts) == list(range(n_items))                       # every item is somebody's
    for idx, ps in parts.items():
        ps.sort()
        assert ps[0][0] == 0 and ps[-1][1] == tiles[idx] and all(a[1] == b[0] for a, b in zip(ps, ps[1:]))   # its key tiles exactly once
        if len(ps) > 1:
            head = ps[0]; assert head[3] == head[4] - 1                 # the head is its pair's last part
            assert [q[2] for q in ps[1:]] == sorted(q[2] for q in ps[1:]) and all(q[2] > head[2] for q in ps[1:])   # the others on later pairs, in order
            assert all(q[3] == R for q in ps[1:])                      # each the first thing after its pair's rounds
    return P, R, max(loads), sum(loads) / P


def test_uniform_batches_use_rounds_and_balance():
    P, R, worst, mean = _check(512, [5120] * 16)
    assert P == 74 and R == 9 and worst <= 1.02 * mean
    P, R, worst, mean = _check(512, [5120])          # 48 items for 74 pairs: no rounds, every item cut
    assert P == 74 and R == 0 and worst <= 1.15 * mean
    P, R, worst, mean = _check(512, [0])             # a 512-token prompt: items of 1 to 4 key tiles stay whole
    assert R == 0 and worst == 4 + E


def test_random_batches_keep_the_invariants():
    rng = random.Random(5)
    for _ in range(400):
        n = rng.choice([1, 1, 2, 3, 4, 8, 16, 33, 64]); M = rng.choice([1, 2, 64, 116, 128, 129, 256, 512, 700, 1024])
        pos = [rng.choice([0, 100, 1000, 3600, 7300, 20000, 32000, 60000]) + rng.randint(0, 300) for _ in range(n)] if rng.random() < 0.6 else [rng.choice([0, 3600, 5120])] * n
        kvh_n = rng.choice([4, 4, 1, 2, 3]); kvh_lo = rng.randint(0, 4 - kvh_n)
        _check(M, pos, kvh_lo=kvh_lo, kvh_n=kvh_n, pairs=rng.choice([74, 74, 66, 10]))


def test_arguments_out_of_range():
    L = C.CDLL(capi.LIB_PATH)
    one = (C.c_int32 * 1)(5); s = (C.c_int32 * 64)(); r = C.c_int32(); a = (C.c_int32 * 75)(); b = (C.c_int32 * 75)(); o = (C.c_uint8 * 1)()
    assert L.kata_attn_prefill_plan(0, 1, one, 0, 4, 74, s, C.byref(r), a, b, o) == -1
    assert L.kata_attn_prefill_plan(128, 1, one, 3, 2, 74, s, C.byref(r), a, b, o) == -1
    assert L.kata_attn_prefill_plan(128, 1, None, 0, 4, 74, s, C.byref(r), a, b, o) == -1
