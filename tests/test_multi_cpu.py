"""World-size-2 (and 3) CPU tests of the multi-GPU host logic over gloo: sequence sharding, key-range split, and the
all-gather + merge of per-rank partials against the single-rank result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kata_b200 import multi


def test_shard_sequences_balances_lengths():
    lens = [32768, 16384, 20000, 30000, 17000, 25000, 31000, 18000]
    for world in (1, 2, 4, 8):
        plan = multi.shard_sequences(lens, world)
        assert sorted(i for p in plan for i in p) == list(range(8))
        loads = [sum(lens[i] for i in p) for p in plan]
        assert max(loads) - min(loads) <= max(lens)


def test_split_keys_covers_range():
    for n, world in ((32768, 8), (1000, 3), (5, 4), (7302, 2)):
        r = multi.split_keys(n, world)
        assert r[0][0] == 0 and r[-1][1] == n and all(r[i][1] == r[i + 1][0] for i in range(world - 1))
        assert all(lo % 16 == 0 for lo, _ in r[1:] if lo < n)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _partial(q, k, v, lo, hi, pos):
    """fp32 partial of rows [24][256] queries over keys [lo, min(hi, pos+1)) -> [24][258]"""
    out = np.zeros((24, 258), np.float32); out[:, 256] = -np.inf
    hi = min(hi, pos + 1)
    if hi <= lo:
        return out
    for h in range(24):
        kv = h // 6
        s = (k[lo:hi, kv] @ (q[h] * np.float32(0.0625))).astype(np.float32)
        m = s.max(); p = np.exp(s - m)
        out[h, :256] = p @ v[lo:hi, kv]; out[h, 256] = m; out[h, 257] = p.sum()
    return out


def _worker(rank, world, port, L, q, k, v, gate, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = multi.split_keys(L, world)[rank]
    part = torch.from_numpy(_partial(q, k, v, lo, hi, L - 1))
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    out = multi.merge_parts_numpy(torch.stack(parts).numpy(), gate)
    if rank == 0:
        ret.put(out)
    dist.barrier(); dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_split_kv_merge_over_gloo(world):
    rng = np.random.default_rng(world)
    L = 333
    q = rng.standard_normal((24, 256)).astype(np.float32); gate = rng.standard_normal((24, 256)).astype(np.float32)
    k = rng.standard_normal((L, 4, 256)).astype(np.float32); v = rng.standard_normal((L, 4, 256)).astype(np.float32)
    full = multi.merge_parts_numpy(_partial(q, k, v, 0, L, L - 1)[None], gate)
    ctx = mp.get_context("spawn"); ret = ctx.Queue(); port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, L, q, k, v, gate, ret)) for r in range(world)]
    for p in procs: p.start()
    out = ret.get(timeout=120)
    for p in procs: p.join(timeout=60)
    assert all(p.exitcode == 0 for p in procs)
    assert np.abs(out - full).max() < 2e-5


def _head_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import kata_oracle as orc
    from kata_b200 import synth
    qn, kn = synth.norm_weights(5)
    qf, kp, vp = synth.token_rows_fast(5, 40)
    planes = orc.KvPlanes(64)
    q, gate = orc.prep(qf, kp, vp, qn, kn, planes, 0)
    full = orc.formula_f32(q[38:], gate[38:], planes, 38)            # every rank can form the whole result on the host ...
    lo, n = multi.shard_kv_heads(world)[rank]
    mine = torch.from_numpy(np.ascontiguousarray(full[:, multi.head_columns(lo, n)]))   # ... but contributes only the columns of its KV heads
    got = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(got, mine)
    whole = torch.cat(got, dim=1).numpy()
    if rank == 0:
        ret.put(bool(np.array_equal(whole, full)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_kv_head_shards_gather_to_whole_rows_over_gloo(world):
    # the host-side plan of the head-sharded group: disjoint column blocks in rank order make up the row
    assert multi.shard_kv_heads(2) == [(0, 2), (2, 2)] and multi.head_columns(1, 2) == slice(1536, 4608)
    ctx = mp.get_context("spawn"); ret = ctx.Queue(); port = _free_port()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    ok = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
    assert ok
