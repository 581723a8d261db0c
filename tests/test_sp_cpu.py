"""Host-side logic of the sequence-parallel path on CPU ranks (gloo, world size 2): shard bounds,
segment slicing, and the two Ulysses exchanges as exact permutations of the single-process layout."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rapid_h3_b200 import sp as spmod


def test_shard_bounds_and_segments():
    b = spmod.shard_bounds(36436, 8)
    assert b[0] == (0, 72 * 64) and b[-1][1] == 36436 and sum(hi - lo for lo, hi in b) == 36436
    assert all(lo % 64 == 0 for lo, _ in b) and all(hi > lo for lo, hi in b)
    assert max(hi - lo for lo, hi in b) - min(hi - lo for lo, hi in b) <= 128
    assert spmod.shard_bounds(37, 2, align=1) == [(0, 19), (19, 37)]
    segs = [(0, 36288, 0), (36288, 36436, 1)]
    lo, hi = b[-1]
    cut = spmod.shard_segments(segs, lo, hi)
    assert cut == [(0, 36288 - lo, 0), (36288 - lo, hi - lo, 1)]
    assert spmod.shard_segments(segs, *b[0]) == [(0, 72 * 64, 0)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, heads, hd, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        qkv_full = torch.randn(total, 3 * heads * hd, generator=g)
        u = spmod.Ulysses(total)
        q, k, v = u.tokens_to_heads(qkv_full[u.lo:u.hi].contiguous(), heads, hd)
        hp = heads // world
        ref = qkv_full.view(total, 3, heads, hd)[:, :, rank * hp:(rank + 1) * hp]
        ok = all(torch.equal(t, ref[:, i]) for i, t in enumerate((q, k, v)))
        # a stand-in "attention" that is local to a head: o = q + 2k - v
        og = (q + 2 * k - v).contiguous()
        back = u.heads_to_tokens(og)                       # [P, S_local, hp*hd]
        mine = back.permute(1, 0, 2).reshape(u.hi - u.lo, heads * hd)
        full = (qkv_full.view(total, 3, heads * hd)[:, 0] + 2 * qkv_full.view(total, 3, heads * hd)[:, 1]
                - qkv_full.view(total, 3, heads * hd)[:, 2])
        ok = ok and torch.equal(mine, full[u.lo:u.hi])
        ok = ok and torch.equal(u.gather_tokens(mine), full)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_ulysses_exchanges_are_exact_permutations():
    world, total, heads, hd = 2, 165, 4, 8   # 165 tokens: uneven shards (128 + 37)
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), total, heads, hd, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_scatter_plan_tiles_every_destination_buffer():
    """The output rows that the P head groups store into rank r's exchange buffer must tile [P, count_r, w]
    exactly (no gap, no overlap), for even and ragged shard sizes and every world size the step supports."""
    from rapid_h3_b200 import sp
    for total in (36436, 17896, 221, 4096):
        for world in (1, 2, 4, 8):
            bounds = sp.shard_bounds(total, world)
            assert bounds[0][0] == 0 and bounds[-1][1] == total
            w = (32 // world) * 128
            for r in range(world):
                count = bounds[r][1] - bounds[r][0]
                spans = []
                for g in range(world):  # source rank g = head group g
                    offsets, starts = sp.scatter_plan(bounds, g, w)
                    assert starts == [a for a, _ in bounds] + [total]
                    spans.append((offsets[r], offsets[r] + count * w * 2))
                spans.sort()
                assert spans[0][0] == 0 and spans[-1][1] == world * count * w * 2
                assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
