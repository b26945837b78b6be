"""Sharding and expert-parallel index logic on CPU ranks (gloo, world size 2 and 3): n-sharded gather == the unsharded product bit for bit, expert-parallel
layer == the single-process layer, uneven expert / row splits included. The reference has no multi-device code; this covers the new design of dist.py."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kyojin_mac_b200 import dist as KD


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _expert_fn(rows, ids, scale=1.0):
    """A stand-in expert stack: expert j multiplies by (j + 1) and adds j (deterministic, differs per expert)."""
    j = ids.to(torch.float32).unsqueeze(1)
    return rows.to(torch.float32) * (j + 1.0) * scale + j


def _worker(rank, world, port, E):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        # ---- dense: W [n, k] sharded by rows
        n, k, m = 80, 32, 3                                                  # 5 tiles of 16 rows: uneven over 2 or 3 ranks
        W = torch.randn((n, k), generator=g)
        x = torch.randn((m, k), generator=g)
        row0, rows = KD.shard_rows(n, world, rank)
        lin = KD.ShardedLinear(lambda a: a @ W[row0:row0 + rows].T, n)
        assert torch.equal(lin(x), x @ W.T)
        n2 = 16 * world * 2                                                  # equal shards: the single all-gather path
        W2 = torch.randn((n2, k), generator=g)
        r0, rr = KD.shard_rows(n2, world, rank)
        assert torch.equal(KD.ShardedLinear(lambda a: a @ W2[r0:r0 + rr].T, n2)(x), x @ W2.T)
        # ---- experts: every rank has its own tokens
        T, K, H = 5 + rank, 3, 8
        gr = torch.Generator().manual_seed(10 + rank)
        xt = torch.randn((T, H), generator=gr)
        inds = torch.stack([torch.randperm(E, generator=gr)[:K] for _ in range(T)])
        scs = torch.rand((T, K), generator=gr)
        e0, ne = KD.expert_range(E, world, rank)
        got = KD.ep_moe(xt, inds, scs, E, lambda rws, ids: _expert_fn(rws, ids + e0))
        want = sum(scs[:, kk:kk + 1] * _expert_fn(xt, inds[:, kk]) for kk in range(K))
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
        # ---- a rank that receives no slot (every token routed to rank 0's experts), expert outputs narrower and of another type than x
        xt64 = xt.to(torch.float64)
        ne0 = KD.expert_range(E, world, 0)[1]
        inds0 = torch.stack([torch.randperm(ne0, generator=gr)[:2] for _ in range(T)])
        scs0 = torch.rand((T, 2), generator=gr)
        half = lambda rws, ids: _expert_fn(rws, ids + e0)[:, :H // 2].contiguous()          # float32 [S, H / 2] from float64 rows
        got0 = KD.ep_moe(xt64, inds0, scs0, E, half, slot_dtype=torch.float32, slot_width=H // 2)
        want0 = sum(scs0[:, kk:kk + 1] * _expert_fn(xt64, inds0[:, kk])[:, :H // 2] for kk in range(2))
        torch.testing.assert_close(got0, want0.to(torch.float32), rtol=1e-6, atol=1e-6)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E", [(2, 8), (3, 7)])
def test_sharding_and_expert_parallel_on_cpu_ranks(world, E):
    mp.spawn(_worker, args=(world, _free_port(), E), nprocs=world, join=True)


def test_shard_rows_cover_every_tile_once():
    for n, world in [(27648, 8), (1024, 8), (80, 3), (16, 4), (5120, 8)]:
        spans = [KD.shard_rows(n, world, r) for r in range(world)]
        assert sum(s[1] for s in spans) == n
        pos = 0
        for r0, rows in spans:
            assert r0 == pos or rows == 0
            assert r0 % 16 == 0
            pos += rows


def test_owner_matches_expert_range():
    for E, world in [(256, 8), (7, 3), (10, 4)]:
        own = KD.owner_of(torch.arange(E), E, world)
        for r in range(world):
            e0, ne = KD.expert_range(E, world, r)
            assert (own[e0:e0 + ne] == r).all()
