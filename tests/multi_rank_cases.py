"""Body of tests/test_gpu_multi.py: run under torchrun with one rank per GPU."""
import os

import numpy as np
import torch
import torch.distributed as dist

from kyojin_mac_b200 import dist as D, ops, synth
from kyojin_mac_b200.foreign_linear import DevPack, ForeignSwitchGLU


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # ---- N-sharded linear: fused all-gather == NCCL all-gather == unsharded product (every rank builds the full matrix from the same seed)
    n, k, m = 1536, 1024, 300
    full = synth.t16_random_device("q4_k", n, k, seed=3)
    t16, row0, rows = D.shard_t16("q4_k", full, n, k, world, rank)
    dp = DevPack.from_t16("q4_k", t16.clone(), rows, k)
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    want = DevPack.from_t16("q4_k", full, n, k).apply(x)
    nccl = D.ShardedLinear(dp.apply, n)(x)
    fused = D.FusedShardedLinear(dp, n, 512)
    for _ in range(3):                                                       # both buffers, and a reuse
        got = fused(x)
        assert torch.equal(got, want), "fused all-gather differs from the unsharded product"
    assert torch.equal(nccl, want), "NCCL all-gather differs from the unsharded product"
    # ---- decode: the slices of several products gathered with one copy launch + one barrier
    shapes = [(1, 512), (4, 512), (8, 256)]
    pgather = D.PeerGather(shapes, x.device)
    for it in range(3):
        outs = [torch.full(sh, float(rank * 10 + i + it), dtype=torch.float16, device="cuda") for i, sh in enumerate(shapes)]
        pgather(outs)
        for i, sh in enumerate(shapes):
            got_i = pgather.gathered(i)
            for r in range(world):
                assert torch.all(got_i[r] == float(r * 10 + i + it)), "peer gather: wrong slice"
    # ---- the same gather in stages: parts of a step sent early on a second stream, one barrier at the end
    side = torch.cuda.Stream()
    for it in range(3):
        outs = [torch.full(sh, float(rank * 10 + i + it + 100), dtype=torch.float16, device="cuda") for i, sh in enumerate(shapes)]
        pgather.begin()
        main = torch.cuda.current_stream()
        for part in ([2], [0, 1]):
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ev)
                pgather.store(part, [outs[i] for i in part])
        main.wait_stream(side)
        pgather.finish()
        for i, sh in enumerate(shapes):
            got_i = pgather.gathered(i)
            for r in range(world):
                assert torch.all(got_i[r] == float(r * 10 + i + it + 100)), "staged peer gather: wrong slice"
    # ---- NVFP4 W4A4 shard
    n4 = 512 * world
    full4 = synth.t16_random_device("nvfp4", n4, k, seed=4)
    t4, r0, rws = D.shard_t16("nvfp4", full4, n4, k, world, rank)
    assert rws % 256 == 0
    dp4 = DevPack.from_t16("nvfp4", t4.clone(), rws, k)
    want4 = DevPack.from_t16("nvfp4", full4, n4, k).apply_a4(x.to(torch.bfloat16), torch.bfloat16)
    got4 = D.FusedShardedLinear(dp4, n4, 512, a4=True, out_dtype=torch.bfloat16)(x.to(torch.bfloat16))
    assert torch.equal(got4, want4), "fused NVFP4 all-gather differs from the unsharded product"
    # ---- expert parallelism: each rank owns E / world experts; tokens split over ranks; result == single-GPU layer on the same tokens
    E, K, H, I, T = 8, 2, 512, 256, 40
    stacks = [synth.t16_random_device("q4_k", E * nn, kk, seed=s) for nn, kk, s in ((I, H, 20), (I, H, 21), (H, I, 22))]
    whole = ForeignSwitchGLU(DevPack.from_t16("q4_k", stacks[0], I, H, E), DevPack.from_t16("q4_k", stacks[1], I, H, E), DevPack.from_t16("q4_k", stacks[2], H, I, E))
    e0, ne = D.expert_range(E, world, rank)
    cut = lambda t, nn, kk: t[e0 * ops.t16_nbytes("q4_k", nn, kk):(e0 + ne) * ops.t16_nbytes("q4_k", nn, kk)].clone()
    mine = ForeignSwitchGLU(DevPack.from_t16("q4_k", cut(stacks[0], I, H), I, H, ne), DevPack.from_t16("q4_k", cut(stacks[1], I, H), I, H, ne),
                            DevPack.from_t16("q4_k", cut(stacks[2], H, I), H, I, ne))
    xs = (torch.randn((T, H), device="cuda", generator=g) * 0.5).to(torch.float16)
    lg = torch.randn((T, E + 1), device="cuda", generator=g)
    inds, scs, _ = ops.moe_select(lg, E, K, True)
    inds, scs = inds.reshape(T, K), scs.reshape(T, K)
    ref = ops.moe_combine(whole(xs, inds).reshape(T * K, H), scs.reshape(-1).contiguous(), K, dtype=torch.float32)
    lo, hi = rank * T // world, (rank + 1) * T // world
    local_experts = lambda rows_, ids: mine(rows_, ids.reshape(-1, 1)).reshape(rows_.shape[0], H)
    out = D.ep_moe(xs[lo:hi], inds[lo:hi], scs[lo:hi], E, local_experts, out_dtype=torch.float32)
    assert torch.allclose(out, ref[lo:hi], rtol=1e-3, atol=1e-3), "expert-parallel layer differs from the single-GPU layer"
    torch.cuda.synchronize()
    ops.check_device_status()
    dist.barrier()
    if rank == 0:
        print("MULTI_RANK_OK", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
