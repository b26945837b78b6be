"""Times the benchmark configurations other than the decode sweep (which bench.py covers) and prints one JSON line per case.

    python -m kyojin_mac_b200.measure cfg0            # Q4_K GEMV 4096 x 4096, M = 1 (weights rotate through copies larger than L2)
    python -m kyojin_mac_b200.measure cfg2            # Q3_K prefill GEMM, M = 2048, 3072 -> 12288 and 12288 -> 3072
    python -m kyojin_mac_b200.measure cfg3            # NVFP4 prefill GEMM, 4096 x 7168 -> 18432, activations quantised on the fly
    python -m kyojin_mac_b200.measure fp4peak         # the vendor library's block-scaled NVFP4 GEMM (torch._scaled_mm), a measured fp4 denominator
    python -m kyojin_mac_b200.measure cfg4 [E [T ...]]  # routed-expert layer, E (default 256) experts, top-8, hidden 7168, T = 64 and 4096 (or the given token counts)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 -m kyojin_mac_b200.measure dist
                                                      # cfg 2 / 3 N-sharded with all-gather, cfg 4 expert-parallel with all-to-all, on N GPUs

Device time by CUDA events on the current stream, after warm-up, minimum and median over the repetitions. Synthetic seeded weights."""
import json
import statistics
import sys

import torch

from . import foreign_moe as FM, ops, synth
from .foreign_linear import DevPack, ForeignSwitchGLU

BPW = {"q4_k": 144 / 256, "q6_k": 210 / 256, "q3_k": 110 / 256, "nvfp4": 144 / 256}


def timeit(fn, iters=20, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return min(ts), statistics.median(ts)


def graph_of(fn):
    """One CUDA graph of fn (warm-up on a side stream first, as torch requires)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def cfg0():
    n = k = 4096
    copies = 32                                                             # 32 x 9.4 MB = 302 MB > L2
    ws = [synth.t16_random_device("q4_k", n, k, seed=i) for i in range(copies)]
    x = torch.randn((1, k), device="cuda").to(torch.float16)
    y = torch.empty((1, n), dtype=torch.float16, device="cuda")

    def step():
        for w in ws:
            ops.gemv("q4_k", w, n, k, x, out=y)
    g = graph_of(step)
    lo, med = timeit(g.replay)
    byt = n * k * BPW["q4_k"] + 2 * k + 2 * n
    print(json.dumps({"case": "cfg0 q4_k gemv 4096x4096 m=1", "us_per_launch_min": lo / copies, "us_per_launch_median": med / copies, "GBps": byt * copies / med / 1e3,
                      "launches_per_graph": copies, "plan": ops.gemv_plan("q4_k", n, k, 1)}), flush=True)


def cfg2():
    m = 2048
    for n, k in ((12288, 3072), (3072, 12288)):
        dp = DevPack.from_t16("q3_k", synth.t16_random_device("q3_k", n, k, seed=2), n, k)
        x = torch.randn((m, k), device="cuda").to(torch.float16)
        w16 = dp.dequant()
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        fl = 2.0 * m * n * k
        t_d = timeit(lambda: dp.dequant())[1]
        t_g = timeit(lambda: ops.gemm_f16(x, w16, out=y))[1]
        t_s = timeit(lambda: dp._prefill_two_step(x))[1]
        t_1 = timeit(lambda: ops.gemm_kq("q3_k", dp.t16, n, k, x, out=y, msub=1))[1]
        t_2 = timeit(lambda: ops.gemm_kq("q3_k", dp.t16, n, k, x, out=y, msub=2))[1]
        t_a = timeit(lambda: dp.apply(x))[1]
        print(json.dumps({"case": f"cfg2 q3_k gemm {k}->{n} m={m}", "dequant_us": t_d, "fp16_gemm_us": t_g, "staged_us": t_s, "fused_msub1_us": t_1, "fused_msub2_us": t_2,
                          "apply_us": t_a, "fp16_gemm_TFLOPs": fl / t_g / 1e6, "staged_TFLOPs": fl / t_s / 1e6, "fused_msub1_TFLOPs": fl / t_1 / 1e6,
                          "fused_msub2_TFLOPs": fl / t_2 / 1e6, "apply_TFLOPs": fl / t_a / 1e6}), flush=True)


def cfg3():
    n, k, m = 18432, 7168, 4096
    dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", n, k, seed=3), n, k)
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    qs, sfb = dp._a4_operands()
    ac, _, asw = ops.nvfp4_quant_rows(x, True, False)
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    fl = 2.0 * m * n * k
    t_q = timeit(lambda: ops.nvfp4_quant_rows(x, True, False))[1]
    t_g = timeit(lambda: ops.gemm_nvfp4(ac, asw, qs, sfb, m, n, k, 1.0, out=y))[1]
    t_a = timeit(lambda: dp.apply_a4(x, torch.bfloat16))[1]
    print(json.dumps({"case": "cfg3 nvfp4 gemm 7168->18432 m=4096", "quant_us": t_q, "gemm_us": t_g, "apply_us": t_a, "gemm_TFLOPs": fl / t_g / 1e6,
                      "apply_TFLOPs": fl / t_a / 1e6, "scale_rule": "e4m3 RNE of 2^U[-8,0]"}), flush=True)


def fp4_library_peak():
    """Block-scaled NVFP4 GEMM of the vendor library through torch._scaled_mm (8192^3, random codes, unit scales) as a measured denominator for the fp4 roofline;
    prints the exception text when this torch build does not expose it."""
    n = 8192
    try:
        a = torch.randint(0, 256, (n, n // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (n, n // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        sa = torch.full((n * n // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        sb = torch.full((n * n // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        f = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
        lo, med = timeit(f)
        print(json.dumps({"case": "library nvfp4 gemm 8192^3 (torch._scaled_mm)", "us_min": lo, "us_median": med, "TFLOPs_best": 2.0 * n ** 3 / lo / 1e6,
                          "TFLOPs_median": 2.0 * n ** 3 / med / 1e6}), flush=True)
    except Exception as e:                                                   # noqa: BLE001 - the probe reports whatever the library says
        print(json.dumps({"case": "library nvfp4 gemm (torch._scaled_mm)", "unavailable": str(e)[:300]}), flush=True)


def cfg4(E=256, Ts=(64, 4096)):
    H, I, K = 7168, 2048, 8
    g = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * I, H, seed=40), I, H, E)
    u = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * I, H, seed=41), I, H, E)
    d = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * H, I, seed=42), H, I, E)
    glu = ForeignSwitchGLU(g, u, d)
    gen = torch.Generator(device="cuda").manual_seed(4)
    gw = torch.randn((E, H), device="cuda", generator=gen) * 0.02
    blk = FM.RoutedBlock(gw, glu, K, True)
    for T in Ts:
        x = torch.randn((T, H), device="cuda", generator=gen).to(torch.float16)
        lg = torch.randn((T, E + 1), device="cuda", generator=gen)           # the benchmark's router logits are N(0, 1) draws
        inds, scs, _ = ops.moe_select(lg, E, K, True)
        touched = int(torch.unique(inds).numel())
        t_sel = timeit(lambda: ops.moe_select(lg, E, K, True))[1]
        t_lg = timeit(lambda: ops.router_logits(x, gw))[1]
        t_mlp = timeit(lambda: glu(x, inds.reshape(T, K)), iters=10)[1]
        y = glu(x, inds.reshape(T, K))
        t_cmb = timeit(lambda: ops.moe_combine(y.reshape(T * K, H), scs, K))[1]
        t_blk = timeit(lambda: blk(x), iters=10)[1]
        rec = {"case": f"cfg4 moe E={E} top{K} H={H} I={I} T={T}", "experts_touched": touched, "router_logits_us": t_lg, "select_us": t_sel, "experts_us": t_mlp, "combine_us": t_cmb,
               "block_us": t_blk}
        if T * K <= max(256, 4 * E):
            byt = touched * 3 * I * H * BPW["q4_k"]
            rec["expert_bytes"] = byt
            rec["experts_GBps"] = byt / t_mlp / 1e3
        else:
            fl = 2.0 * T * K * H * I * 3
            rec["experts_TFLOPs"] = fl / t_mlp / 1e6
            rec["block_TFLOPs"] = fl / t_blk / 1e6
        print(json.dumps(rec), flush=True)


def dist_cases(E=256):
    """Sharded configurations under torchrun (one rank per GPU, NCCL): cfg 2 and cfg 3 column-sharded over N with an all-gather of the output slices, cfg 4
    expert-parallel with all-to-all dispatch and combine. Strong scaling (the problem is fixed, each rank holds 1 / world of the weights). Times are the maximum
    over ranks of CUDA-event durations; rank 0 prints."""
    import os
    import torch.distributed as dist
    from . import dist as D
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def tmax(fn, iters=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e3], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        return statistics.median(ts)

    def say(**kw):
        if rank == 0:
            print(json.dumps(dict(n_gpus=world, **kw)), flush=True)

    m = 2048
    gen = torch.Generator(device="cuda").manual_seed(7)                      # the same activations on every rank
    for n, k in ((12288, 3072), (3072, 12288)):
        row0, rows = D.shard_rows(n, world, rank)
        dp = DevPack.from_t16("q3_k", synth.t16_random_device("q3_k", rows, k, seed=100 + rank), rows, k)
        lin = D.ShardedLinear(dp.apply, n)
        x = torch.randn((m, k), device="cuda", generator=gen).to(torch.float16)
        fused = D.FusedShardedLinear(dp, n, m)
        fused1 = D.FusedShardedLinear(dp, n, m, msub=1)
        t_local, t_all, t_fused, t_fused1 = tmax(lambda: dp.apply(x)), tmax(lambda: lin(x)), tmax(lambda: fused(x)), tmax(lambda: fused1(x))
        same = bool(torch.equal(fused(x), lin(x)))
        fl = 2.0 * m * n * k
        say(case=f"cfg2 q3_k {k}->{n} m={m} N-sharded", local_us=t_local, nccl_allgather_us=t_all, fused_allgather_us=t_fused, fused_msub1_us=t_fused1, local_TFLOPs=fl / t_local / 1e6,
            nccl_allgather_TFLOPs=fl / t_all / 1e6, fused_allgather_TFLOPs=fl / t_fused / 1e6, fused_equals_nccl=same)
    n, k, m = 18432, 7168, 4096
    row0, rows = D.shard_rows(n, world, rank, align=256)
    dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", rows, k, seed=200 + rank), rows, k)
    x = torch.randn((m, k), device="cuda", generator=gen).to(torch.bfloat16)
    lin = D.ShardedLinear(lambda v: dp.apply_a4(v, torch.bfloat16), n)
    fused = D.FusedShardedLinear(dp, n, m, a4=True, out_dtype=torch.bfloat16)
    t_local, t_all, t_fused = tmax(lambda: dp.apply_a4(x, torch.bfloat16)), tmax(lambda: lin(x)), tmax(lambda: fused(x))
    same = bool(torch.equal(fused(x), lin(x)))
    fl = 2.0 * m * n * k
    say(case="cfg3 nvfp4 7168->18432 m=4096 N-sharded", local_us=t_local, nccl_allgather_us=t_all, fused_allgather_us=t_fused, local_TFLOPs=fl / t_local / 1e6,
        nccl_allgather_TFLOPs=fl / t_all / 1e6, fused_allgather_TFLOPs=fl / t_fused / 1e6, fused_equals_nccl=same)
    H, I, K = 7168, 2048, 8
    e0, ne = D.expert_range(E, world, rank)
    mk = lambda rows_, k_, seed: DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", ne * rows_, k_, seed=seed + rank), rows_, k_, ne)
    glu = ForeignSwitchGLU(mk(I, H, 300), mk(I, H, 400), mk(H, I, 500))
    local_experts = lambda rows_, ids: glu(rows_, ids.reshape(-1, 1)).reshape(rows_.shape[0], H)
    for T in (64, 4096):
        Tl = T // world
        g2 = torch.Generator(device="cuda").manual_seed(1000 + rank)
        x = torch.randn((Tl, H), device="cuda", generator=g2).to(torch.float16)
        lg = torch.randn((Tl, E + 1), device="cuda", generator=g2)
        inds, scs, _ = ops.moe_select(lg, E, K, True)
        t = tmax(lambda: D.ep_moe(x, inds.reshape(Tl, K), scs.reshape(Tl, K), E, local_experts, out_dtype=torch.float16), iters=6)
        rec = dict(case=f"cfg4 moe E={E} top{K} T={T} expert-parallel", tokens_per_rank=Tl, layer_us=t)
        if T > 64:
            rec["TFLOPs"] = 2.0 * T * K * H * I * 3 / t / 1e6
        say(**rec)
    torch.cuda.synchronize()
    ops.check_device_status()
    dist.barrier()
    os._exit(0)                                                               # NCCL teardown at interpreter exit hung on the boxes this was developed on


def router(T=4096, E=256, H=7168, iters=10):
    """The fp32 router product alone: x [T, H] fp16 on the gate [E, H] fp32 plus the shared-expert gate row."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((T, H), device="cuda", generator=gen).to(torch.float16)
    gw = torch.randn((E, H), device="cuda", generator=gen) * 0.02
    sgw = torch.randn((H,), device="cuda", generator=gen) * 0.02
    t = timeit(lambda: ops.router_logits(x, gw, sgw), iters=iters)[1]
    print(json.dumps({"case": f"router T={T} E={E} H={H}", "us": t, "fp32_TFLOPs": 2.0 * T * (E + 1) * H / t / 1e6}), flush=True)


def main(argv):
    what = argv[0] if argv else "cfg0"
    if what == "cfg0":
        cfg0()
    elif what == "cfg2":
        cfg2()
    elif what == "cfg3":
        cfg3()
    elif what == "fp4peak":
        fp4_library_peak()
    elif what == "cfg4":
        cfg4(int(argv[1]) if len(argv) > 1 else 256, tuple(int(t) for t in argv[2:]) or (64, 4096))
    elif what == "router":
        router(*(int(a) for a in argv[1:]))
    elif what == "dist":
        dist_cases(int(argv[1]) if len(argv) > 1 else 256)
    else:
        raise SystemExit(f"unknown case {what}")
    torch.cuda.synchronize()
    ops.check_device_status()


if __name__ == "__main__":
    main(sys.argv[1:])
