"""Times the benchmark configurations other than the decode sweep (which bench.py covers) and prints one JSON line per case.

    python -m kyojin_mac_b200.measure cfg0            # Q4_K GEMV 4096 x 4096, M = 1 (weights rotate through copies larger than L2)
    python -m kyojin_mac_b200.measure cfg2            # Q3_K prefill GEMM, M = 2048, 3072 -> 12288 and 12288 -> 3072
    python -m kyojin_mac_b200.measure cfg3            # NVFP4 prefill GEMM, 4096 x 7168 -> 18432, activations quantised on the fly
    python -m kyojin_mac_b200.measure fp4peak         # the vendor library's block-scaled NVFP4 GEMM (torch._scaled_mm), a measured fp4 denominator
    python -m kyojin_mac_b200.measure cfg4 [E [T ...]]  # routed-expert layer, E (default 256) experts, top-8, hidden 7168, T = 64 and 4096 (or the given token counts)
    python -m kyojin_mac_b200.measure gemv q4_k 27648 5120 1   # one decode product a few times (the target of profiler captures)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29511 -m kyojin_mac_b200.measure dist
                                                      # cfg 2 / 3 N-sharded with all-gather, cfg 4 expert-parallel with all-to-all, on N GPUs

Device time by CUDA events on the current stream, after warm-up, minimum and median over the repetitions. Synthetic seeded weights. Every case also
prints the error of its result on a seeded sample against an fp64 product (`parity`) and its roofline fraction; bench.py puts the same records into its line."""
import json
import statistics
import sys

import torch

from . import foreign_moe as FM, ops, synth
from .foreign_linear import DevPack, ForeignSwitchGLU

BPW = {"q4_k": 144 / 256, "q6_k": 210 / 256, "q3_k": 110 / 256, "nvfp4": 144 / 256}


def timeit(fn, iters=20, warm=3, reps=1):
    """(min, median) microseconds per call over `iters` timings, each of `reps` back-to-back calls between two events (reps > 1 takes the launch gap at the head
    of an idle stream out of short kernels' figures)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / reps)
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


def peaks():
    """Measured roofline denominators of this pool's B200s (MEASURED_PEAKS.json beside the package: a copy's HBM GB/s, a dense bf16 GEMM's TFLOP/s as a burst),
    else the stated fallback figures of an earlier measurement."""
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "f16_tflops": float(d["bf16_tflops"]), "source": "measured (MEASURED_PEAKS.json)"}
    except Exception:
        return {"hbm_gbs": 6650.0, "f16_tflops": 1590.0, "source": "fallback (earlier measurement on this pool)"}


def _roof(bound, achieved, peak, unit, source):
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "peak_source": source}


def _rel_fro(got, want):
    return float(torch.linalg.norm(got.double() - want.double()) / torch.linalg.norm(want.double()))


_PARITY_NOTE = "fp64 product on the device of the same activations and this library's fp32 decode of the weights (the decoder is pinned bit-exactly on the golden vectors by the tests)"


def cfg0():
    """Q4_K GEMV 4096 x 4096, M = 1: a CUDA graph of 32 chained products over 32 weight copies (302 MB, larger than L2)."""
    n = k = 4096
    copies = 32
    ws = [synth.t16_random_device("q4_k", n, k, seed=i) for i in range(copies)]
    x = torch.randn((1, k), device="cuda").to(torch.float16)
    y = torch.empty((1, n), dtype=torch.float16, device="cuda")
    err = _rel_fro(ops.gemv("q4_k", ws[0], n, k, x), x.double() @ ops.dequant("q4_k", ws[0], n, k, torch.float32).double().T)

    def step():
        for w in ws:
            ops.gemv("q4_k", w, n, k, x, out=y, chained=True)
    g = graph_of(step)
    lo, med = timeit(g.replay)
    byt = n * k * BPW["q4_k"] + 2 * k + 2 * n
    pk = peaks()
    return [{"case": "cfg0 q4_k gemv 4096x4096 m=1", "value": byt * copies / med / 1e3, "unit": "GB/s", "us_per_launch": med / copies, "us_per_launch_min": lo / copies,
             "launches_per_graph": copies, "plan": ops.gemv_plan("q4_k", n, k, 1), "roofline": _roof("hbm", byt * copies / med / 1e3, pk["hbm_gbs"], "GB/s", pk["source"]),
             "parity": {"rel_fro": err, "against": _PARITY_NOTE}}]


def cfg2(extra=False):
    """Q3_K prefill GEMM at hidden 3072, M = 2048, both shapes, weights decoded inside the tcgen05 GEMM."""
    m, out, pk = 2048, [], peaks()
    for n, k in ((12288, 3072), (3072, 12288)):
        dp = DevPack.from_t16("q3_k", synth.t16_random_device("q3_k", n, k, seed=2), n, k)
        x = torch.randn((m, k), device="cuda").to(torch.float16)
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
        fl = 2.0 * m * n * k
        t_a = timeit(lambda: dp.apply(x), reps=4)[1]
        rows = torch.randperm(n, device="cuda")[:256]
        w32 = ops.dequant("q3_k", dp.t16, n, k, torch.float32)[rows]
        err = _rel_fro(dp.apply(x)[:, rows], x.double() @ w32.double().T)
        rec = {"case": f"cfg2 q3_k gemm {k}->{n} m={m}", "value": fl / t_a / 1e6, "unit": "TFLOP/s", "us": t_a,
               "roofline": _roof("tensor", fl / t_a / 1e6, pk["f16_tflops"], "TFLOP/s", pk["source"] + ": dense bf16 GEMM, burst"),
               "parity": {"rel_fro": err, "sample": "256 output columns x all 2048 rows", "against": _PARITY_NOTE}}
        if extra:
            w16 = dp.dequant()
            rec.update(dequant_us=timeit(lambda: dp.dequant(), reps=4)[1], fp16_gemm_us=timeit(lambda: ops.gemm_f16(x, w16, out=y), reps=4)[1],
                       staged_us=timeit(lambda: dp._prefill_two_step(x), reps=4)[1], fused_pair_us=timeit(lambda: ops.gemm_kq("q3_k", dp.t16, n, k, x, out=y), reps=4)[1],
                       fused_one_cta_msub1_us=timeit(lambda: ops.gemm_kq("q3_k", dp.t16, n, k, x, out=y, msub=1), reps=4)[1],
                       fused_one_cta_msub2_us=timeit(lambda: ops.gemm_kq("q3_k", dp.t16, n, k, x, out=y, msub=2), reps=4)[1])
        out.append(rec)
    return out


def fp4_library_peak():
    """Block-scaled NVFP4 GEMM of the vendor library through torch._scaled_mm (8192^3, random codes, unit scales) as a measured denominator for the fp4 roofline;
    returns the exception text when this torch build does not expose it."""
    n = 8192
    try:
        a = torch.randint(0, 256, (n, n // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (n, n // 2), dtype=torch.uint8, device="cuda").view(torch.float4_e2m1fn_x2)
        sa = torch.full((n * n // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        sb = torch.full((n * n // 16,), 1.0, device="cuda").to(torch.float8_e4m3fn)
        f = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
        lo, med = timeit(f)
        return {"case": "library nvfp4 gemm 8192^3 (torch._scaled_mm)", "us_min": lo, "us_median": med, "TFLOPs_best": 2.0 * n ** 3 / lo / 1e6, "TFLOPs_median": 2.0 * n ** 3 / med / 1e6}
    except Exception as e:                                                   # noqa: BLE001 - the probe reports whatever the library says
        return {"case": "library nvfp4 gemm (torch._scaled_mm)", "unavailable": str(e)[:300]}


def cfg3():
    """NVFP4 W4A4 prefill GEMM 4096 x 7168 -> 18432: GEMM alone and with the activation quantiser. Denominator: the vendor library's block-scaled GEMM measured in
    the same run (nominal dense fp4 figure when that is unavailable)."""
    n, k, m = 18432, 7168, 4096
    dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", n, k, seed=3), n, k)
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    qs, sfb = dp._a4_operands()
    ac, ap, asw = ops.nvfp4_quant_rows(x, True, True)
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    fl = 2.0 * m * n * k
    t_q = timeit(lambda: ops.nvfp4_quant_rows(x, True, False), reps=4)[1]
    t_g = timeit(lambda: ops.gemm_nvfp4(ac, asw, qs, sfb, m, n, k, 1.0, out=y), reps=4)[1]
    t_a = timeit(lambda: dp.apply_a4(x, torch.bfloat16), reps=4)[1]
    lib = fp4_library_peak()
    peak, src = (lib["TFLOPs_best"], "vendor block-scaled NVFP4 GEMM 8192^3 (torch._scaled_mm) measured in this run") if "TFLOPs_best" in lib else (9000.0, "nominal dense fp4 (vendor GEMM unavailable)")
    rows = torch.randperm(n, device="cuda")[:256]
    xq = ops.nvfp4_unpack_rows(ac, ap, torch.float32)
    w32 = ops.dequant("nvfp4", dp.t16, n, k, torch.float32)[rows]
    err = _rel_fro(dp.apply_a4(x, torch.float16)[:, rows], xq.double() @ w32.double().T)
    par = {"rel_fro": err, "sample": "256 output columns x all 4096 rows", "against": "fp64 product on the device of the quantised activations (decoded) and this library's fp32 decode of the weights"}
    return [{"case": "cfg3 nvfp4 w4a4 gemm 7168->18432 m=4096 (GEMM alone)", "value": fl / t_g / 1e6, "unit": "TFLOP/s", "us": t_g, "roofline": _roof("tensor", fl / t_g / 1e6, peak, "TFLOP/s", src),
             "parity": par, "scale_rule": "e4m3 RNE of 2^U[-8,0]"},
            {"case": "cfg3 nvfp4 w4a4 gemm 7168->18432 m=4096 (activation quantiser + GEMM)", "value": fl / t_a / 1e6, "unit": "TFLOP/s", "us": t_a, "quant_us": t_q,
             "roofline": _roof("tensor", fl / t_a / 1e6, peak, "TFLOP/s", src), "parity": par}]


def routed_reference(x, inds, g, u, d, toks):
    """fp64 routed SwiGLU outputs [len(toks) * K, H] of the sampled tokens from this library's fp32 decode of the experts they use (device only), clamped to the
    fp16 range: the kernels saturate at +-65504 as the reference's do, and the synthetic weight scales let a few outputs of a random token exceed it."""
    K = inds.shape[1]
    out = torch.zeros((len(toks) * K, d.n), dtype=torch.float64, device=x.device)
    for i, t in enumerate(toks):
        xt = x[t:t + 1].double()
        for kk in range(K):
            e = int(inds[t, kk])
            wg, wu, wd = (dev.expert(e).dequant(torch.float32).double() for dev in (g, u, d))
            a, b = xt @ wg.T, xt @ wu.T
            out[i * K + kk] = ((a / (1.0 + torch.exp(-a)) * b) @ wd.T)[0]
    return out.clamp(-65504.0, 65504.0)


def cfg4(E=256, Ts=(64, 4096)):
    """Routed-expert layer, E experts, top-8, hidden 7168, expert width 2048, Q4_K: the three expert projections (value) and the whole block (router, experts, combine)."""
    H, I, K = 7168, 2048, 8
    g = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * I, H, seed=40), I, H, E)
    u = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * I, H, seed=41), I, H, E)
    d = DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * H, I, seed=42), H, I, E)
    glu = ForeignSwitchGLU(g, u, d)
    gen = torch.Generator(device="cuda").manual_seed(4)
    gw = torch.randn((E, H), device="cuda", generator=gen) * 0.02
    blk = FM.RoutedBlock(gw, glu, K, True)
    pk, out = peaks(), []
    for T in Ts:
        x = (torch.randn((T, H), device="cuda", generator=gen) * 0.5).to(torch.float16)
        lg = torch.randn((T, E + 1), device="cuda", generator=gen)           # the benchmark's router logits are N(0, 1) draws
        inds, scs, _ = ops.moe_select(lg, E, K, True)
        touched = int(torch.unique(inds).numel())
        t_sel = timeit(lambda: ops.moe_select(lg, E, K, True))[1]
        t_lg = timeit(lambda: ops.router_logits(x, gw))[1]
        t_mlp = timeit(lambda: glu(x, inds.reshape(T, K)), iters=10)[1]
        y = glu(x, inds.reshape(T, K))
        t_cmb = timeit(lambda: ops.moe_combine(y.reshape(T * K, H), scs, K))[1]
        t_blk = timeit(lambda: blk(x), iters=10)[1]
        toks = [0, T // 2, T - 1]
        want = routed_reference(x, inds.reshape(T, K), g, u, d, toks)
        err = _rel_fro(y[toks].reshape(len(toks) * K, H), want)
        rec = {"case": f"cfg4 moe E={E} top{K} H={H} I={I} T={T}", "experts_touched": touched, "router_logits_us": t_lg, "select_us": t_sel, "experts_us": t_mlp, "combine_us": t_cmb,
               "block_us": t_blk, "us": t_mlp,
               "parity": {"rel_fro": err, "sample": "3 tokens x 8 slots x all 7168 columns",
                          "against": "fp64 routed layer on the device from this library's fp32 decode of the experts (two fp16 roundings on the way, as on the reference path: bound 2e-3)"}}
        if T * K <= max(256, 4 * E):
            byt = touched * 3 * I * H * BPW["q4_k"]
            rec.update(value=byt / t_mlp / 1e3, unit="GB/s", expert_bytes=byt, roofline=_roof("hbm", byt / t_mlp / 1e3, pk["hbm_gbs"], "GB/s", pk["source"]))
        else:
            fl = 2.0 * T * K * H * I * 3
            rec.update(value=fl / t_mlp / 1e6, unit="TFLOP/s", block_TFLOPs=fl / t_blk / 1e6,
                       roofline=_roof("tensor", fl / t_mlp / 1e6, pk["f16_tflops"], "TFLOP/s", pk["source"] + ": dense bf16 GEMM, burst"))
        out.append(rec)
    return out


def dist_records(E=256):
    """Sharded configurations on the ranks of an initialised process group (one rank per GPU, NCCL): cfg 2 and cfg 3 column-sharded over N with an all-gather of
    the output slices, cfg 4 expert-parallel with all-to-all dispatch and combine. Strong scaling (the problem is fixed, each rank holds 1 / world of the weights).
    Times are the maximum over ranks of CUDA-event durations. Returns the list of records (the same on every rank)."""
    import torch.distributed as dist
    from . import dist as D
    rank, world = dist.get_rank(), dist.get_world_size()
    pk, recs = peaks(), []

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

    say = lambda **kw: recs.append(dict(n_gpus=world, **kw))
    m = 2048
    gen = torch.Generator(device="cuda").manual_seed(7)                      # the same activations on every rank
    for n, k in ((12288, 3072), (3072, 12288)):
        row0, rows = D.shard_rows(n, world, rank)
        dp = DevPack.from_t16("q3_k", synth.t16_random_device("q3_k", rows, k, seed=100 + rank), rows, k)
        lin = D.ShardedLinear(dp.apply, n)
        x = torch.randn((m, k), device="cuda", generator=gen).to(torch.float16)
        fused = D.FusedShardedLinear(dp, n, m)
        t_local, t_all, t_fused = tmax(lambda: dp.apply(x)), tmax(lambda: lin(x)), tmax(lambda: fused(x))
        # the gather folded into the GEMM against the library all-gather of the SAME local product: the fused kernel does not split k, so the comparison runs
        # with the split-k form off (with it on, the local product of a narrow shard differs from the fused one by fp32 summation order)
        from . import flags as F
        keep, F.GEMM_SPLIT_K = F.GEMM_SPLIT_K, False
        try:
            same = bool(torch.equal(fused(x), lin(x)))
        finally:
            F.GEMM_SPLIT_K = keep
        fl = 2.0 * m * n * k
        say(case=f"cfg2 q3_k {k}->{n} m={m} N-sharded", local_us=t_local, nccl_allgather_us=t_all, fused_allgather_us=t_fused, sharded_output_TFLOPs=fl / t_local / 1e6,
            nccl_allgather_TFLOPs=fl / t_all / 1e6, value=fl / t_fused / 1e6, unit="TFLOP/s", frac_of_n_times_peak=fl / t_fused / 1e6 / (world * pk["f16_tflops"]),
            gather_floor_us=(world - 1) / world * m * n * 2 / 770e3, fused_equals_nccl=same)
        del fused, lin, dp
    n, k, m = 18432, 7168, 4096
    row0, rows = D.shard_rows(n, world, rank, align=256)
    dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", rows, k, seed=200 + rank), rows, k)
    x = torch.randn((m, k), device="cuda", generator=gen).to(torch.bfloat16)
    lin = D.ShardedLinear(lambda v: dp.apply_a4(v, torch.bfloat16), n)
    fused = D.FusedShardedLinear(dp, n, m, a4=True, out_dtype=torch.bfloat16)
    t_local, t_all, t_fused = tmax(lambda: dp.apply_a4(x, torch.bfloat16)), tmax(lambda: lin(x)), tmax(lambda: fused(x))
    same = bool(torch.equal(fused(x), lin(x)))
    fl = 2.0 * m * n * k
    say(case="cfg3 nvfp4 7168->18432 m=4096 N-sharded", local_us=t_local, nccl_allgather_us=t_all, fused_allgather_us=t_fused, sharded_output_TFLOPs=fl / t_local / 1e6,
        nccl_allgather_TFLOPs=fl / t_all / 1e6, value=fl / t_fused / 1e6, unit="TFLOP/s", gather_floor_us=(world - 1) / world * m * n * 2 / 770e3, fused_equals_nccl=same)
    del fused, lin, dp
    torch.cuda.empty_cache()
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
        t = tmax(lambda: D.ep_moe(x, inds.reshape(Tl, K), scs.reshape(Tl, K), E, local_experts, out_dtype=torch.float16, slot_dtype=torch.float16, slot_width=H), iters=6)
        rec = dict(case=f"cfg4 moe E={E} top{K} T={T} expert-parallel", tokens_per_rank=Tl, layer_us=t)
        if T > 64:
            rec.update(value=2.0 * T * K * H * I * 3 / t / 1e6, unit="TFLOP/s")
        say(**rec)
    torch.cuda.synchronize()
    ops.check_device_status()
    return recs


def dist_cases(E=256):
    """dist_records under torchrun: sets the process group up, prints the records on rank 0 and leaves."""
    import os
    import torch.distributed as dist
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    recs = dist_records(E)
    if rank == 0:
        for r in recs:
            print(json.dumps(r), flush=True)
    dist.barrier()
    os._exit(0)                                                               # NCCL teardown at interpreter exit hung on the boxes this was developed on


def router(T=4096, E=256, H=7168, iters=10):
    """The router product alone, x [T, H] fp16 on the gate [E, H] fp32 plus the shared-expert gate row: the fp32 kernels and the tensor-core form."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((T, H), device="cuda", generator=gen).to(torch.float16)
    gw = torch.randn((E, H), device="cuda", generator=gen) * 0.02
    sgw = torch.randn((H,), device="cuda", generator=gen) * 0.02
    t32 = timeit(lambda: ops.router_logits(x, gw, sgw, tensor_cores=False), iters=iters)[1]
    ttc = timeit(lambda: ops.router_logits(x, gw, sgw, tensor_cores=True), iters=iters)[1]
    want = x.double() @ torch.cat([gw, sgw[None]]).double().T
    err = lambda lg: float((lg.double() - want).norm() / want.norm())
    print(json.dumps({"case": f"router T={T} E={E} H={H}", "fp32_kernel_us": t32, "tensor_core_us": ttc, "fp32_kernel_TFLOPs": 2.0 * T * (E + 1) * H / t32 / 1e6,
                      "rel_fro_fp32_kernel": err(ops.router_logits(x, gw, sgw, tensor_cores=False)),
                      "rel_fro_tensor_core": err(ops.router_logits(x, gw, sgw, tensor_cores=True))}), flush=True)


def main(argv):
    what = argv[0] if argv else "cfg0"
    say = lambda recs: [print(json.dumps(r), flush=True) for r in (recs if isinstance(recs, list) else [recs])]
    if what == "cfg0":
        say(cfg0())
    elif what == "cfg2":
        say(cfg2(extra=True))
    elif what == "cfg3":
        say(cfg3())
    elif what == "fp4peak":
        say(fp4_library_peak())
    elif what == "cfg4":
        say(cfg4(int(argv[1]) if len(argv) > 1 else 256, tuple(int(t) for t in argv[2:]) or (64, 4096)))
    elif what == "router":
        router(*(int(a) for a in argv[1:]))
    elif what == "gemv":                                                      # gemv <fmt> <n> <k> <m>: one decode product a few times (profiler target)
        fmt, n, k, m = argv[1], int(argv[2]), int(argv[3]), int(argv[4])
        t16 = synth.t16_random_device(fmt, n, k, seed=0)
        x = torch.randn((m, k), device="cuda").to(torch.float16)
        for _ in range(int(argv[5]) if len(argv) > 5 else 3):
            y = ops.gemv(fmt, t16, n, k, x)
        print(json.dumps({"case": f"gemv {fmt} {n}x{k} m={m}", "plan": ops.gemv_plan(fmt, n, k, m), "mean_abs": float(y.float().abs().mean())}), flush=True)
    elif what == "gemm_kq":                                                   # gemm_kq <fmt> <n> <k> <m> [msub]: one prefill product a few times (profiler target)
        fmt, n, k, m = argv[1], int(argv[2]), int(argv[3]), int(argv[4])
        t16 = synth.t16_random_device(fmt, n, k, seed=0)
        x = torch.randn((m, k), device="cuda").to(torch.float16)
        for _ in range(3):
            y = ops.gemm_kq(fmt, t16, n, k, x, msub=int(argv[5]) if len(argv) > 5 else 0)
        print(json.dumps({"case": f"gemm_kq {fmt} {n}x{k} m={m}", "mean_abs": float(y.float().abs().mean())}), flush=True)
    elif what == "gemm_a4":                                                   # gemm_a4 <n> <k> <m>: activation quantiser + NVFP4 GEMM a few times (profiler target)
        n, k, m = int(argv[1]), int(argv[2]), int(argv[3])
        dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", n, k, seed=0), n, k)
        x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        for _ in range(3):
            y = dp.apply_a4(x)
        print(json.dumps({"case": f"gemm_a4 nvfp4 {n}x{k} m={m}", "mean_abs": float(y.float().abs().mean())}), flush=True)
    elif what == "dist":
        dist_cases(int(argv[1]) if len(argv) > 1 else 256)
    else:
        raise SystemExit(f"unknown case {what}")
    torch.cuda.synchronize()
    ops.check_device_status()


if __name__ == "__main__":
    main(sys.argv[1:])
