"""Benchmark of the dequant-fused quantized linear on B200: decode GEMV sweep over the layer shapes of a 32B-class dense transformer.

Workload (the benchmark's second configuration): hidden 5120, 64 query / 8 KV heads of dim 128, MLP 27648. Projections q 5120->8192,
k and v 5120->1024, o 8192->5120, gate/up 5120->27648 in Q4_K, down 27648->5120 in Q6_K; activations fp16 N(0, 1) at batch
M = 1, 2, 4, 8. One step = one pass over the layer at each of the four batch sizes. Weights are seeded synthetic blocks (random
payload bytes, fp16 d/dmin = |N(0, 1e-3)|, Q6_K scales U[-32, 31]) because no model file is available offline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-group] [--no-configs]

Prints ONE JSON line (rank 0). `value` = GGUF weight bytes + activation bytes moved per second with everything resident in HBM (one
CUDA graph per step); `e2e` = the same through the module API with host activations (pinned h2d, d2h of the results inside the timed
region); `configs` = the other benchmark configurations (Q4_K GEMV 4096^2, Q3_K prefill GEMM, NVFP4 W4A4 GEMM, routed-expert layer at 64 and
4096 tokens), each with its own roofline fraction and the error of its result on a seeded sample against an fp64 product.
N > 1: `value` is weak scaling (every rank holds a full layer-sized shard of an N-times wider layer, output dimension column-sharded, slices
gathered over NVLink); `strong` holds the fixed-size configurations split over the N GPUs (the layer at its stated width N-sharded, the prefill GEMMs
N-sharded with the all-gather folded into the GEMM, the routed layer expert-parallel).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HID, QDIM, KVDIM, MLP = 5120, 8192, 1024, 27648
# name, format, n (out), k (in), same-input group
MATRICES = [("q", "q4_k", QDIM, HID, "qkv"), ("k", "q4_k", KVDIM, HID, "qkv"), ("v", "q4_k", KVDIM, HID, "qkv"), ("o", "q4_k", HID, QDIM, "o"),
            ("gate", "q4_k", MLP, HID, "gateup"), ("up", "q4_k", MLP, HID, "gateup"), ("down", "q6_k", HID, MLP, "down")]
BATCHES = (1, 2, 4, 8)
BPW = {"q4_k": 144 / 256, "q6_k": 210 / 256, "q3_k": 110 / 256, "nvfp4": 144 / 256}
METRIC = "quant GEMV GB/s (% HBM peak)"


# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes in the ncu capture of this kernel on the 27648 x 5120 Q4_K matrix, M = 1 (half of the
# benchmark's gate|up launch; traffic grows with the rows): 79.73 MB over 79.64 MB
NCU_TRAFFIC_RATIO = 1.0011
NCU_TRAFFIC_NOTE = "ncu capture of gemv_t16_kernel on 27648 x 5120 (profiles/gemv_q4k_27648x5120_m1_ncu.md), scaled to this launch by its rows"


def alg_bytes(fmt, n, k, m):
    """Algorithmic bytes of one GEMV: stored weight bytes + fp16 activations in + fp16 results out."""
    return n * k * BPW[fmt] + 2 * m * k + 2 * m * n


def layer_list(group: bool):
    """[(name, fmt, n, k)] of the launches of one layer pass; same-input projections concatenated along n when `group`
    (the reference runs q|k|v and gate|up as one product: kyojin_mlx/foreign_linear.py:1617-1655 group_same_input)."""
    if not group:
        return [(nm, f, n, k) for nm, f, n, k, _ in MATRICES]
    out, seen = [], {}
    for nm, f, n, k, g in MATRICES:
        if g in seen:
            i = seen[g]
            out[i] = (out[i][0] + "|" + nm, f, out[i][2] + n, k)
        else:
            seen[g] = len(out)
            out.append((nm, f, n, k))
    return out


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()                      # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx = max(mx, int(f[1]) if f[1].isdigit() else 0)
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------ CPU arm
def cpu_sample(row_frac=4, m=8, seed=1):
    """The reference's CPU path (its numpy dequantiser on min(8, cores) threads, then a float32 matmul: kyojin_mlx/foreign_gguf.py:376-394 +
    foreign_linear.py:710) on a bounded sample of the workload: every matrix of the layer with 1/row_frac of its rows, batch m.
    Returns (one_pass, bytes per pass, sample text, kind, implementation text)."""
    from oracle import ref_cpu                              # CPU baseline leg: the reference's own decoder when its package is installed beside the repo, else the port
    from kyojin_mac_b200 import synth
    linear, kind, impl = ref_cpu.linear_cpu()
    rng = np.random.default_rng(seed)
    cases = []
    for nm, f, n, k, _ in MATRICES:
        ns = max(16, n // row_frac)
        cases.append((f, ns, k, synth.raw_blocks(f, ns, k, rng), synth.activations(m, k, rng)))
    nbytes = sum(alg_bytes(f, ns, k, m) for f, ns, k, _, _ in cases)
    T = {"q4_k": "Q4_K", "q6_k": "Q6_K"}

    def one_pass():
        t0 = time.perf_counter()
        for f, ns, k, raw, x in cases:
            linear(T[f], raw, k, x)
        return time.perf_counter() - t0

    return one_pass, nbytes, f"every matrix of the layer at 1/{row_frac} of its rows, M={m}, dequant-then-matmul per call", kind, impl


def run_reference(args):
    """The reference's CPU implementation of the path on this box's host cores, on the GPU arm's metric and workload; every step is the bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    one_pass, nbytes, sample, kind, impl = cpu_sample()
    for _ in range(args.warmup):
        one_pass()
    ts = [one_pass() for _ in range(args.steps)]
    t = float(np.mean(ts))
    gbs = nbytes / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "cfg1: decode GEMV sweep over a 32B-class layer (q,k,v,o,gate,up Q4_K; down Q6_K), M=1,2,4,8 per step", "sample": sample,
                       "note": "CPU arm: one step = the bounded sample; one process on rank 0 at every N"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": min(8, cores), "kind": kind, "sample": sample, "host_cores": cores,
                             "note": impl + "; dequant threads = min(8, cores) as the reference, BLAS threads = numpy default"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------ GPU arm
class Sweep:
    """The decode sweep over one list of products [(name, fmt, n, k)] at M = 1, 2, 4, 8: two layer copies of seeded synthetic T16 weights alternate (one layer
    exceeds L2), one CUDA graph per copy holds the chained launches of a step, and with more than one rank the step ends with the peer gather of its outputs."""

    def __init__(self, mats, dev, world, rank, seed0, nccl_gather=False, staged_gather=True):
        import torch
        from kyojin_mac_b200 import synth
        from kyojin_mac_b200.foreign_linear import DevPack
        self.mats, self.dev, self.world, self.rank = mats, dev, world, rank
        self.staged_gather = staged_gather
        self.copies = 2
        self.layers = [[DevPack.from_t16(f, synth.t16_random_device(f, n, k, seed=seed0 + 1000 * rank + 10 * c + i, device=dev), n, k) for i, (nm, f, n, k) in enumerate(mats)]
                       for c in range(self.copies)]
        gen = torch.Generator(device=dev).manual_seed(7 + rank)
        self.xs = {(m, k): torch.randn((m, k), device=dev, generator=gen).to(torch.float16) for m in BATCHES for k in sorted({k for _, _, _, k in mats})}
        self.ys = {(m, i): torch.empty((m, n), dtype=torch.float16, device=dev) for m in BATCHES for i, (_, _, n, _) in enumerate(mats)}
        self.yg = {(m, i): torch.empty((world * m, n), dtype=torch.float16, device=dev) for m in BATCHES for i, (_, _, n, _) in enumerate(mats)} if world > 1 else None
        self.step_bytes = sum(alg_bytes(f, n, k, m) for m in BATCHES for _, f, n, k in mats)
        self.order = [(m, i) for m in BATCHES for i in range(len(mats))]
        self.pg = None
        if world > 1 and not nccl_gather:
            from kyojin_mac_b200.dist import PeerGather
            try:
                self.pg = PeerGather([tuple(self.ys[key].shape) for key in self.order], dev)
            except Exception as e:
                if rank == 0:
                    print(f"[bench] symmetric memory unavailable ({type(e).__name__}: {e}); NCCL all-gathers", file=sys.stderr)
        self.graphs = None
        if self.pg is not None:
            import torch
            self.side = torch.cuda.Stream(device=dev)

    def one_step(self, c):
        import torch.distributed as dist
        from kyojin_mac_b200 import ops
        layer, works = self.layers[c], []
        if self.pg is not None and self.staged_gather:
            # the outputs of a batch size leave for the other ranks on a second stream while the products of the next batch size run; the largest batch goes first,
            # so what is left exposed at the end of the step is the smallest transfer and the one barrier
            import torch
            main = torch.cuda.current_stream()
            self.pg.begin()
            for m in sorted(BATCHES, reverse=True):
                idx = [j for j, (mm, _) in enumerate(self.order) if mm == m]
                for i, (nm, f, n, k) in enumerate(self.mats):
                    ops.gemv(f, layer[i].t16, n, k, self.xs[(m, k)], 1.0, out=self.ys[(m, i)], chained=True)
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(self.side):
                    self.side.wait_event(ev)
                    self.pg.store(idx, [self.ys[self.order[j]] for j in idx])
            main.wait_stream(self.side)
            self.pg.finish()
            return
        for m in BATCHES:
            for i, (nm, f, n, k) in enumerate(self.mats):
                ops.gemv(f, layer[i].t16, n, k, self.xs[(m, k)], 1.0, out=self.ys[(m, i)], chained=True)      # the weights were generated long before: chained launches
                if self.world > 1 and self.pg is None:               # gathers run on NCCL's stream and overlap the following products; joined at the end of the step
                    works.append(dist.all_gather_into_tensor(self.yg[(m, i)], self.ys[(m, i)], async_op=True))
        for w in works:
            w.wait()
        if self.pg is not None:
            self.pg([self.ys[key] for key in self.order])

    def capture(self):
        import torch
        for c in range(self.copies):
            self.one_step(c)
        torch.cuda.synchronize()
        try:
            graphs = []
            for c in range(self.copies):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.one_step(c)
                graphs.append(g)
            self.graphs = graphs
        except Exception as e:                                        # collectives that cannot be captured: time eager launches instead
            self.graphs = None
            if self.rank == 0:
                print(f"[bench] CUDA graph capture unavailable ({type(e).__name__}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()

    def run_step(self, s):
        if self.graphs is not None:
            self.graphs[s % self.copies].replay()
        else:
            self.one_step(s % self.copies)

    def timed(self, steps, warmup, barrier):
        """ms per step: device time between two events around `steps` steps, maximum over ranks."""
        import torch
        import torch.distributed as dist
        for s in range(warmup):
            self.run_step(s)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(steps):
            self.run_step(s)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def dominant_launch_us(self, reps=4):
        """Average duration of the largest product's launch per batch size: a CUDA graph of 2 * reps chained launches of that product alone, alternating the two
        layer copies (each copy of that matrix exceeds L2), events around the replay."""
        import torch
        from kyojin_mac_b200 import ops
        dom = max(range(len(self.mats)), key=lambda i: self.mats[i][2] * self.mats[i][3] * BPW[self.mats[i][1]])
        nm, f, n, k = self.mats[dom]
        per_m = {}
        for m in BATCHES:
            def body():
                for r in range(reps):
                    for c in range(self.copies):
                        ops.gemv(f, self.layers[c][dom].t16, n, k, self.xs[(m, k)], 1.0, out=self.ys[(m, dom)], chained=True)
            body()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                body()
            ts = []
            for _ in range(6):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / (reps * self.copies))
            per_m[m] = float(np.mean(ts[1:]))
        return dom, per_m


def run_ours(args):
    import torch
    import torch.distributed as dist
    from kyojin_mac_b200 import ops
    from kyojin_mac_b200.foreign_linear import ForeignLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    mats = layer_list(not args.no_group)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: weak scaling (every rank streams a full layer-sized shard), one CUDA graph per layer copy, device-timed
    sw = Sweep(mats, dev, world, rank, seed0=0, nccl_gather=args.nccl_gather, staged_gather=not args.end_gather)
    sw.capture()
    for s in range(args.warmup):
        sw.run_step(s)
    with ClockSampler(local) as clk:
        time.sleep(0.25)
        ms_per_step = sw.timed(args.steps, 0, barrier)
        # the timed region lasts a few milliseconds, less than one sampling period: the same steps keep running (untimed, the same count on every rank: a step
        # holds a cross-rank barrier) for about another second so that the clock record holds samples taken under this load
        n_load = 2000
        for s in range(n_load):
            sw.run_step(s)
            if s % 100 == 99:
                torch.cuda.synchronize()
        barrier()
    ops.check_device_status()
    step_bytes = sw.step_bytes
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    launches_per_step = sum(1 + (ops.gemv_workspace_bytes(f, n, k, m) > 0) for m in BATCHES for _, f, n, k in mats)     # products with shared row tiles add the finalize launch

    # ---- roofline of the dominant kernel (the largest Q4_K product of the layer): its average launch duration inside a CUDA graph of chained launches
    dom, per_m = sw.dominant_launch_us()
    nm, f, n, k = mats[dom]
    dom_us = float(np.mean(list(per_m.values())))
    dom_bytes = float(np.mean([alg_bytes(f, n, k, m) for m in per_m]))
    peak, peak_src = peaks()
    achieved = dom_bytes / (dom_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": f"gemv_t16_kernel<{f}> on {nm} [{n} x {k}]", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": peak_src, "traffic": dom_bytes * NCU_TRAFFIC_RATIO, "traffic_source": NCU_TRAFFIC_NOTE, "alg_bytes_per_launch": dom_bytes, "us_per_launch": dom_us,
                "us_per_launch_by_m": {str(m): v for m, v in per_m.items()},
                "timing": "CUDA graph of 8 chained launches of this product alone, alternating two weight copies (each larger than L2), CUDA events around the replay",
                "whole_step_frac_of_peak": value / world / peak}

    # ---- e2e: the module API with host activations (pinned h2d each step, d2h of every result)
    layers, copies, xs, pg = sw.layers, sw.copies, sw.xs, sw.pg
    mods = [[ForeignLinear(dp) for dp in layer] for layer in layers]
    ks = sorted({k for _, _, _, k in mats})
    hx = {(m, k): xs[(m, k)].cpu().pin_memory() for m in BATCHES for k in ks}
    hy = {(m, i): torch.empty((m, n), dtype=torch.float16).pin_memory() for m in BATCHES for i, (_, _, n, _) in enumerate(mats)}
    h2d = sum(2 * m * k for m in BATCHES for k in ks)
    d2h = sum(2 * m * n for m in BATCHES for _, _, n, _ in mats)

    def e2e_eager(s):
        layer = mods[s % copies]
        for m in BATCHES:
            dx = {k: hx[(m, k)].to(dev, non_blocking=True) for k in ks}
            for i, (nm_, f_, n_, k_) in enumerate(mats):
                y = layer[i](dx[k_])
                if world > 1:
                    dist.all_gather_into_tensor(sw.yg[(m, i)], y)
                hy[(m, i)].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    # the step goes through the package's HostGraph (pinned inputs -> h2d -> the layer's modules -> d2h into pinned outputs, one CUDA graph per
    # layer copy): the same copies and launches as the eager loop, without the per-call Python dispatch
    hgraphs = None
    if (world == 1 or pg is not None) and not args.e2e_eager:
        from kyojin_mac_b200.host_graph import HostGraph
        try:
            hgraphs = []
            pgs = None
            if world > 1:                                                        # N > 1: every stage ends with the peer gather of its four products
                from kyojin_mac_b200.dist import PeerGather
                pgs = {m: PeerGather([(m, n_) for _, _, n_, _ in mats], dev) for m in BATCHES}
            for c in range(copies):
                layer = mods[c]
                stages = []
                for m in sorted(BATCHES, reverse=True):                           # one stage per batch size: its upload / download overlap the neighbours' products; the largest batch first, so the download left exposed at the end of the step is the smallest
                    def stage_fn(*dx, layer=layer, m=m):
                        d = dict(zip(ks, dx))
                        outs = [layer[i](d[k_]) for i, (nm_, f_, n_, k_) in enumerate(mats)]
                        if pgs is not None:
                            pgs[m](outs)
                        return outs
                    stages.append((stage_fn, [hx[(m, k)] for k in ks]))
                hgraphs.append(HostGraph.staged(stages, dev))
            h2d, d2h = hgraphs[0].h2d_bytes, hgraphs[0].d2h_bytes                 # what the copies of a step move (inputs / results, 256-byte aligned slots)
        except Exception as e:
            hgraphs = None
            print(f"[bench] HostGraph capture unavailable ({type(e).__name__}: {e}); e2e through eager module calls", file=sys.stderr)

    def e2e_step(s):
        if hgraphs is not None:
            hgraphs[s % copies]()
        else:
            e2e_eager(s)

    for s in range(args.warmup):
        e2e_step(s)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for s in range(args.steps):
        e2e_step(s)
    e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), wall_ms)                                    # every step ends with a host wait for its results: host and device time agree; the larger is reported
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_val = world * step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9

    # ---- the other configurations (1 GPU) / the fixed-size configurations split over the ranks (N > 1)
    configs, strong = None, None
    e2e_through_graph = hgraphs is not None
    if not args.no_configs:
        from kyojin_mac_b200 import measure
        e2e_through_graph = hgraphs is not None
        del mods, hgraphs
        if world == 1:
            configs = {}
            for name, fn in (("cfg0", measure.cfg0), ("cfg2", measure.cfg2), ("cfg3", measure.cfg3), ("cfg4", measure.cfg4)):
                try:
                    configs[name] = fn()
                except Exception as e:                                            # noqa: BLE001 - a failing side configuration must not take the headline down
                    configs[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()
        else:
            from kyojin_mac_b200.dist import shard_rows
            sharded = [(nm_, f_, shard_rows(n_, world, rank)[1], k_) for nm_, f_, n_, k_ in mats]
            ss = Sweep(sharded, dev, world, rank, seed0=50000, nccl_gather=args.nccl_gather, staged_gather=not args.end_gather)
            ss.capture()
            ms_strong = ss.timed(args.steps, args.warmup, barrier)
            strong = {"cfg1": {"case": "the layer at its stated width, every matrix N-sharded by rows, peer gather per step", "ms_per_step": ms_strong,
                               "value": step_bytes / (ms_strong * 1e-3) / 1e9, "unit": "GB/s", "frac_of_n_times_peak": step_bytes / (ms_strong * 1e-3) / 1e9 / (world * peak)}}
            del ss
            torch.cuda.empty_cache()
            try:
                strong["prefill_and_moe"] = measure.dist_records()
            except Exception as e:                                                # noqa: BLE001
                strong["prefill_and_moe"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        ops.check_device_status()

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            one_pass, nbytes, sample, kind, impl = cpu_sample(row_frac=2)
            one_pass()
            ts = [one_pass() for _ in range(8)]
            cpu = {"value": nbytes / float(np.mean(ts)) / 1e9, "unit": "GB/s", "cores": min(8, os.cpu_count() or 1), "kind": kind, "sample": sample + ", 8 passes after one warm-up",
                   "host_cores": os.cpu_count(), "implementation": impl}
        line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate (u8 stored blocks)", "data": "synthetic",
                "config": {"workload": "cfg1: decode GEMV sweep over a 32B-class layer (q,k,v,o,gate,up Q4_K; down Q6_K), M=1,2,4,8 per step",
                           "launch_list": [f"{nm}:{f}:{n}x{k}" for nm, f, n, k in mats], "same_input_groups": not args.no_group,
                           "l2": "two layer copies alternate; one layer (328 MB) exceeds the 126 MB L2",
                           "timing": ("CUDA graph per step (chained launches), CUDA events, max over ranks" if sw.graphs is not None else "eager launches, CUDA events, max over ranks"),
                           "parallelism": ((f"weak scaling: n-sharded x{world} of an {world}x wider layer + peer-store gather of the output slices: one copy launch per batch size on a second stream (under the next batch size's products), one barrier per step" if sw.staged_gather
                                             else f"weak scaling: n-sharded x{world} of an {world}x wider layer + peer-store gather of the step's output slices (one launch + one barrier per step)") if pg is not None
                                           else f"weak scaling: n-sharded x{world} of an {world}x wider layer + NCCL all-gather of output slices") if world > 1 else "single GPU",
                           "bytes_per_step": step_bytes},
                "roofline": roofline, "cpu_baseline": cpu,
                "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
                        "api": "kyojin_mac_b200.host_graph.HostGraph.staged over ForeignLinear modules, one stage per batch size (pinned host activations in, pinned host results out)" if e2e_through_graph
                        else "ForeignLinear modules called eagerly (pinned host activations in, pinned host results out)"},
                "gpu_launches": launches_per_step * args.steps,
                "clocks": dict(clk.summary(), note=f"sampled every 200 ms from 0.25 s before the timed steps to the end of {n_load} further untimed steps of the same kind")}
        if configs is not None:
            line["configs"] = configs
        if strong is not None:
            line["strong"] = strong
        print(json.dumps(line))
    if world > 1:
        # leave without tearing NCCL down: captured collectives keep communicator resources alive and a destroy can block at exit
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-group", action="store_true", help="launch q, k, v and gate, up separately instead of as same-input groups")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-configs", action="store_true", help="skip the other benchmark configurations (1 GPU) / the strong-scaling forms (N > 1)")
    ap.add_argument("--end-gather", action="store_true", help="N > 1: gather all outputs of a step with one copy launch at its end instead of one per batch size on a second stream")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: one NCCL all-gather per product instead of the one-launch peer gather of the step")
    ap.add_argument("--e2e-eager", action="store_true", help="end-to-end leg through eager module calls instead of the HostGraph step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
