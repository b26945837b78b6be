"""Runs one operator on synthetic weights a few times: a quick check and the target of profiler captures.

    python -m kyojin_mac_b200.probe gemv q4_k 27648 5120 1        # fmt n k m
    python -m kyojin_mac_b200.probe gemm q3_k 12288 3072 2048     # dequant + tcgen05 GEMM
    python -m kyojin_mac_b200.probe gemm_kq q3_k 12288 3072 2048  # tcgen05 GEMM with the weights decoded inside (6th argument: msub 1 | 2)
    python -m kyojin_mac_b200.probe gemm_a4 nvfp4 18432 7168 4096 # activation quantiser + block-scaled tcgen05 GEMM
"""
import sys

import torch

from . import ops, synth


def main(argv):
    op, fmt, n, k, m = argv[0], argv[1], int(argv[2]), int(argv[3]), int(argv[4])
    reps = int(argv[5]) if len(argv) > 5 else 3
    t16 = synth.t16_random_device(fmt, n, k, seed=0)
    x = torch.randn((m, k), device="cuda").to(torch.float16)
    if op == "gemv":
        print(ops.gemv_plan(fmt, n, k, m))
    for _ in range(reps):
        if op == "gemv":
            y = ops.gemv(fmt, t16, n, k, x)
        elif op == "gemm":
            y = ops.gemm_f16(x, ops.dequant(fmt, t16, n, k, torch.float16))
        elif op == "gemm_kq":
            y = ops.gemm_kq(fmt, t16, n, k, x, msub=int(argv[6]) if len(argv) > 6 else 0)
        elif op == "gemm_a4":
            from .foreign_linear import DevPack
            y = DevPack.from_t16(fmt, t16, n, k).apply_a4(x.to(torch.bfloat16))
        else:
            raise SystemExit(f"unknown op {op}")
    torch.cuda.synchronize()
    ops.check_device_status()
    print("ok", float(y.float().abs().mean()))


if __name__ == "__main__":
    main(sys.argv[1:])
