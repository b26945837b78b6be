"""Fused routed-MoE layer: torch mirror of kyojin_mlx/moe_fused.py:26-46 (`MoeFused`, `wrap`). The reference wraps an EXL3 `MoeGather` whose pairs
routed to the same expert share one weight decode; here the same call shape runs on K-quant / NVFP4 expert stacks (a ForeignSwitchGLU) with expert
election in the gathered GEMV, and returns the routing-weighted fp32 sum over the top-k slots."""
from __future__ import annotations

import torch

from . import ops


class MoeFused:
    def __init__(self, gather):
        self.m = gather                      # a ForeignSwitchGLU

    def __call__(self, x, ids, wts, fq8: bool = False):
        """x [rows, H], ids [rows, topk], wts [rows, topk] -> f32 [rows, H]."""
        if fq8:
            raise NotImplementedError("fq8 (fp8 fake-quant of the input) belongs to another model family and is not built")
        rows = x.shape[0]
        ids2, w2 = ids.reshape(rows, -1), wts.reshape(rows, -1)
        K = ids2.shape[1]
        y = self.m(x, ids2)                                               # [rows, K, H] unweighted
        return ops.moe_combine(y.reshape(rows * K, -1), w2.reshape(-1).to(torch.float32).contiguous(), K, dtype=torch.float32)


def wrap(gather) -> MoeFused:
    return MoeFused(gather)
