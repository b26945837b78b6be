"""Device-side MoE slot sort, torch mirror of kyojin_mlx/moe_sort.py:58-78 `plan_device` (one launch: histogram, scan, scatter)."""
from __future__ import annotations

import torch

from . import ops


def plan_device(ids: torch.Tensor, wts: torch.Tensor, experts: int, topk: int, rank: torch.Tensor | None = None):
    """ids i32 [P], wts f32 [P] (P = T * topk); rank u32 [E] optional (position of each expert's segment).
    Returns (tok u32 [P] sorted slot -> token, ids_s i32 [P], wts_s f32 [P], inv u32 [P] pair -> sorted slot, cum u32 [E+1] segment starts).
    Any permutation inside an expert's segment is valid (a slot's arithmetic never depends on where it sits)."""
    P = ids.numel()
    if wts.numel() != P or P % topk:
        raise ValueError("ids / wts sizes do not match topk")
    pl = ops.moe_plan(ids, experts, topk, 128, wts=wts, rank=rank)
    return pl["tok"], pl["ids_s"], pl["wts_s"], pl["inv"], pl["off"]
