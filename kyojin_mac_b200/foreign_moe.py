"""Routed-expert block around the quantized expert products: torch mirror of kyojin_mlx/foreign_moe.py (`_logits` :122-130, `_select` :132-138, `_silu_mul`
:150-153, `_combine` :155-158, `_fused_call` :234-266, `_pf_call` :221-231). Router in fp32, softmax / top-k / renormalise in one launch, experts through
ForeignSwitchGLU (gathered GEMV for decode, grouped tcgen05 GEMM for prefill), one combine launch (scores, sigmoid-gated shared expert, saturated fp16 or fp32)."""
from __future__ import annotations

import torch

from . import ops

E_MAX = 1024


def _logits(x2, gw, sgw, T, E, H, has_s):
    """fp32 [T, E + 1]: x2 [T, H] on the fp32 gate gw [E, H]; column E holds the shared-expert gate logit when has_s."""
    if x2.shape != (T, H) or gw.shape != (E, H):
        raise ValueError("router: x2 [T, H], gw [E, H]")
    return ops.router_logits(x2, gw, sgw if has_s else None)


def _select(lg, T, E, K, norm):
    """(inds i32 [T K], scs f32 [T K], sgs f32 [T]): softmax over E logits, top-k by value (lowest index on ties), weights top / sum(top) when norm; sgs =
    sigmoid of column E."""
    return ops.moe_select(lg, E, K, bool(norm), has_shared=lg.shape[1] > E)


def _silu_mul(a, b, act=None):
    if act is not None:
        raise NotImplementedError("only the silu-gated activation is built")
    return ops.silu_mul(a, b)


def _combine(y, scs, sgs, sh, T, K, H, has_s, ot=torch.float32):
    """[T, H] = sum_k f32(y[t K + k]) scs[t K + k] (+ sgs[t] f32(sh[t]) when has_s); fp16 output saturated."""
    return ops.moe_combine(y.reshape(T * K, H), scs, K, sgs if has_s else None, sh if has_s else None, ot)


class RoutedBlock(torch.nn.Module):
    """A sparse-MoE block with the attribute names the reference patches on mlx-lm blocks (gate.weight fp32 [E, H], switch_mlp, top_k, num_experts,
    norm_topk_prob, shared_expert, shared_expert_gate.weight [1, H]); forward = the reference's fused call."""

    def __init__(self, gate_weight: torch.Tensor, switch_mlp, top_k: int, norm_topk_prob: bool = True, shared_expert=None, shared_gate_weight=None,
                 out_dtype=torch.float16):
        super().__init__()
        if gate_weight.dtype != torch.float32 or gate_weight.shape[0] > E_MAX:
            raise ValueError("the router gate is fp32 [E, H] with E <= 1024")
        self.gate_weight, self.switch_mlp, self.top_k, self.num_experts = gate_weight, switch_mlp, top_k, gate_weight.shape[0]
        self.norm_topk_prob, self.shared_expert, self.shared_gate_weight, self.out_dtype = norm_topk_prob, shared_expert, shared_gate_weight, out_dtype
        if (shared_expert is None) != (shared_gate_weight is None):
            raise ValueError("a shared expert comes with its gate row")

    def route(self, x2):
        T, H = x2.shape
        has_s = self.shared_expert is not None
        lg = _logits(x2, self.gate_weight, self.shared_gate_weight, T, self.num_experts, H, has_s)
        return _select(lg, T, self.num_experts, self.top_k, self.norm_topk_prob)

    def forward(self, x):
        lead, H = x.shape[:-1], x.shape[-1]
        x2 = x.reshape(-1, H)
        T, K = x2.shape[0], self.top_k
        inds, scs, sgs = self.route(x2)
        y = self.switch_mlp(x2, inds.reshape(T, K))
        has_s = self.shared_expert is not None
        sh = self.shared_expert(x2).reshape(T, H).to(torch.float16).contiguous() if has_s else None
        return _combine(y.reshape(T * K, H), scs, sgs, sh, T, K, H, has_s, self.out_dtype).reshape(*lead, H)
