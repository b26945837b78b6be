"""Installers over a module tree (GPU): same-input grouping (q | k | v and gate | up become one product each, results unchanged bit for bit) and the fused dense
gated MLP (activation formed inside the down projection's launch), on a small torch model built from ForeignLinears; mirrors the reference's
tests/test_foreign_group.py and tests/test_dense_glu.py in what they check: same outputs, fewer launches, other activations left alone."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_linear as FL, foreign_pack as FP, ops, synth

pytestmark = pytest.mark.gpu
H, KV, I = 512, 256, 1024


def _lin(fmt, n, k, seed):
    tn = {"q4_k": "Q4_K", "q6_k": "Q6_K"}[fmt]
    return FL.ForeignLinear(FP.to_pack(tn, synth.raw_blocks(fmt, n, k, np.random.default_rng(seed), d_sigma=3e-4), k))


def _norm(x):
    return (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype)


class MLP(torch.nn.Module):
    def __init__(self, act="silu"):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = _lin("q4_k", I, H, 1), _lin("q4_k", I, H, 2), _lin("q6_k", H, I, 3)
        self.act = act

    def forward(self, x):
        a = self.gate_proj(x).float()
        a = torch.nn.functional.silu(a) if self.act == "silu" else torch.nn.functional.gelu(a)
        return self.down_proj((a * self.up_proj(x).float()).to(x.dtype))


class Block(torch.nn.Module):
    def __init__(self, act="silu"):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = _lin("q4_k", H, H, 4), _lin("q4_k", KV, H, 5), _lin("q6_k", KV, H, 6), _lin("q4_k", H, H, 7)
        self.mlp = MLP(act)

    def forward(self, x):
        xn = _norm(x)
        q, k, v = self.q_proj(xn), self.k_proj(xn), self.v_proj(xn)
        h = x + self.o_proj(_norm(q * (k.mean(-1, keepdim=True) + v.mean(-1, keepdim=True))))
        return h + self.mlp(_norm(h))


class Tiny(torch.nn.Module):
    def __init__(self, act="silu"):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.embed = torch.nn.Embedding(64, H, _weight=torch.randn((64, H), generator=g)).cuda().half()
        self.layers = torch.nn.ModuleList([Block(act), Block(act)])

    def forward(self, tokens):
        x = self.embed(tokens)
        for l in self.layers:
            x = l(x)
        return x


def test_group_same_input_and_dense_glu():
    model = Tiny()
    tokens = torch.tensor([[3, 7, 11]], device="cuda")
    with torch.no_grad():
        want = model(tokens)
    logs = []
    got = FL.group_same_input(model, log=logs.append)
    # per block: q | k (Q4_K, same input; v is Q6_K and stays alone) and gate | up
    assert got == {"groups": 4, "members": 8, "launches_saved": 4}, (got, logs)
    assert type(model.layers[0].q_proj) is FL.GroupMember and type(model.layers[0].v_proj) is FL.ForeignLinear
    with torch.no_grad():
        assert torch.equal(model(tokens), want)                            # the grouped rows are the members' own rows
        assert torch.equal(model(tokens[:, :1]), want[:, :1])
    assert FL.group_same_input(model, log=logs.append)["groups"] == 0       # nothing left to group
    n = FL.install_dense_glu(model, log=logs.append)
    assert n == 2 and FL.install_dense_glu(model, log=logs.append) == 0
    with torch.no_grad():
        fused = model(tokens)
    # the stock forward multiplies silu(a) by b in fp32 as the fused staging does; the two exponentials may differ in the last place: one fp16 step
    torch.testing.assert_close(fused.float(), want.float(), rtol=4e-3, atol=4e-3)
    x70 = torch.randint(0, 64, (1, 70), device="cuda")                      # more rows than the decode limit: the module's own forward runs
    with torch.no_grad():
        assert model(x70).shape == (1, 70, H)
    ops.check_device_status()


def test_other_activations_keep_their_forward():
    model = Tiny(act="gelu")
    assert FL.install_dense_glu(model, log=lambda s: None) == 0
    assert not FL.silu_gated(model.layers[0].mlp)
