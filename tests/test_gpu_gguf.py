"""GGUF file -> device modules (GPU): a linear and an expert stack loaded from the fixture file give the results of the same bytes handed over directly."""
import os

import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_gguf as GG, foreign_pack as FP, synth
from kyojin_mac_b200.foreign_linear import DevPack, ForeignLinear
from oracle import kq_numpy as O

pytestmark = pytest.mark.gpu
PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny.gguf")


def test_linear_and_experts_from_file():
    rng = np.random.default_rng(1)
    with GG.GgufFile(PATH) as g:
        for name, tname in (("blk.0.attn_q.weight", "Q4_K"), ("blk.0.ffn_down.weight", "Q6_K"), ("blk.0.attn_k.weight", "Q3_K"), ("blk.0.attn_v.weight", "Q5_K"),
                            ("blk.0.attn_output.weight", "Q8_0")):
            ti = g.tensors[name]
            k, n = ti.ne
            lin = g.load_linear(name)
            x = torch.from_numpy(synth.activations(3, k, rng)).cuda()
            raw = np.array(g.raw(name))
            assert torch.equal(lin(x), ForeignLinear(FP.to_pack(tname, raw, k))(x))
            w = lin.dev.dequant(torch.float32).cpu().numpy()
            np.testing.assert_array_equal(w.view(np.uint32), O.dequant(tname, raw, k).view(np.uint32))     # bit-exact decode of the file's bytes
        st = g.load_experts("blk.0.ffn_gate_exps.weight")
        assert (st.E, st.n, st.k) == (3, 16, 256)
        raw = np.array(g.raw("blk.0.ffn_gate_exps.weight"))
        x = torch.from_numpy(synth.activations(2, 256, rng)).cuda()
        for e in range(3):
            one = DevPack(FP.to_pack("Q4_K", raw[e], 256))
            assert torch.equal(st.expert(e).apply(x), one.apply(x))
