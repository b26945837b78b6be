"""Host-side step API (GPU): a step captured by HostGraph returns what the eager module calls return."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_pack as FP, synth
from kyojin_mac_b200.foreign_linear import ForeignLinear
from kyojin_mac_b200.host_graph import HostGraph

pytestmark = pytest.mark.gpu


def test_host_graph_step_equals_eager():
    """Pinned inputs -> modules -> pinned outputs in one CUDA graph: same bits as the eager calls, call after call with new inputs."""
    rng = np.random.default_rng(8)
    k = 1024
    lins = [ForeignLinear(FP.to_pack("Q4_K", synth.raw_blocks("q4_k", n, k, rng), k)) for n in (256, 4096)]
    step = HostGraph(lambda x, x2: [l(x) for l in lins] + [lins[0](x2)], [(4, k), (1, k)])
    for it in range(3):
        a, b = torch.from_numpy(synth.activations(4, k, rng)), torch.from_numpy(synth.activations(1, k, rng))
        step.inputs[0].copy_(a)
        step.inputs[1].copy_(b)
        outs = step()
        want = [l(a.cuda()) for l in lins] + [lins[0](b.cuda())]
        assert len(outs) == 3
        for o, w in zip(outs, want):
            assert torch.equal(o, w.cpu())
    hx = torch.from_numpy(synth.activations(2, k, rng)).pin_memory()
    one = HostGraph(lambda x: lins[0](x), [hx])                              # a pinned tensor as input: shape and contents are taken over
    assert torch.equal(one()[0], lins[0](hx.cuda()).cpu())
    st = HostGraph.staged([(lambda x: lins[0](x), [(2, k)]), (lambda x: [lins[1](x), lins[0](x)], [(3, k)])])    # stages: copies overlap the neighbouring stage
    for it in range(2):
        a, b = torch.from_numpy(synth.activations(2, k, rng)), torch.from_numpy(synth.activations(3, k, rng))
        st.inputs[0].copy_(a)
        st.inputs[1].copy_(b)
        o = st()
        assert torch.equal(o[0], lins[0](a.cuda()).cpu()) and torch.equal(o[1], lins[1](b.cuda()).cpu()) and torch.equal(o[2], lins[0](b.cuda()).cpu())
    with pytest.raises(ValueError):
        HostGraph(lambda x: lins[0](x), [torch.zeros((4, k), dtype=torch.float16)])       # not pinned
