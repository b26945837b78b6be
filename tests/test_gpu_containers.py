"""Container operations and the router block (GPU): DevPack.rows / grouped, StoredEmbedding (token rows decoded from the stored blocks, tied head),
router logits vs fp64, the routed block with a shared expert vs the fp64 layer (tests/test_foreign_moe.py:73-118 in the reference)."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_moe as FM, foreign_pack as FP, ops, synth
from kyojin_mac_b200.foreign_linear import DevPack, ForeignLinear, ForeignSwitchGLU, StoredEmbedding
from oracle import kq_numpy as O, moe_numpy as M

pytestmark = pytest.mark.gpu
T_ = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q3_k", "nvfp4"])
def test_stored_embedding_rows_bit_exact(fmt):
    rng = np.random.default_rng(5)
    n, k = 200, 512                                                          # a table whose row count is not a multiple of 16
    raw = synth.raw_blocks(fmt, n, k, rng)
    emb = StoredEmbedding(FP.to_pack(T_[fmt], raw, k))
    ids = torch.from_numpy(rng.integers(0, n, (3, 7))).cuda()
    got = emb(ids)
    assert got.shape == (3, 7, k) and got.dtype == torch.float16
    ref = O.sat_f16(O.dequant(T_[fmt], raw, k))
    if fmt == "nvfp4":                                                       # the device decodes code 8 as -0 (pack form); the GGUF-form decoder gives +0
        np.testing.assert_array_equal(got.cpu().numpy().astype(np.float32), ref[ids.cpu().numpy()].astype(np.float32))
    else:
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16), ref[ids.cpu().numpy()].view(np.uint16))
    x = torch.from_numpy(synth.activations(2, k, rng)).cuda()
    assert torch.equal(emb.as_linear(x), emb.dev.apply(x))                  # the tied head is the stored product


def test_rows_and_grouped():
    rng = np.random.default_rng(6)
    k = 768
    raws = [synth.raw_blocks("q4_k", n, k, rng) for n in (40, 24, 64)]       # 40 and 24 are not multiples of 16: members are re-tiled
    devs = [DevPack(FP.to_pack("Q4_K", r, k)) for r in raws]
    g = DevPack.grouped(devs)
    ref = O.dequant("Q4_K", np.concatenate(raws), k)
    np.testing.assert_array_equal(g.dequant(torch.float32).cpu().numpy().view(np.uint32), ref.view(np.uint32))
    x = torch.from_numpy(synth.activations(3, k, rng)).cuda()
    y = g.apply(x)
    parts = torch.cat([d.apply(x) for d in devs], dim=1)
    assert torch.equal(y, parts)                                            # a row's bits do not depend on which matrix it sits in
    head = g.rows(50)
    np.testing.assert_array_equal(head.dequant(torch.float32).cpu().numpy().view(np.uint32), ref[:50].view(np.uint32))
    pick = [127, 3, 3, 64, 90]
    sub = g.rows(pick)
    np.testing.assert_array_equal(sub.dequant(torch.float32).cpu().numpy().view(np.uint32), ref[pick].view(np.uint32))
    assert sub.n == 5 and g.rows(32).n == 32 and len(g.arrays()) == 2


@pytest.mark.parametrize("T,E,H,dt", [(5, 64, 512, torch.float16), (300, 256, 7168, torch.float16), (2000, 32, 1024, torch.float32), (33, 16, 256, torch.bfloat16),
                                       (1500, 256, 7168, torch.float16), (1101, 20, 512, torch.bfloat16)])
def test_router_logits_vs_fp64(T, E, H, dt):
    g = torch.Generator(device="cuda").manual_seed(T)
    x = torch.randn((T, H), device="cuda", generator=g).to(dt)
    gw = torch.randn((E, H), device="cuda", generator=g) * 0.05
    sgw = torch.randn((H,), device="cuda", generator=g) * 0.05
    lg = ops.router_logits(x, gw, sgw, tensor_cores=False)
    want = x.double() @ torch.cat([gw, sgw[None]]).double().T
    assert lg.shape == (T, E + 1) and (lg.double() - want).abs().max().item() < 1e-4 * want.abs().max().item()
    lg0 = ops.router_logits(x, gw, None, tensor_cores=False)
    assert torch.equal(lg0[:, :E], lg[:, :E]) and (lg0[:, E] == 0).all()
    if T >= 1024:                                                           # many tokens take the weight-resident kernel: same bits as the token-resident one
        parts = torch.cat([ops.router_logits(x[i:i + 500], gw, sgw, tensor_cores=False) for i in range(0, T, 500)])
        assert torch.equal(parts, lg)


@pytest.mark.parametrize("T,E,H", [(256, 256, 7168), (300, 64, 512), (1500, 256, 7168), (4096, 20, 1024), (70, 8, 256)])
def test_router_logits_on_tensor_cores(T, E, H):
    """The gate cut into three fp16 pieces, one tcgen05 product with fp32 accumulation, recombined: against the fp64 logits (same bound as the fp32 kernels, and
    a tighter one on the relative Frobenius error), with and without the shared-expert row, rows with very different magnitudes (per-row scales), a zero row,
    and the default dispatch (fp16 batches of 512 tokens or more take this path)."""
    g = torch.Generator(device="cuda").manual_seed(T + 1)
    x = torch.randn((T, H), device="cuda", generator=g).to(torch.float16)
    gw = torch.randn((E, H), device="cuda", generator=g) * 0.05
    gw[1] *= 1e-4
    gw[2] *= 3e3
    gw[3] = 0
    gw[4, ::2] *= 1e-6                                                      # entries far below the row's maximum
    sgw = torch.randn((H,), device="cuda", generator=g) * 0.05
    want = x.double() @ torch.cat([gw, sgw[None]]).double().T
    lg = ops.router_logits(x, gw, sgw, tensor_cores=True)
    ops.check_device_status()
    err = (lg.double() - want).abs()
    scale = want.abs().amax(0, keepdim=True).clamp_min(1e-30)
    assert lg.shape == (T, E + 1) and (err / scale).max().item() < 1e-4       # per gate row: every row is held to its own magnitude
    assert (err.norm() / want.norm()).item() < 1e-5
    assert (lg[:, 3] == 0).all()
    f32 = ops.router_logits(x, gw, sgw, tensor_cores=False)
    assert ((lg - f32).abs() / scale.float()).max().item() < 1e-4
    lg0 = ops.router_logits(x, gw, None, tensor_cores=True)
    assert torch.equal(lg0[:, :E], lg[:, :E]) and (lg0[:, E] == 0).all()
    if T >= 512:
        assert torch.equal(ops.router_logits(x, gw, sgw), lg)
    with pytest.raises(ValueError):
        ops.router_logits(x.float(), gw, sgw, tensor_cores=True)


def _stack(fmt, E, n, k, seed):
    rng = np.random.default_rng(seed)
    raws = [synth.raw_blocks(fmt, n, k, rng) for _ in range(E)]
    return DevPack([FP.to_pack(T_[fmt], r, k) for r in raws]), np.stack([O.dequant(T_[fmt], r, k) for r in raws])


@pytest.mark.parametrize("T", [5, 160])
def test_routed_block_with_shared_expert(T):
    E, K, H, I = 8, 2, 512, 256
    g, Wg = _stack("q4_k", E, I, H, 20)
    u, Wu = _stack("q4_k", E, I, H, 21)
    d, Wd = _stack("q4_k", E, H, I, 22)
    rng = np.random.default_rng(23)
    x = (synth.activations(T, H, rng).astype(np.float32) * 0.5).astype(np.float16)
    gw = (rng.standard_normal((E, H)) * 0.1).astype(np.float32)
    sgw = (rng.standard_normal((1, H)) * 0.1).astype(np.float32)
    raw_s = synth.raw_blocks("q6_k", H, H, rng)
    shared = ForeignLinear(FP.to_pack("Q6_K", raw_s, H))
    Ws = O.dequant("Q6_K", raw_s, H).astype(np.float64)
    blk = FM.RoutedBlock(torch.from_numpy(gw).cuda(), ForeignSwitchGLU(g, u, d), K, True, shared, torch.from_numpy(sgw).cuda(), out_dtype=torch.float32)
    xd = torch.from_numpy(x).cuda()
    out = blk(xd)
    ops.check_device_status()
    inds, scs, sgs = blk.route(xd)
    ie, sc = inds.cpu().numpy().reshape(T, K), scs.cpu().numpy().reshape(T, K).astype(np.float64)
    lg = x.astype(np.float64) @ np.concatenate([gw, sgw]).astype(np.float64).T
    oi, os_, osg = M.select(lg.astype(np.float32), K, True, E)
    np.testing.assert_array_equal(ie.reshape(-1), oi)                        # no near-ties in this seed: the device router picks the oracle's experts
    y = M.routed_layer(x, ie, Wg, Wu, Wd, K, ref_path=False).reshape(T, K, H)
    want = (y * sc[..., None]).sum(1) + sgs.cpu().numpy().astype(np.float64)[:, None] * (x.astype(np.float64) @ Ws.T)
    assert out.dtype == torch.float32 and O.rel_fro(out.cpu().numpy(), want) <= 2e-3
