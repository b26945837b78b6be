"""Routed-expert path parity (GPU). Mirrors the reference's tests: router vs fp64 softmax / argsort as sets (tests/test_foreign_moe.py:95-118), device sort
vs the numpy plan incl. zero-row experts (tests/test_moe_sort.py:13-76), tiles cover every slot once (tests/test_kq_rt2.py:31-54), grouped == per-expert
(tests/test_foreign_moe.py:200-220), election == per-slot gather bitwise (tests/test_moe_union.py:66-88), block vs stock (tests/test_foreign_moe.py:73-91)."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_kqgmm as KQ, foreign_pack as FP, moe_fused, moe_sort, ops, synth
from kyojin_mac_b200.foreign_linear import DevPack, ForeignSwitchGLU
from oracle import kq_numpy as O, moe_numpy as M

pytestmark = pytest.mark.gpu
T_ = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}


@pytest.mark.parametrize("T,E,K,norm", [(64, 256, 8, True), (7, 64, 4, False), (300, 128, 8, True)])
def test_router_select(T, E, K, norm):
    rng = np.random.default_rng(T + E)
    lg = rng.standard_normal((T, E + 1)).astype(np.float32)
    inds, scs, sgs = ops.moe_select(torch.from_numpy(lg).cuda(), E, K, norm, has_shared=True)
    inds, scs, sgs = inds.cpu().numpy().reshape(T, K), scs.cpu().numpy().reshape(T, K), sgs.cpu().numpy()
    p = np.exp(lg[:, :E].astype(np.float64) - lg[:, :E].max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.argsort(-p, axis=-1, kind="stable")[:, :K]
    for t in range(T):
        assert set(inds[t]) == set(want[t])
        w = p[t, inds[t]]
        np.testing.assert_allclose(scs[t], w / w.sum() if norm else w, rtol=1e-3)
    np.testing.assert_allclose(sgs, 1 / (1 + np.exp(-lg[:, E].astype(np.float64))), rtol=1e-5)
    oi, os_, _ = M.select(lg, K, norm, E)                                   # the restatement agrees, order included
    np.testing.assert_array_equal(inds.reshape(-1), oi)
    np.testing.assert_allclose(scs.reshape(-1), os_, rtol=1e-5)


def test_router_ties_take_lowest_index():
    lg = np.zeros((3, 16), np.float32)
    inds, scs, _ = ops.moe_select(torch.from_numpy(lg).cuda(), 16, 4, True)
    np.testing.assert_array_equal(inds.cpu().numpy().reshape(3, 4), np.tile(np.arange(4), (3, 1)))
    np.testing.assert_allclose(scs.cpu().numpy(), 0.25, rtol=1e-6)


@pytest.mark.parametrize("P,E,topk", [(512, 256, 8), (32768, 256, 8), (40, 8, 4), (1024, 64, 2)])
def test_plan_device(P, E, topk):
    rng = np.random.default_rng(P)
    ids = rng.integers(0, E, P).astype(np.int32)
    ids[ids == 3] = 4                                                        # a zero-row expert
    wts = rng.random(P).astype(np.float32)
    tok, ids_s, wts_s, inv, cum = moe_sort.plan_device(torch.from_numpy(ids).cuda(), torch.from_numpy(wts).cuda(), E, topk)
    tok, ids_s, wts_s, inv, cum = (a.cpu().numpy() for a in (tok, ids_s, wts_s, inv, cum))
    cnt, off, tb = M.host_plan(ids, E, 128)
    np.testing.assert_array_equal(cum.astype(np.uint32), off)
    assert (np.diff(ids_s) >= 0).all()                                       # sorted by expert
    np.testing.assert_array_equal(ids_s[inv], ids)                          # inv maps every pair to a slot of its expert
    assert sorted(inv.tolist()) == list(range(P))                           # a permutation
    np.testing.assert_array_equal(tok[inv], np.arange(P) // topk)
    np.testing.assert_array_equal(wts_s[inv], wts)
    order, tbd, offd = KQ.csort(torch.from_numpy(ids).cuda(), E)
    np.testing.assert_array_equal(tbd.cpu().numpy().astype(np.uint32), tb)
    np.testing.assert_array_equal(offd.cpu().numpy().astype(np.uint32), off)
    o = order.cpu().numpy()
    assert sorted(o.tolist()) == list(range(P)) and (np.diff(ids[o]) >= 0).all()
    bad = ids.copy()
    bad[5], bad[P - 1] = -1, E + 3                                            # ids outside the stack: sorted behind the last segment
    order, tbd, offd = KQ.csort(torch.from_numpy(bad).cuda(), E)
    o, offd = order.cpu().numpy(), offd.cpu().numpy()
    assert sorted(o.tolist()) == list(range(P)) and offd[E] == P - 2 and set(o[P - 2:].tolist()) == {5, P - 1}
    assert (np.diff(bad[o[:P - 2]]) >= 0).all()


def _stack(fmt, E, n, k, seed):
    rng = np.random.default_rng(seed)
    raws = [synth.raw_blocks(fmt, n, k, rng) for _ in range(E)]
    packs = [FP.to_pack(T_[fmt], r, k) for r in raws]
    W = np.stack([O.dequant(T_[fmt], r, k) for r in raws])
    return DevPack(packs), W


@pytest.mark.parametrize("fmt", ["q4_k", "q6_k", "q3_k", "nvfp4", "q5_k", "q8_0", "q2_k", "iq4_xs"])
def test_gather_election_equals_per_expert(fmt):
    """Gathered GEMV with expert election == the expert's own one-matrix GEMV on the same row, bit for bit, and matches fp64."""
    E, n, k, S = 6, 64, 512, 37
    dev, W = _stack(fmt, E, n, k, 1)
    rng = np.random.default_rng(2)
    x = synth.activations(9, k, rng)
    eids = rng.integers(0, E, S).astype(np.int32)
    eids[:12] = 2                                                             # more than 8 slots on one expert: two groups
    xrows = rng.integers(0, 9, S).astype(np.int32)
    xd = torch.from_numpy(x).cuda()
    y = dev.gather(xd, torch.from_numpy(xrows).cuda(), torch.from_numpy(eids).cuda())
    ops.check_device_status()
    for s in range(S):
        one = dev.expert(int(eids[s])).apply(xd[xrows[s]:xrows[s] + 1])
        assert torch.equal(one[0], y[s]), s
    want = np.stack([O.matmul_f64(x[xrows[s]:xrows[s] + 1], W[eids[s]])[0] for s in range(S)])
    assert O.rel_fro(y.cpu().numpy(), want) <= 1e-3


def test_pair_and_glu_launches_vs_per_expert_products():
    """gate | up in one launch and the down product with the activation formed while its rows are staged: each slot equals the expert's own one-matrix product
    (another kernel entry, the dense GEMV) on the same input, bit for bit, and the gated input equals the numpy restatement of the activation."""
    E, n, k, S = 4, 64, 256, 21
    g, _ = _stack("q4_k", E, n, k, 3)
    u, _ = _stack("q4_k", E, n, k, 4)
    d, Wd = _stack("q6_k", E, 256, 256, 5)
    rng = np.random.default_rng(6)
    x = torch.from_numpy(synth.activations(5, k, rng)).cuda()
    en = rng.integers(0, E, S).astype(np.int32)
    en[:11] = 1                                                               # more than 8 slots on one expert: two groups
    rn = rng.integers(0, 5, S).astype(np.int32)
    eids, xrows = torch.from_numpy(en).cuda(), torch.from_numpy(rn).cuda()
    a, b = g.gather_pair(u, x, xrows, eids)
    ops.check_device_status()
    for s in range(S):
        assert torch.equal(a[s], g.expert(int(en[s])).apply(x[rn[s]:rn[s] + 1])[0]), s
        assert torch.equal(b[s], u.expert(int(en[s])).apply(x[rn[s]:rn[s] + 1])[0]), s
    aa = torch.from_numpy(synth.activations(S, 256, rng)).cuda()
    bb = torch.from_numpy(synth.activations(S, 256, rng)).cuda()
    ar = torch.arange(S, dtype=torch.int32, device="cuda")
    for limit in (None, 0.5):
        h = M.glu(aa.cpu().numpy(), bb.cpu().numpy(), limit)                  # numpy restatement of the activation
        np.testing.assert_array_equal(ops.silu_mul(aa, bb, limit).cpu().numpy(), h)
        y = d.gather_glu(aa, bb, ar, eids, limit=limit)
        ops.check_device_status()
        hd = torch.from_numpy(h).cuda()
        for s in range(S):
            assert torch.equal(y[s], d.expert(int(en[s])).apply(hd[s:s + 1])[0]), (limit, s)
        want = np.stack([O.matmul_f64(h[s:s + 1], Wd[en[s]])[0] for s in range(S)])
        assert O.rel_fro(y.cpu().numpy(), want) <= 1e-3


def test_slots_without_an_expert_are_tolerated():
    """A token whose router logits hold a NaN gets the id 0xFFFFFFFF from the select kernel. Such slots must not reach an unbounded read: the sort puts them
    behind the last segment with weight 0, their output rows are zeros on both routed paths, every other slot is unaffected."""
    E, H, I, T, K = 4, 256, 256, 40, 2
    g, Wg = _stack("q4_k", E, I, H, 30)
    u, Wu = _stack("q4_k", E, I, H, 31)
    d, Wd = _stack("q4_k", E, H, I, 32)
    rng = np.random.default_rng(33)
    x = (synth.activations(T, H, rng).astype(np.float32) * 0.5).astype(np.float16)
    lg = rng.standard_normal((T, E)).astype(np.float32)
    lg[7, 1] = np.nan
    inds, scs, _ = ops.moe_select(torch.from_numpy(lg).cuda(), E, K, True)
    ie = inds.cpu().numpy().reshape(T, K)
    assert (ie[7].astype(np.uint32) >= E).all() and (np.delete(ie, 7, 0).astype(np.uint32) < E).all()
    pl = ops.moe_plan(inds, E, K, 128, wts=scs)
    order, off, wts_s = pl["order"].cpu().numpy(), pl["off"].cpu().numpy(), pl["wts_s"].cpu().numpy()
    assert sorted(order.tolist()) == list(range(T * K)) and off[E] == T * K - K
    assert set(order[off[E]:].tolist()) == {7 * K, 7 * K + 1} and (wts_s[off[E]:] == 0).all()
    blk = ForeignSwitchGLU(g, u, d)
    xd = torch.from_numpy(x).cuda()
    good = np.delete(np.arange(T), 7)
    want = M.routed_layer(x[good], ie[good], Wg, Wu, Wd, K, ref_path=False).reshape(T - 1, K, H)
    from kyojin_mac_b200 import foreign_kqgmm as KQ2
    for name, y in (("gathered", blk._gather_path(xd, inds, K)), ("grouped", KQ2.mlp(blk, xd, inds, K))):
        ops.check_device_status()
        yn = y.reshape(T, K, H).cpu().numpy()
        assert (yn[7] == 0).all(), name
        assert O.rel_fro(yn[good], want) <= 2e-3, name


@pytest.mark.parametrize("T,K", [(6, 4), (200, 4)])
def test_switch_glu_block_vs_fp64(T, K):
    """Whole routed layer (decode path for 24 slots, sorted grouped GEMM for 800) against the fp64 layer and the reference-path restatement."""
    E, H, I = 8, 512, 256
    g, Wg = _stack("q4_k", E, I, H, 10)
    u, Wu = _stack("q4_k", E, I, H, 11)
    d, Wd = _stack("q4_k", E, H, I, 12)
    # scale weights' effect down: keep |h| moderate so fp16 intermediates stay in range like a real layer
    rng = np.random.default_rng(13)
    x = (synth.activations(T, H, rng).astype(np.float32) * 0.5).astype(np.float16)
    lg = rng.standard_normal((T, E)).astype(np.float32)
    inds, scs, _ = ops.moe_select(torch.from_numpy(lg).cuda(), E, K, True)
    blk = ForeignSwitchGLU(g, u, d)
    y = blk(torch.from_numpy(x).cuda(), inds.reshape(T, K))
    ops.check_device_status()
    assert y.shape == (T, K, H)
    ie = inds.cpu().numpy()
    want = M.routed_layer(x, ie, Wg, Wu, Wd, K, ref_path=False)
    refp = M.routed_layer(x, ie, Wg, Wu, Wd, K, ref_path=True)
    err, ref_err = O.rel_fro(y.reshape(T * K, H).cpu().numpy(), want), O.rel_fro(refp, want)
    assert err <= 2e-3 and err <= 2 * ref_err + 1e-6, (err, ref_err)       # two fp16 roundings on the way (a, b, h) as in the reference path
    out = moe_fused.wrap(blk)(torch.from_numpy(x).cuda(), inds.reshape(T, K), scs.reshape(T, K))
    wantc = (want.reshape(T, K, H) * scs.cpu().numpy().reshape(T, K, 1).astype(np.float64)).sum(1)
    assert out.dtype == torch.float32 and O.rel_fro(out.cpu().numpy(), wantc) <= 2e-3
    c16 = ops.moe_combine(y.reshape(T * K, H), scs, K)
    # fp32 multiply-adds are fused on the device: equal to the restatement up to one fp16 ulp
    np.testing.assert_allclose(c16.float().cpu().numpy(), M.combine(y.reshape(T * K, H).cpu().numpy(), scs.cpu().numpy(), K).astype(np.float32), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("mt", [128, 256])
def test_grouped_gemm_equals_per_expert(mt):
    E, n, k, S = 5, 256, 512, 700
    dev, W = _stack("q3_k", E, n, k, 20)
    rng = np.random.default_rng(21)
    e = rng.integers(0, E, S).astype(np.int32)
    e[e == 1] = 0                                                             # an expert without rows
    x = synth.activations(S, k, rng)
    order, tb, off = KQ.csort(torch.from_numpy(e).cuda(), E, mt)
    xg = KQ.gather_perm(torch.from_numpy(x).cuda(), order, 1)
    y = KQ.gmm(dev, xg, tb, off, S, mt, orow=order)                               # scattered back to slot order
    ops.check_device_status()
    yn = y.cpu().numpy()
    for ex in range(E):
        rows = np.nonzero(e == ex)[0]
        if rows.size == 0:
            continue
        one = dev.expert(ex)._prefill(torch.from_numpy(x[rows]).cuda()).cpu().numpy()
        np.testing.assert_array_equal(yn[rows], one)                          # same tile arithmetic, row for row
        want = O.matmul_f64(x[rows], W[ex])
        assert O.rel_fro(yn[rows], want) <= 1e-3


@pytest.mark.parametrize("fmt,mt,limit", [("q4_k", 256, None), ("q4_k", 128, 7.0), ("q6_k", 256, None), ("nvfp4", 256, 3.0), ("q5_k", 256, None), ("q8_0", 128, 5.0), ("q2_k", 256, None), ("iq4_xs", 256, 2.0)])
def test_gated_pair_in_one_grouped_product(fmt, mt, limit):
    """gate | up as ONE grouped product with silu(a) * b in its epilogue == two grouped products + the activation launch, bit for bit (the epilogue rounds both
    products to fp16 first, as the separate launches store them), on ragged segments incl. an empty expert, segments of more than 128 and more than 256 rows,
    and slots without an expert (rows of zeros)."""
    E, n, k, S = 6, 512, 512, 1100
    g, _ = _stack(fmt, E, n, k, 30)
    u, _ = _stack(fmt, E, n, k, 31)
    rng = np.random.default_rng(32)
    e = rng.choice(E, S, p=[0.45, 0.0, 0.05, 0.2, 0.2, 0.1]).astype(np.int32)  # expert 1 empty, expert 0 ~ 500 rows
    e[5:9] = -1
    x = torch.from_numpy(synth.activations(S, k, rng)).cuda()
    order, tb, off = KQ.csort(torch.from_numpy(e).cuda(), E, mt)
    xg = KQ.gather_perm(x, order, 1)
    a = KQ.gmm(g, xg, tb, off, S, mt)
    b = KQ.gmm(u, xg, tb, off, S, mt)
    want = KQ.silu_perm(a, b, None, limit)
    gsg, gsu = (g.gs, u.gs) if fmt == "nvfp4" else (None, None)
    got = ops.gemm_kq_grouped_glu(fmt, g.t16, u.t16, n, k, E, xg, tb, off, gsg, gsu, limit, mt)
    ops.check_device_status()
    assert torch.equal(got, want)
    assert (got[S - 4:] == 0).all()                                            # the four slots without an expert sort to the tail
