"""Parity at the benchmark's full sizes (GPU): the Q3_K prefill GEMM at hidden 3072 (both shapes, M = 2048, one and two activation blocks per work item),
the NVFP4 W4A4 GEMM 4096 x 7168 -> 18432 with scale bytes drawn into the e4m3 subnormal range, and the routed-expert layer with 256 experts, top-8, hidden 7168
at 64 and 4096 tokens. Small shapes do not make the persistent schedulers wrap, do not fill both accumulators, and draw few subnormal scales; these do.

Two checks per case. (1) A seeded sample of output rows / columns against the ORACLE: the stored blocks of the sampled weight rows are taken back from the
device tiles (the repack is a tested bit permutation), decoded by the numpy oracle and multiplied in fp64: rel. Frobenius <= 1e-3 and <= 2 x the error of the
reference path's own arithmetic (fp16-staged weights), as tests/test_foreign_formats.py:319-339 and tests/test_kq_rt2.py:31-54 of the reference do at their
sizes. (2) Every output element against an fp64 product on the device whose weights come from this library's own decoder; that decoder is pinned bit-exactly on
the golden vectors in test_gpu_dequant.py, so this covers every tile of the schedule, not only the sample."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_kqgmm as KQ, ops, synth
from kyojin_mac_b200.foreign_linear import DevPack, ForeignSwitchGLU
from oracle import fp4_numpy as F4, kq_numpy as O, moe_numpy as M

pytestmark = pytest.mark.gpu
T_ = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}


class _Experts(dict):
    """Decoded weights of the experts a sample touches, indexed by expert id like the [E, n, k] array the oracle's layer takes."""

    def __init__(self, shape):
        super().__init__()
        self.shape = shape


def _sample(rng, total, count):
    """`count` distinct indices incl. the first and the last."""
    idx = rng.choice(total, size=min(count, total), replace=False)
    idx[0], idx[-1] = 0, total - 1
    return np.unique(idx)


def _oracle_rows(fmt, t16, n, k, rows):
    """float32 [len(rows), k]: the oracle's decode of the stored blocks of the given rows."""
    raw = ops.t16_to_raw(fmt, t16, n, k)[torch.from_numpy(rows).cuda()].cpu().numpy()
    return O.dequant(T_[fmt], raw, k)


def _device_rel_fro(y, x, w32):
    want = x.double() @ w32.double().T
    return float(torch.linalg.norm(y.double() - want) / torch.linalg.norm(want))


@pytest.mark.parametrize("n,k", [(12288, 3072), (3072, 12288)])
@pytest.mark.parametrize("msub", [1, 2])
def test_q3k_prefill_gemm_full_size(n, k, msub):
    m = 2048
    t16 = synth.t16_random_device("q3_k", n, k, seed=n + msub)
    g = torch.Generator(device="cuda").manual_seed(k)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    y = ops.gemm_kq("q3_k", t16, n, k, x, msub=msub)
    ops.check_device_status()
    rng = np.random.default_rng(n * 3 + msub)
    rows, toks = _sample(rng, n, 64), _sample(rng, m, 512)
    w = _oracle_rows("q3_k", t16, n, k, rows)
    xs = x[torch.from_numpy(toks).cuda()].cpu().numpy()
    got = y[torch.from_numpy(toks).cuda()][:, torch.from_numpy(rows).cuda()].cpu().numpy()
    want = O.matmul_f64(xs, w)
    err, ref_err = O.rel_fro(got, want), O.rel_fro(O.matmul_ref_path(xs, w), want)
    assert err <= 1e-3 and err <= 2 * ref_err + 1e-6, (err, ref_err)
    assert np.abs(got.astype(np.float64) - want).max() <= 4e-3 * np.abs(want).max()
    w32 = ops.dequant("q3_k", t16, n, k, torch.float32)
    assert np.array_equal(w32[torch.from_numpy(rows).cuda()].cpu().numpy().view(np.uint32), w.view(np.uint32))     # the decoder is bit-exact at this size too
    assert _device_rel_fro(y, x, w32) <= 1e-3


def test_nvfp4_w4a4_gemm_full_size():
    n, k, m = 18432, 7168, 4096
    dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", n, k, seed=3), n, k)       # scale bytes e4m3(2^U[-8, 0]): a quarter lie in the subnormal range
    g = torch.Generator(device="cuda").manual_seed(33)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.bfloat16)
    y = dp.apply_a4(x, torch.float16)
    ops.check_device_status()
    rng = np.random.default_rng(5)
    rows, toks = _sample(rng, n, 64), _sample(rng, m, 256)
    w = _oracle_rows("nvfp4", dp.t16, n, k, rows)
    sc = ops.t16_to_raw("nvfp4", dp.t16, n, k).reshape(n, k // 64, 36)[:, :, :4]
    assert int(((sc & 0x78) == 0).sum()) > n * (k // 16) // 10               # plenty of subnormal (exponent 0) weight scales in the draw
    tk = torch.from_numpy(toks).cuda()
    acodes, asp, _ = ops.nvfp4_quant_rows(x[tk].contiguous(), swizzled=False, plain=True)
    wc, ws = F4.pack(x[tk].float().cpu().numpy())                            # the activation codec restated in numpy
    np.testing.assert_array_equal(acodes.cpu().numpy(), wc)
    np.testing.assert_array_equal(asp.cpu().numpy(), ws)
    want = F4.unpack(wc, ws).astype(np.float64) @ w.astype(np.float64).T
    got = y[tk][:, torch.from_numpy(rows).cuda()].cpu().numpy()
    err = O.rel_fro(got, want)
    assert err <= 1e-3, err                                                  # both operands are exact products of 4-bit values and scales: fp16 output rounding only
    # every element: the dequantised activations (device unpack, equal to the restatement above on the sample) times the device-decoded weights, in fp64 in slabs
    ac, ap, _ = ops.nvfp4_quant_rows(x, swizzled=False, plain=True)
    xq = ops.nvfp4_unpack_rows(ac, ap, torch.float32)
    num = den = 0.0
    for r0 in range(0, n, 4608):
        w32 = ops.dequant("nvfp4", dp.t16, n, k, torch.float32, 1.0, r0, 4608)
        wantd = xq.double() @ w32.double().T
        num += float(((y[:, r0:r0 + 4608].double() - wantd) ** 2).sum())
        den += float((wantd ** 2).sum())
    assert (num / den) ** 0.5 <= 1e-3


@pytest.mark.parametrize("T", [64, 4096])
def test_routed_layer_full_size(T):
    E, H, I, K = 256, 7168, 2048, 8
    mk = lambda rows, k_, seed: DevPack.from_t16("q4_k", synth.t16_random_device("q4_k", E * rows, k_, seed=seed), rows, k_, E)
    gq, uq, dq = mk(I, H, 40), mk(I, H, 41), mk(H, I, 42)
    blk = ForeignSwitchGLU(gq, uq, dq)
    g = torch.Generator(device="cuda").manual_seed(T)
    x = (torch.randn((T, H), device="cuda", generator=g) * 0.5).to(torch.float16)
    lg = torch.randn((T, E), device="cuda", generator=g)                     # router logits N(0, 1); top-8 weights renormalised
    inds, scs, _ = ops.moe_select(lg, E, K, True)
    y = blk(x, inds.reshape(T, K))
    ops.check_device_status()
    assert y.shape == (T, K, H) and bool(torch.isfinite(y).all())
    ie = inds.cpu().numpy().reshape(T, K)
    if T * K > max(256, 4 * E):
        # the sorted plan at this size: tiles cover every slot exactly once
        for mt in (128, 256):
            order, tb, off = KQ.csort(inds, E, mt)
            cnt, woff, wtb = M.host_plan(ie, E, mt)
            np.testing.assert_array_equal(off.cpu().numpy().astype(np.uint32), woff)
            np.testing.assert_array_equal(tb.cpu().numpy().astype(np.uint32), wtb)
            o, tbn, offn = order.cpu().numpy(), tb.cpu().numpy(), off.cpu().numpy()
            assert sorted(o.tolist()) == list(range(T * K)) and (np.diff(ie.reshape(-1)[o]) >= 0).all()
            seen = np.zeros(T * K, np.int32)
            for e in range(E):
                for tile in range(tbn[e], tbn[e + 1]):
                    r0 = offn[e] + (tile - tbn[e]) * mt
                    seen[r0:min(r0 + mt, offn[e + 1])] += 1
            assert (seen == 1).all()
    # sample of tokens against the fp64 layer built from the oracle's decode of the experts those tokens use
    rng = np.random.default_rng(T)
    toks = _sample(rng, T, 6)
    used = np.unique(ie[toks])
    def stack(dev):
        W = _Experts((E, dev.n, dev.k))
        for e in used:
            ex = dev.expert(int(e))
            W[int(e)] = O.dequant("Q4_K", ops.t16_to_raw("q4_k", ex.t16, ex.n, ex.k).cpu().numpy(), ex.k)
        return W
    Wg, Wu, Wd = stack(gq), stack(uq), stack(dq)
    xs = x[torch.from_numpy(toks).cuda()].cpu().numpy()
    want = M.routed_layer(xs, ie[toks], Wg, Wu, Wd, K, ref_path=False)
    refp = M.routed_layer(xs, ie[toks], Wg, Wu, Wd, K, ref_path=True)
    got = y[torch.from_numpy(toks).cuda()].reshape(len(toks) * K, H).cpu().numpy()
    err, ref_err = O.rel_fro(got, want), O.rel_fro(refp, want)
    assert err <= 2e-3 and err <= 2 * ref_err + 1e-6, (err, ref_err)         # two fp16 roundings on the way (a | b, h), as on the reference path
    # the two routed paths (gathered GEMV with election, sorted grouped GEMM) agree on the same slots to fp16 rounding of their intermediates
    if T == 64:
        y2 = KQ.mlp(blk, x, inds, K).reshape(T, K, H)
        assert float(torch.linalg.norm(y2.double() - y.double()) / torch.linalg.norm(y.double())) <= 2e-3
