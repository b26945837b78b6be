"""Prefill GEMM parity (GPU): tcgen05 fp16 GEMM against torch fp32 / the fp64 dequant-then-matmul oracle; mirrors the reference's large-row checks
(tests/test_foreign_formats.py:321-339: R = 24, 70 through dequant + matmul, max-abs <= 4e-3 max|ref|) with the benchmark's 1e-3 Frobenius bound."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_pack as FP, ops, synth
from kyojin_mac_b200.foreign_linear import ForeignLinear
from oracle import kq_numpy as O

pytestmark = pytest.mark.gpu
T = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 256), (256, 512, 1024), (70, 200, 320), (1000, 1300, 2048), (2048, 3072, 3072)])
def test_gemm_f16_vs_fp32(m, n, k):
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    b = (torch.randn((n, k), device="cuda", generator=g) * 0.05).to(torch.float16)
    d = ops.gemm_f16(a, b)
    ops.check_device_status()
    want = a.double() @ b.double().T
    err = (torch.linalg.norm(d.double() - want) / torch.linalg.norm(want)).item()
    assert err < 5e-4, err                                    # fp16 output rounding only (2^-11 relative per element)
    assert (d.double() - want).abs().max().item() <= 2e-3 * want.abs().max().item()


def test_gemm_f16_exact_small_integers():
    """Integer-valued operands: every product and partial sum is exact in fp32, so the result must be exact."""
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-3, 4, (256, 512), device="cuda", generator=g).to(torch.float16)
    b = torch.randint(-3, 4, (384, 512), device="cuda", generator=g).to(torch.float16)
    d = ops.gemm_f16(a, b)
    assert torch.equal(d.float(), a.float() @ b.float().T)


def test_gemm_saturates_and_scales():
    a = torch.full((128, 64), 100.0, dtype=torch.float16, device="cuda")
    b = torch.full((128, 64), 100.0, dtype=torch.float16, device="cuda")
    d = ops.gemm_f16(a, b)
    assert torch.isfinite(d).all() and (d == 65504).all()
    d2 = ops.gemm_f16(a, b, gscale=1e-3)
    torch.testing.assert_close(d2.float(), torch.full((128, 128), 640.0, device="cuda"), rtol=1e-3, atol=0)
    d3 = ops.gemm_f16(-a, b)
    assert (d3 == -65504).all()
    a[5, 7] = float("nan")                                     # a NaN is not turned into a finite value by the saturation
    d4 = ops.gemm_f16(a, b)
    assert torch.isnan(d4[5]).all() and (d4[:5] == 65504).all() and (d4[6:] == 65504).all()


@pytest.mark.parametrize("fmt", ["q3_k", "q4_k", "q6_k", "nvfp4", "q5_k", "q8_0", "q2_k", "iq4_xs"])
@pytest.mark.parametrize("rows", [70, 300])
def test_linear_prefill_vs_fp64(fmt, rows):
    n, k = 384, 1024
    rng = np.random.default_rng(rows)
    raw = synth.raw_blocks(fmt, n, k, rng)
    x = synth.activations(rows, k, rng)
    w = O.dequant(T[fmt], raw, k)
    lin = ForeignLinear(FP.to_pack(T[fmt], raw, k))
    y = lin(torch.from_numpy(x).cuda()).cpu().numpy()
    ops.check_device_status()
    want = O.matmul_f64(x, w)
    err, ref_err = O.rel_fro(y, want), O.rel_fro(O.matmul_ref_path(x, w), want)
    assert err <= 1e-3 and err <= 2 * ref_err + 1e-6, (err, ref_err)
    assert np.abs(y.astype(np.float64) - want).max() <= 4e-3 * np.abs(want).max()


@pytest.mark.parametrize("fmt", ["q3_k", "q4_k", "q6_k", "nvfp4", "q5_k", "q8_0", "q2_k", "iq4_xs"])
def test_fused_decode_gemm_vs_staged(fmt):
    """Weights decoded inside the GEMM: the CTA-pair kernel (the default for more than 128 rows) and the one-CTA kernel with one and two activation blocks per
    work item give the same bits; NVFP4 equals the staged form bit for bit (its fp16
    weights are exact), K-quants stay within the accuracy bound and within a few fp16 roundings of the staged form."""
    n, k, m = 1040, 2048, 520                                               # n and m with ragged last tiles
    t16 = synth.t16_random_device(fmt, n, k, seed=11)
    g = torch.Generator(device="cuda").manual_seed(12)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    y1 = ops.gemm_kq(fmt, t16, n, k, x, msub=1)
    y2 = ops.gemm_kq(fmt, t16, n, k, x, msub=2)
    y0 = ops.gemm_kq(fmt, t16, n, k, x)
    ops.check_device_status()
    assert torch.equal(y1, y2) and torch.equal(y0, y1)
    w16 = ops.dequant(fmt, t16, n, k, torch.float16)
    staged = ops.gemm_f16(x, w16)
    if fmt == "nvfp4":
        assert torch.equal(y1, staged)
    want = x.double() @ ops.dequant(fmt, t16, n, k, torch.float32).double().T
    err = ((y1.double() - want).norm() / want.norm()).item()
    err_staged = ((staged.double() - want).norm() / want.norm()).item()
    assert err <= 1e-3 and err <= 2.5 * err_staged + 1e-6, (err, err_staged)
    ys = ops.gemm_kq(fmt, t16, n, k, x[:3], gscale=0.5)                      # a short block of rows, output scale
    assert torch.allclose(ys.float(), y1[:3].float() * 0.5, rtol=2e-3, atol=1e-4)


@pytest.mark.parametrize("fmt", ["q4_k", "q3_k", "q6_k", "nvfp4"])
def test_split_k_adds_the_ranges_in_k_order(fmt):
    """Split-k (tile, k-range) items + the pass that adds the ranges: deterministic, within the accuracy bound, and within fp32 summation-order distance of the
    unsplit product; ragged last tiles in both directions; the workspace is checked."""
    from kyojin_mac_b200 import _lib
    n, k, m = 1040, 4096, 520
    t16 = synth.t16_random_device(fmt, n, k, seed=21)
    g = torch.Generator(device="cuda").manual_seed(22)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    y1 = ops.gemm_kq(fmt, t16, n, k, x, split=1)
    want = x.double() @ ops.dequant(fmt, t16, n, k, torch.float32).double().T
    err1 = ((y1.double() - want).norm() / want.norm()).item()
    for sp in (2, 4, 8):
        ys = ops.gemm_kq(fmt, t16, n, k, x, split=sp)
        assert torch.equal(ys, ops.gemm_kq(fmt, t16, n, k, x, split=sp))
        err = ((ys.double() - want).norm() / want.norm()).item()
        assert err <= 1e-3 and err <= 1.5 * err1 + 1e-6, (sp, err, err1)
        assert torch.allclose(ys.float(), y1.float(), rtol=2e-3, atol=2e-3 * want.abs().max().item())
    ops.check_device_status()
    L = _lib.lib()
    assert L.kyb_gemm_kq_split(ops._fmt("q3_k"), 768, 12288, 2048) == 6                       # 24 tiles of 256 x 256 on 148 SMs: sixths fill one round
    assert L.kyb_gemm_kq_split(ops._fmt("q3_k"), 12288, 3072, 2048) == 1 and L.kyb_gemm_kq_split(ops._fmt(fmt), n, 2048, m) == 1
    y = torch.empty((m, n), dtype=torch.float16, device="cuda")
    small = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    rc = L.kyb_gemm_kq_splitk(ops._fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), x.stride(0), m, 1.0, y.data_ptr(), y.stride(0), 2, small.data_ptr(), small.numel(), 0)
    assert rc == _lib.EWORKSPACE
    rc = L.kyb_gemm_kq_splitk(ops._fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), x.stride(0), m, 1.0, y.data_ptr(), y.stride(0), 3, small.data_ptr(), small.numel(), 0)
    assert rc != 0                                                                            # 16 blocks do not split into 3 equal ranges


def test_gather_epilogue_writes_every_destination():
    """The GEMM + all-gather entry points on one GPU: two 'ranks' (two shards, two output matrices in this process), every shard's tiles land in both matrices
    at the shard's column offset; the result equals the plain GEMM of each shard."""
    k, m, shards = 1024, 200, [(0, 512), (512, 272)]                       # second shard with a ragged last tile
    n_total = 784
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
    outs = [torch.zeros((m, n_total), dtype=torch.float16, device="cuda") for _ in range(2)]
    want = torch.zeros((m, n_total), dtype=torch.float16, device="cuda")
    for col0, n in shards:
        t16 = synth.t16_random_device("q4_k", n, k, seed=col0 + 1)
        ops.gemm_kq_ag("q4_k", t16, n, k, x, [o.data_ptr() for o in outs], n_total, col0)
        want[:, col0:col0 + n] = ops.gemm_kq("q4_k", t16, n, k, x)
    ops.check_device_status()
    assert torch.equal(outs[0], want) and torch.equal(outs[1], want)
    # NVFP4 W4A4 form
    from kyojin_mac_b200.foreign_linear import DevPack
    n_total, outs = 768, [torch.zeros((m, 768), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    want = torch.zeros((m, 768), dtype=torch.bfloat16, device="cuda")
    codes, _, asw = ops.nvfp4_quant_rows(x.to(torch.bfloat16), swizzled=True, plain=False)
    for col0, n in [(0, 512), (512, 256)]:
        dp = DevPack.from_t16("nvfp4", synth.t16_random_device("nvfp4", n, k, seed=col0 + 7), n, k)
        qs, sfb = dp._a4_operands()
        ops.gemm_nvfp4_ag(codes, asw, qs, sfb, m, n, k, [o.data_ptr() for o in outs], n_total, col0, 1.0, torch.bfloat16)
        want[:, col0:col0 + n] = ops.gemm_nvfp4(codes, asw, qs, sfb, m, n, k, 1.0, torch.bfloat16)
    ops.check_device_status()
    assert torch.equal(outs[0], want) and torch.equal(outs[1], want)


def test_gemm_errors():
    a = torch.zeros((128, 96), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.gemm_f16(a, a)                                     # k % 64 != 0
    with pytest.raises(ValueError):
        ops.gemm_f16(a.float(), a.float())
