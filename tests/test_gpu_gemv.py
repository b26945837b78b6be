"""Decode GEMV parity (GPU) against the fp64 dequant-then-matmul oracle; tolerances follow the reference's own
(tests/test_foreign_formats.py:319-339 max-abs 4e-3, tests/test_types2_metal.py:24-28 2e-3) and the benchmark contract:
relative Frobenius error <= 1e-3 and <= 2x the error of the reference path's arithmetic (fp16-staged weights)."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import layout as L, ops, synth
from oracle import kq_numpy as O

pytestmark = pytest.mark.gpu
T = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}
REL_FRO = 1e-3          # benchmark contract
MAX_ABS = 2e-3          # reference's K-class tolerance, relative to max |want|


def _case(fmt, n, k, m, seed):
    rng = np.random.default_rng(seed)
    raw = synth.raw_blocks(fmt, n, k, rng)
    x = synth.activations(m, k, rng)
    w = O.dequant(T[fmt], raw, k)
    return raw, x, w


def _check(y, x, w):
    want = O.matmul_f64(x, w)
    err = O.rel_fro(y, want)
    ref_err = O.rel_fro(O.matmul_ref_path(x, w), want)
    assert err <= REL_FRO, f"rel. Frobenius {err:.3e}"
    assert err <= 2 * ref_err + 1e-6, f"error {err:.3e} above twice the reference path's {ref_err:.3e}"
    assert np.abs(y.astype(np.float64) - want).max() <= MAX_ABS * np.abs(want).max()


@pytest.mark.parametrize("fmt", L.FORMATS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 16, 24, 32])
def test_gemv_vs_fp64(fmt, m):
    n, k = 192, 1024
    raw, x, w = _case(fmt, n, k, m, 11 + m)
    t16 = ops.to_device_t16(fmt, raw, n, k)
    y = ops.gemv(fmt, t16, n, k, torch.from_numpy(x).cuda()).cpu().numpy()
    ops.check_device_status()
    assert y.shape == (m, n) and y.dtype == np.float16
    _check(y, x, w)


@pytest.mark.parametrize("fmt", L.FORMATS)
@pytest.mark.parametrize("n,k", [(1000, 2560), (16, 256), (4096, 4096), (40, 7168)])
def test_gemv_shapes(fmt, n, k):
    raw, x, w = _case(fmt, n, k, 4, n + k)
    t16 = ops.to_device_t16(fmt, raw, n, k)
    y = ops.gemv(fmt, t16, n, k, torch.from_numpy(x).cuda()).cpu().numpy()
    ops.check_device_status()
    _check(y, x, w)


@pytest.mark.parametrize("fmt", L.FORMATS)
def test_rows_invariant(fmt):
    """Row r of an m = 8 (and m = 32) call equals the m = 1 call on that row, bit for bit (reference: tests/test_q4mma.py:24-45)."""
    n, k = 512, 5120
    raw, x, _ = _case(fmt, n, k, 32, 3)
    t16 = ops.to_device_t16(fmt, raw, n, k)
    xd = torch.from_numpy(x).cuda()
    y32 = ops.gemv(fmt, t16, n, k, xd)
    y8 = ops.gemv(fmt, t16, n, k, xd[:8])
    for r in (0, 3, 7):
        y1 = ops.gemv(fmt, t16, n, k, xd[r:r + 1])
        assert torch.equal(y1[0], y8[r]) and torch.equal(y1[0], y32[r])
    y1 = ops.gemv(fmt, t16, n, k, xd[20:21])
    assert torch.equal(y1[0], y32[20])


def test_gemv_saturates_and_scales():
    """fp16 output saturates at +-65504 (never inf) and the NVFP4 per-tensor scale multiplies the fp32 result once."""
    n, k = 64, 1024
    rng = np.random.default_rng(5)
    raw = synth.raw_blocks("q4_k", n, k, rng, d_sigma=50.0)                         # huge scales -> overflow
    x = synth.activations(2, k, rng)
    y = ops.gemv("q4_k", ops.to_device_t16("q4_k", raw, n, k), n, k, torch.from_numpy(x).cuda())
    assert torch.isfinite(y).all() and (y.abs() == 65504).any()
    raw = synth.raw_blocks("nvfp4", n, k, rng)
    t16 = ops.to_device_t16("nvfp4", raw, n, k)
    xd = torch.from_numpy(x).cuda()
    y1 = ops.gemv("nvfp4", t16, n, k, xd, gscale=1.0).float()
    yg = ops.gemv("nvfp4", t16, n, k, xd, gscale=0.03125).float()
    torch.testing.assert_close(yg, y1 * 0.03125, rtol=2e-3, atol=1e-4)


def test_gemv_nvfp4_special_scale_codes():
    """Scale bytes 0x00, 0x7F (NaN code -> 0), subnormals and signed codes decode as the reference's pack-form decoder does."""
    n, k = 16, 256
    rng = np.random.default_rng(9)
    codes = rng.integers(0, 16, (n, k), dtype=np.uint8)
    sc = rng.integers(0x28, 0x46, (n, k // 16), dtype=np.uint8)
    sc[0, :8] = (0x00, 0x7F, 0x01, 0x07, 0x08, 0x7E, 0x80 | 0x38, 0xFF)
    qs, meta = L.nvfp4_codes_to_pack(codes, sc)
    w = O.dequant_nvfp4_pack(qs, meta)
    t16 = torch.from_numpy(L.nvfp4_codes_to_t16(codes, sc)).cuda()
    got = ops.dequant("nvfp4", t16, n, k, torch.float32).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), w.view(np.uint32))
    x = (synth.activations(1, k, rng).astype(np.float32) * 0.01).astype(np.float16)  # keep 448-scaled rows inside fp16
    y = ops.gemv("nvfp4", t16, n, k, torch.from_numpy(x).cuda()).cpu().numpy()
    want = O.matmul_f64(x, w)
    assert O.rel_fro(y, want) <= REL_FRO


def test_gemv_errors():
    t = torch.zeros(2304, dtype=torch.uint8, device="cuda")
    x = torch.zeros((1, 256), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.gemv("q4_k", t, 16, 256, x.float())
    with pytest.raises(ValueError):
        ops.gemv("q4_k", t, 16, 256, x.cpu())
    with pytest.raises(Exception):
        ops.gemv("q4_k", t, 16, 256, torch.zeros((40, 256), dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        ops.gemv("q9_k", t, 16, 256, x)


@pytest.mark.parametrize("fmt,n,k", [("q4_k", 27648, 5120), ("q6_k", 5120, 27648), ("q4_k", 1024, 5120)])
def test_full_size_properties(fmt, n, k):
    """Benchmark-size matrices: GEMV == dequant kernel (bit-exact weights) + fp32 matmul within tolerance, and linear in x."""
    t16 = synth.t16_random_device(fmt, n, k, seed=1)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((8, k), device="cuda", generator=g).to(torch.float16)
    y = ops.gemv(fmt, t16, n, k, x).float()
    ops.check_device_status()
    want = torch.zeros((8, n), dtype=torch.float64, device="cuda")
    for r0 in range(0, n, 4096):                                                    # dequant in row slabs to bound memory
        nr = min(4096, n - r0)
        w = ops.dequant(fmt, t16, n, k, torch.float32, row0=r0, nrows=nr)
        want[:, r0:r0 + nr] = x.double() @ w.double().T
    err = (torch.linalg.norm(y.double() - want) / torch.linalg.norm(want)).item()
    assert err <= REL_FRO, err
    # linearity: W(2x) = 2 W x exactly (power-of-two scaling commutes with every rounding, no overflow at these magnitudes)
    y2 = ops.gemv(fmt, t16, n, k, (x * 2).to(torch.float16)).float()
    assert torch.equal(y2, y * 2)


FORMS = {"whole row tiles per warp": 1, "runs of chunks + finalize launch": 0, "whole row tiles per CTA, sums in shared memory": 2}


@pytest.mark.parametrize("fmt,n,k,m,form", [("q4_k", 512, 5120, 8, 0), ("q6_k", 1024, 8192, 3, 2), ("q4_k", 10240, 5120, 1, 2), ("q6_k", 5120, 27648, 8, 0), ("q3_k", 48, 3072, 5, 0),
                                            ("q4_k", 4096, 4096, 8, 2), ("q4_k", 5120, 8192, 8, 2), ("q5_k", 1030, 2560, 2, 2), ("q4_k", 55296, 5120, 2, 1)])
def test_product_equals_exposed_partial_sums(fmt, n, k, m, form):
    """The product == the two-step entry points whose chunk sums are all written out (mma_gemv.partial_mma) and added in k order (finalize_rows), bit for bit,
    call after call, plain and chained launches, whichever of its three ways the library deals the work (the cases cover all three; n = 1030 ends inside a row
    tile)."""
    from kyojin_mac_b200 import mma_gemv
    from kyojin_mac_b200.foreign_linear import DevPack
    assert ops.gemv_plan(fmt, n, k, m)["aligned"] == form, ops.gemv_plan(fmt, n, k, m)
    assert (ops.gemv_workspace_bytes(fmt, n, k, m) > 0) == (form == 0)
    t16 = synth.t16_random_device(fmt, n, k, seed=3)
    g = torch.Generator(device="cuda").manual_seed(4)
    dev = DevPack.from_t16(fmt, t16, n, k)
    for _ in range(3):
        x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
        want = mma_gemv.finalize_rows(dev, mma_gemv.partial_mma(dev, x, m), m)
        assert torch.equal(ops.gemv(fmt, t16, n, k, x), want)
        assert torch.equal(ops.gemv(fmt, t16, n, k, x, chained=True), want)
        assert torch.equal(ops.gemv(fmt, t16, n, k, x, chained=True), want)             # ... directly behind another chained product
    ops.check_device_status()


@pytest.mark.parametrize("fmt,n,k,m", [("q6_k", 512, 2048, 1), ("q4_k", 4096, 1024, 7), ("q4_k", 640, 5120, 20)])
def test_gated_input_formed_while_staging(fmt, n, k, m):
    """DevPack.apply_glu on decode rows: the activation fp16(silu(a) * b) is formed inside the product's staging. Equal, bit for bit, to the plain product on the
    output of the activation kernel (another kernel; that one agrees with the numpy restatement of the activation to one fp16 step: the device and the host
    exponential may differ in the last place), with and without the clamp."""
    from kyojin_mac_b200.foreign_linear import DevPack
    from oracle import moe_numpy as M
    dev = DevPack.from_t16(fmt, synth.t16_random_device(fmt, n, k, seed=8), n, k)
    rng = np.random.default_rng(m)
    a, b = synth.activations(m, k, rng), synth.activations(m, k, rng)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    for limit in (None, 0.75):
        h = ops.silu_mul(ad, bd, limit)
        np.testing.assert_allclose(h.float().cpu().numpy(), M.glu(a, b, limit).astype(np.float32), rtol=1.1e-3, atol=1e-7)
        assert torch.equal(dev.apply_glu(ad, bd, limit), dev.apply(h)), limit
    ops.check_device_status()
