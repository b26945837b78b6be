"""NVFP4 tensor-core path parity (GPU): activation quantiser == the numpy restatement of kyojin_mlx/fp4pack.py bit for bit (codes and scale bytes, incl. an
all-zero row; reference test tests/test_fp4pack.py:8-18), scale re-layout round trip exact incl. zero / subnormal / 0x7F codes (tests/test_fp4tile.py:29-40),
block-scaled GEMM vs the fp64 product of the dequantised operands < 1e-3 (tests/test_fp4tile.py:58, tests/test_foreign_g2a.py:27-70)."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import fp4pack, layout as L, ops, synth
from oracle import fp4_numpy as F4, kq_numpy as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_quantiser_equals_restatement(dtype):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn((96, 512), device="cuda", generator=g) * torch.exp(torch.rand((96, 1), device="cuda", generator=g) * 6 - 3)).to(dtype)
    x[3] = 0
    x[4, :16] = 1e4 if dtype == torch.float16 else 3e4                    # large block: scale near the top of e4m3
    # a block whose scale is exactly 1 (amax 6) with values ON the rounding thresholds, one step above / below them, and a negative zero
    ties = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -0.0], device="cuda").to(dtype)
    x[5, :16] = ties
    up = (ties.view(torch.int16) + 1).view(dtype)                          # next representable value away from zero
    x[5, 16:32] = up
    x[5, 16] = 6.0
    x[5, 32:48] = (ties.view(torch.int16) - 1).view(dtype)
    x[5, 32], x[5, 47] = 6.0, 0.0
    codes, sc = fp4pack.pack(x, 16, True)
    wc, ws = F4.pack(x.float().cpu().numpy())
    np.testing.assert_array_equal(sc.cpu().numpy(), ws)
    np.testing.assert_array_equal(codes.cpu().numpy(), wc)
    y = fp4pack.unpack(codes, sc, 16, True, torch.float32)
    np.testing.assert_array_equal(y.cpu().numpy(), F4.unpack(wc, ws))
    xs = x[:, :48].contiguous()                                            # a width that is not a multiple of 64 takes the general kernel
    c2, s2 = fp4pack.pack(xs, 16, True)
    np.testing.assert_array_equal(c2.cpu().numpy(), wc[:, :24])
    np.testing.assert_array_equal(s2.cpu().numpy(), ws[:, :3])


def test_sf_layout_round_trip():
    rng = np.random.default_rng(1)
    rows, k = 200, 512
    sc = rng.integers(0, 127, (rows, k // 16), dtype=np.uint8)
    sc[0, :6] = (0x00, 0x01, 0x07, 0x08, 0x7E, 0x7F)
    swz = ops.nvfp4_sf_swizzle(torch.from_numpy(sc).cuda(), k)
    back = ops.nvfp4_sf_unswizzle(swz, rows, k).cpu().numpy()
    want = sc.copy()
    want[want == 0x7F] = 0                                               # the NaN code decodes as 0 in the reference and is stored as 0
    np.testing.assert_array_equal(back, want)
    s = swz.cpu().numpy().reshape(-1, k // 64, 512)                       # chunk layout: byte (r % 32) * 16 + (r / 32) * 4 + c
    r, j = 77, 13
    assert s[r // 128, j // 4, (r % 128 % 32) * 16 + (r % 128 // 32) * 4 + j % 4] == want[r, j]


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (256, 512, 1024), (200, 256, 768), (1024, 1024, 2048)])
def test_gemm_nvfp4_vs_fp64(m, n, k):
    rng = np.random.default_rng(m + n)
    wcodes = rng.integers(0, 16, (n, k), dtype=np.uint8)
    wsc = synth.nvfp4_scale_bytes(rng, (n, k // 16))                      # e4m3 nearest to 2^U[-8, 0]: mantissa bits and subnormals
    qs, meta = L.nvfp4_codes_to_pack(wcodes, wsc)
    w = O.dequant_nvfp4_pack(qs, meta)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    acodes, asp, asw = ops.nvfp4_quant_rows(x)
    xq = F4.unpack(acodes.cpu().numpy(), asp.cpu().numpy())
    sfb = ops.nvfp4_sf_swizzle(torch.from_numpy(wsc).cuda(), k)
    d = ops.gemm_nvfp4(acodes, asw, torch.from_numpy(qs).cuda(), sfb, m, n, k, 1.0, torch.float16)
    ops.check_device_status()
    want = xq.astype(np.float64) @ w.astype(np.float64).T
    err = O.rel_fro(d.cpu().numpy(), want)
    assert err < 1e-3, err
    d2 = ops.gemm_nvfp4(acodes, asw, torch.from_numpy(qs).cuda(), sfb, m, n, k, 0.25, torch.bfloat16)
    assert O.rel_fro(d2.float().cpu().numpy(), want * 0.25) < 5e-3       # bf16 output rounding


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_power_of_two_form_equals_restatement(dtype):
    """fp4pack with block = 32 and power-of-two scales: codes and exponent bytes equal to the numpy restatement, incl. an all-zero block, amax / 6 exactly a power
    of two and one step above it; unpack equal in fp32."""
    g = torch.Generator(device="cuda").manual_seed(2)
    x = (torch.randn((64, 512), device="cuda", generator=g) * torch.exp(torch.rand((64, 1), device="cuda", generator=g) * 8 - 4)).to(dtype)
    x[3] = 0
    x[4, :32] = 0
    x[4, 0] = 6.0
    x[5, :32] = 0
    x[5, 0] = (torch.tensor([6.0], device="cuda").to(dtype).view(torch.int16) + 1).view(dtype)[0]
    x[6, :32] = torch.tensor([3.0, -1.5, 0.75, -0.25, 0.25001, 5.0, -5.5, 1.75] * 4, device="cuda").to(dtype)
    codes, sc = fp4pack.pack(x, 32, False)
    wc, ws = F4.pack(x.float().cpu().numpy(), 32, False)
    np.testing.assert_array_equal(sc.cpu().numpy(), ws)
    np.testing.assert_array_equal(codes.cpu().numpy(), wc)
    np.testing.assert_array_equal(fp4pack.unpack(codes, sc, 32, False, torch.float32).cpu().numpy(), F4.unpack(wc, ws, 32, False))
    with pytest.raises(ValueError):
        fp4pack.pack(x, 32, True)
