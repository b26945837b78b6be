"""The numpy restatement of the NVFP4 activation codec against an independent formulation: every value maps to the nearest e2m1 point of its block scale
(ties to the even code), scales are the nearest e4m3 to amax / 6, pack / unpack round-trips are idempotent (mirrors the reference's tests/test_fp4pack.py:8-18)."""
import numpy as np

from oracle import fp4_numpy as F4, kq_numpy as O


def test_codes_are_nearest_e2m1():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((64, 256)) * np.exp(rng.uniform(-3, 3, (64, 1)))).astype(np.float16)
    x[0] = 0                                                              # an all-zero row: scale floor 6 * 2^-9 / 6 = 2^-9
    codes, sc = F4.pack(x)
    assert sc[0].tolist() == [1] * 16 and not codes[0].any()
    y = F4.unpack(codes, sc)
    scale = O.e4m3_unsigned(sc)
    grid = np.concatenate([-F4.LUT[::-1], F4.LUT])
    v = np.clip(x.astype(np.float32).reshape(64, -1, 16) / scale[..., None], -6, 6)
    best = np.abs(v[..., None] - grid).min(-1)
    got = np.abs(v - y.reshape(64, -1, 16) / np.where(scale[..., None] == 0, 1, scale[..., None]))
    np.testing.assert_allclose(got, best, atol=1e-6)
    c2, s2 = F4.pack(y)                                                   # quantising a quantised tensor changes nothing
    np.testing.assert_array_equal(F4.unpack(c2, s2), y)


def test_e4m3_rounding_table():
    tab = O.e4m3_unsigned(np.arange(127, dtype=np.uint8))
    np.testing.assert_array_equal(F4.e4m3_rn(tab), np.arange(127))
    mid = (tab[1:] + tab[:-1]) / 2                                        # exact midpoints go to the even code
    r = F4.e4m3_rn(mid)
    assert ((r % 2) == 0).all()
    assert F4.e4m3_rn(np.array([1e9]))[0] == 126                          # saturates at 448


def test_power_of_two_form():
    """Block 32 with an exponent byte: the scale is the smallest power of two with amax / scale <= 6, an all-zero block stores exponent byte 1, pack / unpack
    round-trips are idempotent."""
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((32, 256)) * np.exp(rng.uniform(-4, 4, (32, 1)))).astype(np.float16)
    x[0] = 0
    x[1, :32] = 0
    x[1, 0] = 6.0                                                         # amax / 6 exactly 1: exponent 0
    x[2, :32] = 0
    x[2, 0] = 6.0078125                                                   # one fp16 step above 6: exponent 1
    codes, sc = F4.pack(x, 32, False)
    assert sc[0].tolist() == [1] * 8 and not codes[0].any()
    assert sc[1, 0] == 127 and sc[2, 0] == 128
    scale = np.ldexp(1.0, sc.astype(np.int32) - 127)
    amax = np.abs(x.astype(np.float64)).reshape(32, -1, 32).max(-1)
    nz = amax > 0
    assert (amax[nz] / scale[nz] <= 6.0).all() and (amax[nz] / scale[nz] > 3.0).all()
    y = F4.unpack(codes, sc, 32, False)
    c2, s2 = F4.pack(y, 32, False)
    np.testing.assert_array_equal(F4.unpack(c2, s2, 32, False), y)
