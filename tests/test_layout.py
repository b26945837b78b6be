"""T16 repack: lossless, invertible, same byte count as the GGUF blocks (mirrors the reference's lossless-repack checks,
tests/test_foreign_formats.py:213-219 and the tile round trip of tests/test_fp4tile.py:29-40)."""
import numpy as np
import pytest

from kyojin_mac_b200 import layout as L


def _raw(fmt, n, k, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, 256, (n, L.raw_row_bytes(fmt, k)), dtype=np.uint8)


@pytest.mark.parametrize("fmt", L.FORMATS)
@pytest.mark.parametrize("n,k", [(16, 256), (48, 1024), (5, 512), (33, 256)])
def test_round_trip_exact(fmt, n, k):
    raw = _raw(fmt, n, k, 3)
    t = L.raw_to_t16(fmt, raw, n, k)
    assert t.dtype == np.uint8 and t.size == L.t16_nbytes(fmt, n, k)
    np.testing.assert_array_equal(L.t16_to_raw(fmt, t, n, k), raw)


@pytest.mark.parametrize("fmt", L.FORMATS)
def test_same_byte_count_as_stored(fmt):
    n, k = 64, 2048
    assert L.t16_nbytes(fmt, n, k) == n * L.raw_row_bytes(fmt, k)


@pytest.mark.parametrize("fmt", L.FORMATS)
def test_bit_permutation(fmt):
    """Every stored bit lands in exactly one T16 bit: flipping one input bit flips exactly one output bit."""
    n, k = 16, 256
    base = np.zeros((n, L.raw_row_bytes(fmt, k)), np.uint8)
    t0 = L.raw_to_t16(fmt, base, n, k)
    seen = set()
    rng = np.random.default_rng(0)
    for _ in range(200):
        r, by, bit = int(rng.integers(n)), int(rng.integers(base.shape[1])), int(rng.integers(8))
        x = base.copy()
        x[r, by] = 1 << bit
        d = np.unpackbits(L.raw_to_t16(fmt, x, n, k) ^ t0)
        assert d.sum() == 1
        seen.add(int(np.flatnonzero(d)[0]))
    assert len(seen) > 150                                                       # distinct inputs -> distinct outputs


def test_padding_rows_are_zero_blocks():
    raw = _raw("q6_k", 5, 256, 1)
    t = L.raw_to_t16("q6_k", raw, 5, 256)
    full = L.t16_to_raw("q6_k", t, 16, 256)
    np.testing.assert_array_equal(full[:5], raw)
    assert not full[5:].any()


def test_nvfp4_pack_forms_agree():
    rng = np.random.default_rng(2)
    n, k = 32, 512
    raw = _raw("nvfp4", n, k, 4)
    codes, sc = L.nvfp4_raw_to_codes(raw, k)
    np.testing.assert_array_equal(L.nvfp4_codes_to_raw(codes, sc), raw)
    qs, meta = L.nvfp4_codes_to_pack(codes, sc)
    c2, s2 = L.nvfp4_pack_to_codes(qs, meta)
    np.testing.assert_array_equal(c2, codes)
    np.testing.assert_array_equal(s2, sc)
    np.testing.assert_array_equal(L.nvfp4_codes_to_t16(codes, sc), L.raw_to_t16("nvfp4", raw, n, k))


def test_bad_shapes_raise():
    with pytest.raises(ValueError):
        L.raw_to_t16("q4_k", np.zeros((4, 100), np.uint8), 4, 256)
    with pytest.raises(ValueError):
        L.t16_nbytes("q4_k", 16, 100)
    with pytest.raises(ValueError):
        L.t16_nbytes("iq3_s", 16, 256)
