"""The numpy oracle is bit-equal to ggml's dequantiser and to the reference decoder on the committed fixtures
(mirrors the reference's tests/test_gguf_types.py:26-37 and tests/test_foreign_formats.py:213-219)."""
import numpy as np
import pytest

from oracle import kq_numpy as O


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("t", ["Q4_K", "Q3_K", "Q6_K", "Q5_K", "Q8_0", "Q2_K", "IQ4_XS"])
def test_bit_equal_to_ggml(ggml_golden, t):
    raw, ref = ggml_golden[t + "_raw"], ggml_golden[t + "_ref"]
    be, bb = O.BLOCK[t]
    assert ref.size == raw.shape[0] * be
    rows2 = O.dequant(t, raw.reshape(-1, 2 * bb), 2 * be).reshape(-1)         # rows of two blocks
    np.testing.assert_array_equal(_bits(rows2), _bits(ref))
    one = O.dequant(t, raw.reshape(1, -1), ref.size).reshape(-1)              # one row of all blocks
    np.testing.assert_array_equal(_bits(one), _bits(ref))


@pytest.mark.parametrize("t", ["Q4_K", "Q3_K", "Q6_K", "NVFP4", "Q5_K", "Q8_0", "Q2_K", "IQ4_XS"])
def test_bit_equal_to_reference_decoder(ref_golden, t):
    k = int(ref_golden[t + "_k"])
    np.testing.assert_array_equal(_bits(O.dequant(t, ref_golden[t + "_raw"], k)), _bits(ref_golden[t + "_f32"]))
    if t != "NVFP4":
        np.testing.assert_array_equal(_bits(O.dequant(t, ref_golden[t + "_raw_small"], k)), _bits(ref_golden[t + "_f32_small"]))


def test_nvfp4_pack_form(ref_golden):
    k = int(ref_golden["NVFP4_k"])
    qs, meta = O.nvfp4_gguf_to_pack(ref_golden["NVFP4_raw"], k)
    np.testing.assert_array_equal(qs, ref_golden["NVFP4_pack_qs"])
    np.testing.assert_array_equal(meta, ref_golden["NVFP4_pack_meta"])
    g = float(ref_golden["NVFP4_pack_gscale"])
    np.testing.assert_array_equal(_bits(O.dequant_nvfp4_pack(qs, meta, g)), _bits(ref_golden["NVFP4_pack_f32"]))
    np.testing.assert_array_equal(_bits(O.dequant_nvfp4_pack(qs, meta, g, apply_gscale=False)), _bits(ref_golden["NVFP4_pack_f32_nog"]))
    # the two NVFP4 forms describe the same weights (the GGUF form halves the scale and doubles the table); they differ only in the
    # sign of zero (code 8) and on scale bytes with the top bit set (rows 0-1 of the fixture hold those special codes)
    np.testing.assert_array_equal(ref_golden["NVFP4_pack_f32_nog"][2:], ref_golden["NVFP4_f32"][2:])


def test_threaded_chunks_equal_single_call():
    rng = np.random.default_rng(5)
    k = 4096
    raw = rng.integers(0, 256, (2100, O.row_bytes("Q4_K", k)), dtype=np.uint8)      # more rows than one 2^22-element chunk
    raw.reshape(2100, -1, 144)[..., 0:4] = np.abs(rng.normal(0, 1e-3, (2100, k // 256, 2))).astype("<f2").view(np.uint8).reshape(2100, k // 256, 4)
    a = O.dequant("Q4_K", raw, k)
    b = O._dequant_chunk("Q4_K", raw, k)
    np.testing.assert_array_equal(_bits(a), _bits(b))


def test_bad_row_size_raises():
    with pytest.raises(ValueError):
        O.dequant("Q6_K", np.zeros((2, 100), np.uint8), 256)
    with pytest.raises(ValueError):
        O.row_bytes("Q4_K", 100)
