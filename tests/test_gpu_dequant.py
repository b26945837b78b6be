"""CUDA dequant and repack parity (GPU): bit-exact against ggml's golden vectors, the reference decoder fixtures and the numpy
oracle; mirrors the reference's tests/test_gguf_types.py:26-37 and tests/test_foreign_formats.py:159-165,213-219."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import layout as L, ops, synth
from oracle import kq_numpy as O

pytestmark = pytest.mark.gpu
T = {"q4_k": "Q4_K", "q6_k": "Q6_K", "q3_k": "Q3_K", "nvfp4": "NVFP4", "q5_k": "Q5_K", "q8_0": "Q8_0", "q2_k": "Q2_K", "iq4_xs": "IQ4_XS"}


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _deq32(fmt, raw, n, k, **kw):
    return ops.dequant(fmt, ops.to_device_t16(fmt, raw, n, k), n, k, torch.float32, **kw).cpu().numpy()


@pytest.mark.parametrize("fmt", L.FORMATS)
@pytest.mark.parametrize("n,k", [(16, 256), (37, 512), (64, 2048)])
def test_device_repack_equals_numpy_and_inverts(fmt, n, k):
    raw = np.random.default_rng(n + k).integers(0, 256, (n, L.raw_row_bytes(fmt, k)), dtype=np.uint8)
    dev = ops.to_device_t16(fmt, raw, n, k)
    np.testing.assert_array_equal(dev.cpu().numpy(), L.raw_to_t16(fmt, raw, n, k))
    np.testing.assert_array_equal(ops.t16_to_raw(fmt, dev, n, k).cpu().numpy(), raw)


@pytest.mark.parametrize("fmt", ["q4_k", "q3_k", "q6_k", "q5_k", "q8_0", "q2_k", "iq4_xs"])
def test_dequant_kat_ggml(ggml_golden, fmt):
    raw, ref = ggml_golden[T[fmt] + "_raw"], ggml_golden[T[fmt] + "_ref"]
    if fmt == "q8_0":                                                              # 36 blocks of 32 in the fixture: the first 32 make whole 256-input blocks
        raw, ref = raw[:32], ref[:1024]
    bb = raw.shape[1]
    got = _deq32(fmt, raw.reshape(1, -1), 1, ref.size).reshape(-1)              # one row of all 8 blocks
    np.testing.assert_array_equal(_bits(got), _bits(ref))
    got2 = _deq32(fmt, raw.reshape(-1, raw.shape[0] * bb // 4), 4, ref.size // 4).reshape(-1)                # four rows
    np.testing.assert_array_equal(_bits(got2), _bits(ref))


@pytest.mark.parametrize("fmt", L.FORMATS)
def test_dequant_reference_fixture(ref_golden, fmt):
    t = T[fmt]
    k = int(ref_golden[t + "_k"])
    raw = ref_golden[t + "_raw"]
    got = _deq32(fmt, raw, raw.shape[0], k)
    if fmt == "nvfp4":                                                             # device semantics = the pack form (sign of scale ignored, -0 kept)
        np.testing.assert_array_equal(_bits(got), _bits(ref_golden["NVFP4_pack_f32_nog"]))
        g = float(ref_golden["NVFP4_pack_gscale"])
        np.testing.assert_array_equal(_bits(_deq32(fmt, raw, raw.shape[0], k, gscale=g)), _bits(ref_golden["NVFP4_pack_f32"]))
    else:
        np.testing.assert_array_equal(_bits(got), _bits(ref_golden[t + "_f32"]))
        got = _deq32(fmt, ref_golden[t + "_raw_small"], raw.shape[0], k)
        want = ref_golden[t + "_f32_small"]
        nan = np.isnan(want)                                                       # random fp16 scale fields may be NaN (Q8_0 blocks of the fixture): NaN wherever the reference has one
        np.testing.assert_array_equal(np.isnan(got), nan)
        np.testing.assert_array_equal(_bits(got)[~nan], _bits(want)[~nan])


@pytest.mark.parametrize("fmt", L.FORMATS)
@pytest.mark.parametrize("n,k", [(40, 1024), (256, 4096)])
def test_dequant_random_vs_oracle(fmt, n, k):
    rng = np.random.default_rng(7)
    raw = synth.raw_blocks(fmt, n, k, rng)
    want = O.dequant(T[fmt], raw, k)
    t16 = ops.to_device_t16(fmt, raw, n, k)
    got = ops.dequant(fmt, t16, n, k, torch.float32).cpu().numpy()
    if fmt == "nvfp4":
        np.testing.assert_array_equal(got, want)                                   # +-0 aside
    else:
        np.testing.assert_array_equal(_bits(got), _bits(want))
    got16 = ops.dequant(fmt, t16, n, k, torch.float16).cpu().numpy()
    np.testing.assert_array_equal(got16, O.sat_f16(want))
    # a row range: rows [16, 16 + 20)
    part = ops.dequant(fmt, t16, n, k, torch.float32, row0=16, nrows=20).cpu().numpy()
    np.testing.assert_array_equal(part, got[16:36])


def test_dequant_rejects_bad_arguments():
    t = torch.zeros(2304, dtype=torch.uint8, device="cuda")
    with pytest.raises(Exception):
        ops.dequant("q4_k", t, 16, 256, torch.float32, row0=8)
    with pytest.raises(ValueError):
        ops.dequant("q4_k", t, 16, 256, torch.bfloat16)
    with pytest.raises(ValueError):
        ops.dequant("q4_k", t.cpu(), 16, 256)
