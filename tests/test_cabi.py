"""The C-ABI library builds, loads and exports every symbol include/kyb.h declares (no compute calls: no GPU needed)."""
import ctypes
import os
import re

import pytest

from kyojin_mac_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "kyb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kyb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 10
    raw = ctypes.CDLL(_lib.SO_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/kyb.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_size_helpers(lib):
    assert lib.kyb_version() >= 100
    assert lib.kyb_t16_nbytes(0, 4096, 4096) == 4096 * 4096 // 256 * 144
    assert lib.kyb_t16_nbytes(1, 5120, 27648) == 5120 * 27648 // 256 * 210
    assert lib.kyb_t16_nbytes(2, 12288, 3072) == 12288 * 3072 // 256 * 110
    assert lib.kyb_t16_nbytes(0, 5, 256) == 2304                      # padded to one 16-row tile
    assert lib.kyb_t16_nbytes(0, 16, 100) == 0 and lib.kyb_t16_nbytes(9, 16, 256) == 0
    assert lib.kyb_raw_row_bytes(3, 128) == 72 and lib.kyb_raw_row_bytes(0, 100) == 0
    assert lib.kyb_status_string(-3).decode().startswith("a bounded")


def test_argument_errors_are_reported_without_a_device(lib):
    # shape errors are detected before any CUDA call
    assert lib.kyb_gemv_t16(0, None, 16, 100, None, 1, 100, 1.0, None, 16, None, 0, 0, None) == _lib.EINVAL
    assert b"multiple of 256" in lib.kyb_last_error()
    assert lib.kyb_gemv_t16(7, None, 16, 256, None, 1, 256, 1.0, None, 16, None, 0, 0, None) == _lib.EINVAL
    assert lib.kyb_gemv_t16(0, None, 16, 256, None, 40, 256, 1.0, None, 16, None, 0, 0, None) == _lib.EINVAL
    assert lib.kyb_dequant_t16(0, None, 16, 256, 0, 16, 1.0, 0, None, 256, None) == _lib.EINVAL
    with pytest.raises(_lib.KybError):
        _lib.check(lib.kyb_repack_raw_to_t16(0, None, 16, 256, None, None))
