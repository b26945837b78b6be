"""The bounded-wait report path end to end: a kernel whose wait can never complete gives up by itself, the host reads KYB_ETIMEOUT once, and the device stays
usable. The failure is made of a barrier that nothing arrives at and a small poll limit; no fault, trap or endless loop is involved."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_once_and_the_device_stays_usable():
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    ops.check_device_status()                                               # clean before
    _lib.check(L.kyb_selftest_wait_timeout(200, st))
    with pytest.raises(_lib.KybError) as ei:
        ops.check_device_status()
    assert ei.value.status == _lib.ETIMEOUT and "bounded wait" in str(ei.value)
    ops.check_device_status()                                               # the word was cleared by the failing check
    # a product right after: same context, correct result
    n, k = 64, 512
    t16 = synth.t16_random_device("q4_k", n, k, seed=3)
    x = torch.randn((2, k), device="cuda").to(torch.float16)
    y = ops.gemv("q4_k", t16, n, k, x)
    w = ops.dequant("q4_k", t16, n, k, torch.float32)
    want = x.double() @ w.double().T                                        # the device decoder is pinned bit-exactly on the golden vectors elsewhere
    err = float((y.double() - want).norm() / want.norm())
    assert err < 1e-3
    ops.check_device_status()


def test_poll_limit_is_validated():
    L = _lib.lib()
    assert L.kyb_selftest_wait_timeout(0, None) == _lib.EINVAL and L.kyb_selftest_wait_timeout(100000, None) == _lib.EINVAL
