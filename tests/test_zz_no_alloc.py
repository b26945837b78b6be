"""kyb_gemv_t16_static: the GEMV for callers that must not allocate device memory (a server whose HBM is fully handed to its KV-cache pool, a decode
loop that cannot take cudaMalloc's device-wide synchronisation, a plug-in host that forbids callee allocation). It keeps its split-k scratch in a fixed
array inside the library, so this test drives it through the C ABI with plain pointers and checks, on two calls in a row, that it returns exactly what
kyb_gemv_t16 returns with a caller workspace; it also checks that an oversized shape is refused instead of overrunning the array.
Collected last on purpose: a run that stops at the first failure has already run every other test."""
import pytest
import torch

from kyojin_mac_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def _static(fmt, t16, n, k, x, check=1):
    y = torch.full((x.shape[0], n), float("nan"), dtype=torch.float16, device=x.device)
    rc = _lib.lib().kyb_gemv_t16_static(ops._fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), x.shape[0], x.stride(0), 1.0, y.data_ptr(), y.stride(0), check,
                                        torch.cuda.current_stream().cuda_stream)
    return rc, y


@pytest.mark.parametrize("fmt,n,k,m", [("q4_k", 512, 5120, 8), ("q6_k", 1024, 8192, 3), ("q4_k", 4096, 1024, 1)])
def test_static_scratch_matches_workspace_variant(fmt, n, k, m):
    t16 = synth.t16_random_device(fmt, n, k, seed=5)
    g = torch.Generator(device="cuda").manual_seed(6)
    for call in range(2):                                              # the shared array keeps the previous call's partial sums: results must not depend on them
        x = torch.randn((m, k), device="cuda", generator=g).to(torch.float16)
        want = ops.gemv(fmt, t16, n, k, x)
        rc, got = _static(fmt, t16, n, k, x)
        assert rc == 0, _lib.lib().kyb_last_error()
        assert torch.equal(got, want), f"call {call}"
    if (fmt, n) == ("q4_k", 512):
        assert _lib.lib().kyb_gemv_workspace_bytes(ops._fmt(fmt), n, k, m) > 0     # this case really goes through the scratch array


def test_static_scratch_refuses_oversized_shape():
    fmt, n, k, m = "q4_k", 8192, 65536, 32                              # 32 chunks of 8 k-blocks x 32 rows x 8192 outputs of chunk sums: 33.5 MB > 16 MiB
    assert _lib.lib().kyb_gemv_workspace_bytes(ops._fmt(fmt), n, k, m) > (16 << 20)
    t16 = synth.t16_random_device(fmt, n, k, seed=1)
    x = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    rc, _ = _static(fmt, t16, n, k, x)
    assert rc == _lib.EWORKSPACE and b"16" in _lib.lib().kyb_last_error()
    assert ops.gemv(fmt, t16, n, k, x).abs().max().item() == 0        # the workspace variant serves it


def test_static_call_allocates_nothing_and_serves_another_stream():
    """After one warm-up call (which looks up the array's address), a call with preallocated x and y leaves the device's free memory and the caching allocator's
    books unchanged, in the asynchronous form (check = 0) and in the checked form; the same product issued on a second stream, after the first has been waited
    for (calls that overlap would race on the shared array), returns the same bits."""
    fmt, n, k, m = "q4_k", 1024, 5120, 4
    t16 = synth.t16_random_device(fmt, n, k, seed=9)
    x = torch.randn((m, k), device="cuda").to(torch.float16)
    want = ops.gemv(fmt, t16, n, k, x)
    L = _lib.lib()
    y = torch.empty((m, n), dtype=torch.float16, device="cuda")
    call = lambda check, st: L.kyb_gemv_t16_static(ops._fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), m, x.stride(0), 1.0, y.data_ptr(), y.stride(0), check, st)
    cur = torch.cuda.current_stream()
    assert call(1, cur.cuda_stream) == 0                                # warm-up: first call on this device
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    y.zero_()
    assert call(0, cur.cuda_stream) == 0                                # asynchronous form
    assert call(1, cur.cuda_stream) == 0                                # checked form right behind it (same stream: ordered, no race)
    assert (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (free0, alloc0, reserved0)
    assert torch.equal(y, want)
    side = torch.cuda.Stream()
    side.wait_stream(cur)
    y.zero_()
    cur.synchronize()
    assert call(1, side.cuda_stream) == 0
    assert torch.equal(y, want)
