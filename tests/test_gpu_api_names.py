"""Call-surface bindings kept from the reference (GPU): mma_gemv partial / finalize, q4mma on affine 4-bit operands (row-count invariance as
tests/test_q4mma.py:24-45), fp4tile layout round trip and gathered GEMV vs the fp64 tile_ref (tests/test_fp4tile.py:29-60)."""
import numpy as np
import pytest
import torch

from kyojin_mac_b200 import foreign_pack as FP, fp4tile, mma_gemv, ops, q4mma, synth
from kyojin_mac_b200.foreign_linear import DevPack
from oracle import kq_numpy as O

pytestmark = pytest.mark.gpu


def test_mma_gemv_two_steps_equal_one_call():
    rng = np.random.default_rng(0)
    n, k, rows = 256, 5120, 6
    raw = synth.raw_blocks("q4_k", n, k, rng)
    g = DevPack(FP.to_pack("Q4_K", raw, k))
    x = torch.from_numpy(synth.activations(rows, k, rng)).cuda()
    part = mma_gemv.partial_mma(g, x, rows)
    assert part.dtype == torch.float32 and part.shape[1] == rows
    y = mma_gemv.finalize_rows(g, part, rows)
    assert torch.equal(y, g.apply(x))


@pytest.mark.parametrize("group", [32, 64])
def test_q4mma_rows_invariant_and_accurate(group):
    rng = np.random.default_rng(group)
    n, k = 96, 1024
    if group == 32:
        raw = synth.raw_blocks("q4_k", n, k, rng, d_sigma=0.02)
        w, s, b = q4mma.q4k_affine(raw, k)
        ref = O.dequant("Q4_K", raw, k)                                     # the affine view rounds d sc and dmin mn to fp16: tolerance class
    else:
        w = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
        s = (rng.random((n, k // 64)) * 0.02).astype(np.float16)
        b = (rng.standard_normal((n, k // 64)) * 0.05).astype(np.float16)
        q = ((w[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).reshape(n, k).astype(np.float32)
        ref = q * np.repeat(s.astype(np.float32), 64, 1) + np.repeat(b.astype(np.float32), 64, 1)
    x = synth.activations(16, k, rng)
    wd, sd, bd = (torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).cuda() for a in (w, s, b))
    xd = torch.from_numpy(x).cuda()
    y16 = q4mma.q4mma(q4mma.prep_x(xd), wd, sd, bd, 16)
    want = O.matmul_f64(x, ref)
    assert O.rel_fro(y16.cpu().numpy(), want) < 2e-3
    for r in (1, 5, 8):
        yr = q4mma.q4mma3(q4mma.prep_x(xd), wd, sd, bd, r)
        assert torch.equal(yr, y16[:r])                                      # bits do not depend on the row count


def test_q4mma_ragged_shapes_and_all_row_counts():
    """Weight rows not a multiple of the warp's 16, k a multiple of 64 only (a partial last 256-input chunk), 17 to 32 activation rows (four column tiles)."""
    rng = np.random.default_rng(9)
    n, k = 100, 1088
    w = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    s = (rng.random((n, k // 32)) * 0.02).astype(np.float16)
    b = (rng.standard_normal((n, k // 32)) * 0.05).astype(np.float16)
    q = ((w[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).reshape(n, k).astype(np.float32)
    ref = q * np.repeat(s.astype(np.float32), 32, 1) + np.repeat(b.astype(np.float32), 32, 1)
    x = synth.activations(32, k, rng)
    wd, sd, bd = (torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).cuda() for a in (w, s, b))
    xd = q4mma.prep_x(torch.from_numpy(x).cuda())
    y32 = q4mma.q4mma4(xd, wd, sd, bd, 32)
    assert O.rel_fro(y32.cpu().numpy(), O.matmul_f64(x, ref)) < 1e-3
    for r in (1, 9, 16, 17, 24):
        assert torch.equal(q4mma.q4mma(xd, wd, sd, bd, r), y32[:r]), r


def test_fp4tile_round_trip_and_gather():
    rng = np.random.default_rng(3)
    E, n, k, S = 3, 64, 512, 20
    qs = rng.integers(0, 2 ** 32, (E, n, k // 8), dtype=np.uint64).astype(np.uint32)
    meta = rng.integers(0x28, 0x46, (E, n, k // 16), dtype=np.uint8).view("<u2").reshape(E, n, k // 32)
    gs = np.array([1.0, 0.5, 0.25], np.float32)
    tl = fp4tile.to_tile(qs, meta)
    q2, m2 = fp4tile.from_tile(tl, n, k)
    np.testing.assert_array_equal(q2, qs)
    np.testing.assert_array_equal(m2, meta)
    ref = fp4tile.tile_ref(qs, meta, gs)
    w16 = fp4tile.dequant(tl, torch.from_numpy(gs).cuda(), E, n, k)
    np.testing.assert_allclose(w16.float().cpu().numpy(), ref, rtol=1e-3, atol=0)
    x = synth.activations(4, k, rng)
    eids = rng.integers(0, E, S).astype(np.int32)
    xrows = rng.integers(0, 4, S).astype(np.int32)
    y = fp4tile.gather(torch.from_numpy(x).cuda(), torch.from_numpy(xrows).cuda(), torch.from_numpy(eids).cuda(), tl, torch.from_numpy(gs).cuda(), n, k)
    want = np.stack([x[xrows[s]].astype(np.float64) @ ref[eids[s]].T for s in range(S)])
    assert np.abs(y.cpu().numpy() - want).max() < 1e-3 * np.abs(want).max()
