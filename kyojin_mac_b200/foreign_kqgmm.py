"""Expert-grouped GEMM on routed slots (prefill), torch mirror of kyojin_mlx/foreign_kqgmm.py: `csort` :191-196, `plan` :210-216, `gmm` :225-239,
`gather_perm` :264-268, `silu_perm` :283-290, `mlp` :293-314, `dense` :343-354. Slots are sorted by expert on the device (no host readback), tiles of MT
rows of ONE expert run on tcgen05 (kyb_gemm_f16_grouped), the down projection scatters its rows back to slot order.
The weights are decoded from their T16 tiles inside the grouped GEMM (kyb_gemm_kq_grouped; no fp16 copy of the stack in HBM), as the reference decodes
inside its own grouped kernel; formats without a fused decoder and stacks with n % 256 != 0 take the staged form (fp16 copy of the stack, kyb_gemm_f16_grouped)."""
from __future__ import annotations

import torch

from . import flags as F
from . import ops

MT = 128                     # rows of one expert per tile of the staged fp16 grouped GEMM = UMMA M
MT_FUSED = 256               # rows of one expert per work item when the weights are decoded inside the GEMM: one decode serves two 128-row blocks


def fused_ok(dev) -> bool:
    """The expert stack can go through the grouped GEMM that decodes its T16 tiles in the kernel."""
    from .layout import PREFILL_FUSED
    return dev.n % 256 == 0 and not F.PREFILL_TWO_STEP and dev.fmt in PREFILL_FUSED


def glu_fused_ok(glu) -> bool:
    """gate and up can run as one grouped product: both decoded inside the GEMM, one format and shape, 128 output columns per work item."""
    g, u = glu.g, glu.u
    return fused_ok(g) and fused_ok(u) and (g.fmt, g.n, g.k, g.E) == (u.fmt, u.n, u.k, u.E) and g.n % 128 == 0


def csort(e32: torch.Tensor, E: int, mt: int = MT):
    """Slots -> (order [S] sorted position -> slot, tb [E+1] first tile of each expert, off [E+1] first row of each expert)."""
    pl = ops.moe_plan(e32, E, 1, mt)
    return pl["order"], pl["tb"], pl["off"]


def plan(e32: torch.Tensor, E: int, mt: int = MT):
    """(order, tb, off, max_tiles): max_tiles bounds the grid without reading the device (S / mt + E)."""
    order, tb, off = csort(e32, E, mt)
    return order, tb, off, (e32.numel() + mt - 1) // mt + E


def gather_perm(x2: torch.Tensor, order: torch.Tensor, K: int, xperm=None) -> torch.Tensor:
    """Rows of x2 [T, k] gathered into sorted slot order (slot s reads token s // K), optional column permutation."""
    return ops.gather_rows(x2, order, K, xperm)


def silu_perm(a: torch.Tensor, b: torch.Tensor, xperm=None, limit=None) -> torch.Tensor:
    return ops.silu_mul(a, b, limit, xperm)


def gmm(dev, xg: torch.Tensor, tb: torch.Tensor, off: torch.Tensor, S: int, mt: int = MT, orow=None, out_rows=None, w16=None) -> torch.Tensor:
    """Sorted grouped product: row r of xg (expert segment e) times expert e of `dev` -> [S, n] (or scattered to rows orow[r])."""
    gs = dev.gs if dev.fmt == "nvfp4" else None
    if w16 is None and fused_ok(dev):                                                # weights decoded inside the grouped GEMM; tb counts mt-row tiles
        if mt not in (128, 256):
            raise ValueError("work items are 128 or 256 rows of one expert")
        return ops.gemm_kq_grouped(dev.fmt, dev.t16, dev.n, dev.k, dev.E, xg, tb, off, orow, gs, out_rows=out_rows or S, mt=mt)
    if mt != MT:
        raise ValueError(f"tiles of the staged form are {MT} rows (UMMA M)")
    if w16 is None:
        w16 = ops.dequant(dev.fmt, dev.t16, dev.nrows, dev.k, torch.float16, 1.0)
    return ops.gemm_f16_grouped(xg, w16, dev.n, dev.E, tb, off, orow, gs, out_rows=out_rows or S)


def mlp(glu, x2: torch.Tensor, e32: torch.Tensor, K: int, mt: int | None = None) -> torch.Tensor:
    """Routed SwiGLU MLP on sorted slots -> unweighted per-slot outputs [S, H] in slot order (foreign_kqgmm.py:293-314)."""
    S = e32.numel()
    if mt is None:
        mt = MT_FUSED if all(fused_ok(d) for d in (glu.g, glu.u, glu.d)) else MT
    order, tb, off = csort(e32, glu.g.E, mt)
    xg = gather_perm(x2, order, K)
    if glu_fused_ok(glu):                                                            # gate | up as one grouped product, silu(a) * b in its epilogue
        gsg, gsu = (glu.g.gs, glu.u.gs) if glu.g.fmt == "nvfp4" else (None, None)
        h = ops.gemm_kq_grouped_glu(glu.g.fmt, glu.g.t16, glu.u.t16, glu.g.n, glu.g.k, glu.g.E, xg, tb, off, gsg, gsu, glu.limit, mt)
    else:
        a = gmm(glu.g, xg, tb, off, S, mt)
        b = gmm(glu.u, xg, tb, off, S, mt)
        h = silu_perm(a, b, None, glu.limit)
    return gmm(glu.d, h, tb, off, S, mt, orow=order)


def dense_ok(dev, R: int) -> bool:
    return not dev.E and dev.n % 128 == 0 and R > 32


def dense(dev, x2: torch.Tensor) -> torch.Tensor:
    """A dense linear as ONE group of the grouped kernel (foreign_kqgmm.py:343-354): same result as DevPack.apply's prefill path."""
    return dev._prefill(x2)
