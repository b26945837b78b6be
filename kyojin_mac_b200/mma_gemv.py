"""Few-row GEMV in two steps (split-k partial sums, then finalize): torch mirror of kyojin_mlx/mma_gemv.py:129-149 (`partial_mma`, `finalize_rows`).
The reference's handle `g` is an EXL3 `Mul1Gemv`; here it is a DevPack of a K-quant / NVFP4 matrix (attributes n, k, out_dtype are read the same way).
There is no Hadamard / sign step (that belongs to the trellis format)."""
from __future__ import annotations

import torch

from . import _lib, ops


def partial_mma(g, xh: torch.Tensor, rows: int, ws: int = 4) -> torch.Tensor:
    """GEMV partials of `rows` (<= 32) rows: f32 [parts, rows, n padded to 16]; parts = canonical k-chunks of the matrix (ws is accepted for call
    compatibility; the launch shape is planned by the library)."""
    if xh.dtype != torch.float16 or xh.shape[0] < rows:
        raise ValueError("xh must be float16 with at least `rows` rows")
    L = _lib.lib()
    parts = L.kyb_gemv_chunks(g.n, g.k)
    npad = (g.n + 15) // 16 * 16
    part = torch.empty((parts, rows, npad), dtype=torch.float32, device=xh.device)
    x = xh[:rows].contiguous()
    _lib.check(L.kyb_gemv_partial_t16(ops._fmt(g.fmt), g.t16.data_ptr(), g.n, g.k, x.data_ptr(), rows, x.stride(0), part.data_ptr(), ops._stream()))
    return part


def finalize_rows(g, part: torch.Tensor, rows: int) -> torch.Tensor:
    """Sum over the parts (k order), apply the matrix's output scale, saturate, cast -> [rows, n]."""
    y = torch.empty((rows, g.n), dtype=torch.float16, device=part.device)
    _lib.check(_lib.lib().kyb_gemv_finalize(part.data_ptr(), part.shape[0], rows, g.n, float(getattr(g, "gscale", 1.0)), y.data_ptr(), y.stride(0), ops._stream()))
    od = getattr(g, "out_dtype", torch.float16)
    return y if od == torch.float16 else y.to(od)
