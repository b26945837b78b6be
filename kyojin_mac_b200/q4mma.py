"""Few-row product on affine 4-bit weights: torch mirror of kyojin_mlx/q4mma.py (`prep_x` :86-94, `q4mma` :97-106, `q4mma3` / `q4mma4` :451-474,
`Q4Linear` :727-754, `install` :781-794). Operands are MLX's affine layout: w uint32 [n, k/8], scales / biases [n, k/group], group 32 or 64.
`q4k_affine` gives the affine view of a Q4_K pack (kyojin_mlx/foreign_pack.py:136-176 `mq_arrays`: group 32, scale = fp16(d sc), bias = fp16(-dmin mn))."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib, ops


def prep_x(x: torch.Tensor) -> torch.Tensor:
    """The reference transposes and zero-pads x to [k, 8 | 16] for its simdgroup fragments; the CUDA kernel reads x [rows, k] as it is, so this only makes it
    contiguous fp16."""
    return x.to(torch.float16).contiguous()


def q4mma(xt: torch.Tensor, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, rows: int, nt: int = 1, ws: int = 4) -> torch.Tensor:
    """y [rows, n] (dtype of scales) = x[:rows] @ (scales * q + biases)^T; rows <= 32; the result of a row does not depend on `rows`. nt / ws are accepted for
    call compatibility."""
    n, k = w.shape[0], w.shape[1] * 8
    group = k // scales.shape[1]
    x = prep_x(xt)[:rows]
    s16, b16 = scales.to(torch.float16).contiguous(), biases.to(torch.float16).contiguous()
    y = torch.empty((rows, n), dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().kyb_q4mma(w.contiguous().data_ptr(), s16.data_ptr(), b16.data_ptr(), group, x.data_ptr(), x.stride(0), rows, n, k, y.data_ptr(), y.stride(0), ops._stream()))
    return y.to(scales.dtype)


q4mma3 = q4mma          # the reference's v3 / v4 differ in tiling only; one CUDA kernel serves all row counts up to 32
q4mma4 = q4mma


def q4k_affine(raw: np.ndarray, k: int):
    """Stored Q4_K rows -> (w uint32 [n, k/8], scales fp16 [n, k/32], biases fp16 [n, k/32]): the affine group-32 view of the same codes."""
    raw = np.asarray(raw, np.uint8)
    n = raw.shape[0]
    B = raw.reshape(n, k // 256, 144)
    d = np.ascontiguousarray(B[..., 0:2]).view("<f2")[..., 0].astype(np.float32)
    dmin = np.ascontiguousarray(B[..., 2:4]).view("<f2")[..., 0].astype(np.float32)
    s12 = B[..., 4:16]
    sc = np.empty(s12.shape[:-1] + (8,), np.float32)
    mn = np.empty_like(sc)
    for j in range(4):
        sc[..., j], mn[..., j] = s12[..., j] & 63, s12[..., j + 4] & 63
        sc[..., j + 4] = (s12[..., j + 8] & 15) | ((s12[..., j] >> 6) << 4)
        mn[..., j + 4] = (s12[..., j + 8] >> 4) | ((s12[..., j + 4] >> 6) << 4)
    sat = lambda a: np.clip(a, -65504.0, 65504.0).astype(np.float16)
    scales = sat(d[..., None] * sc).reshape(n, k // 32)
    biases = sat(-dmin[..., None] * mn).reshape(n, k // 32)
    q = B[..., 16:144].reshape(n, k // 256, 4, 32)
    codes = np.stack([q & 15, q >> 4], 3).reshape(n, k // 8, 8).astype(np.uint32)      # natural element order, 8 per word
    w = (codes << (4 * np.arange(8, dtype=np.uint32))).sum(-1, dtype=np.uint32)
    return w, scales, biases


class Q4Linear(torch.nn.Module):
    """Affine 4-bit linear served by q4mma for rows <= 32 (kyojin_mlx/q4mma.py:727-754). More rows are sliced in 32-row calls."""

    def __init__(self, w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bias: torch.Tensor | None = None):
        super().__init__()
        self.w, self.scales, self.biases, self.bias = w, scales, biases, bias

    def forward(self, x):
        shape = x.shape
        x2 = prep_x(x.reshape(-1, shape[-1]))
        ys = [q4mma(x2[i:i + 32], self.w, self.scales, self.biases, min(32, x2.shape[0] - i)) for i in range(0, x2.shape[0], 32)]
        y = torch.cat(ys, 0)
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*shape[:-1], self.w.shape[0])


def install(model: torch.nn.Module) -> int:
    """Swaps every submodule that carries affine 4-bit operands (attributes weight uint32, scales, biases) for a Q4Linear; returns the count
    (kyojin_mlx/q4mma.py:781-794)."""
    n = 0
    for name, child in list(model.named_children()):
        w, s, b = getattr(child, "weight", None), getattr(child, "scales", None), getattr(child, "biases", None)
        if isinstance(w, torch.Tensor) and w.dtype in (torch.int32, torch.uint32) and s is not None and b is not None:
            setattr(model, name, Q4Linear(w, s, b, getattr(child, "bias", None)))
            n += 1
        else:
            n += install(child)
    return n
