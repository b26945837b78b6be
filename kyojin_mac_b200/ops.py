"""Thin torch-tensor front end of the C ABI: pointers, sizes and the current CUDA stream go straight to libkyb.so."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .layout import FMT_ID, padded_rows


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _fmt(fmt) -> int:
    if isinstance(fmt, str):
        if fmt not in FMT_ID:
            raise ValueError(f"unknown format {fmt!r}")
        return FMT_ID[fmt]
    return int(fmt)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and (not isinstance(t, torch.Tensor) or not t.is_cuda):
            raise ValueError("kyojin_mac_b200 operators take CUDA tensors (there is no CPU path)")


def t16_nbytes(fmt, n: int, k: int) -> int:
    v = _lib.lib().kyb_t16_nbytes(_fmt(fmt), n, k)
    if v == 0:
        raise ValueError(f"bad T16 shape fmt={fmt} n={n} k={k} (k must be a positive multiple of 256)")
    return v


def raw_to_t16(fmt, raw: torch.Tensor, n: int, k: int) -> torch.Tensor:
    """GGUF rows uint8 [n, row_bytes] on the device -> T16 bytes on the device."""
    _need_cuda(raw)
    raw = raw.contiguous()
    out = torch.empty(t16_nbytes(fmt, n, k), dtype=torch.uint8, device=raw.device)
    _lib.check(_lib.lib().kyb_repack_raw_to_t16(_fmt(fmt), raw.data_ptr(), n, k, out.data_ptr(), _stream()))
    return out


def t16_to_raw(fmt, t16: torch.Tensor, n: int, k: int) -> torch.Tensor:
    _need_cuda(t16)
    rb = _lib.lib().kyb_raw_row_bytes(_fmt(fmt), k)
    out = torch.empty((n, rb), dtype=torch.uint8, device=t16.device)
    _lib.check(_lib.lib().kyb_repack_t16_to_raw(_fmt(fmt), t16.data_ptr(), n, k, out.data_ptr(), _stream()))
    return out


def dequant(fmt, t16: torch.Tensor, n: int, k: int, dtype=torch.float16, gscale: float = 1.0, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    """T16 -> [nrows, k] float32 (bit-equal to the reference decoder) or float16 (that value rounded, saturated)."""
    _need_cuda(t16)
    nrows = n - row0 if nrows is None else nrows
    if dtype not in (torch.float32, torch.float16):
        raise ValueError("dequant output is float32 or float16")
    out = torch.empty((nrows, k), dtype=dtype, device=t16.device)
    _lib.check(_lib.lib().kyb_dequant_t16(_fmt(fmt), t16.data_ptr(), n, k, row0, nrows, float(gscale), 0 if dtype == torch.float32 else 1,
                                          out.data_ptr(), k, _stream()))
    return out


_ws: dict = {}


def workspace(device, nbytes: int) -> torch.Tensor:
    """Grow-only scratch buffer per (device, stream): split-k partial sums of the GEMV live here."""
    key = (device.index, _stream())
    buf = _ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _ws[key] = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    return buf


def gemv(fmt, t16: torch.Tensor, n: int, k: int, x: torch.Tensor, gscale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """y fp16 [m, n] = x fp16 [m, k] @ W^T for m <= 32, W in T16."""
    _need_cuda(t16, x)
    if x.dtype != torch.float16 or x.dim() != 2 or x.shape[1] != k:
        raise ValueError(f"x must be float16 [m, {k}], got {x.dtype} {tuple(x.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    m = x.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    L = _lib.lib()
    need = L.kyb_gemv_workspace_bytes(_fmt(fmt), n, k, m)
    ws = workspace(x.device, need) if need else None
    _lib.check(L.kyb_gemv_t16(_fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), m, x.stride(0), float(gscale), y.data_ptr(), y.stride(0),
                              ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream()))
    return y


def gemm_f16(a: torch.Tensor, b: torch.Tensor, gscale: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """d fp16 [m, n] = a fp16 [m, k] @ b fp16 [n, k]^T on tcgen05 (fp32 accumulation in tensor memory, saturated fp16 result)."""
    _need_cuda(a, b)
    if a.dtype != torch.float16 or b.dtype != torch.float16 or a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"gemm_f16 takes float16 [m, k] and [n, k], got {a.dtype} {tuple(a.shape)} and {b.dtype} {tuple(b.shape)}")
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    m, k = a.shape
    n = b.shape[0]
    d = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=a.device)
    _lib.check(_lib.lib().kyb_gemm_f16_tn(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), m, n, k, float(gscale), d.data_ptr(), d.stride(0), _stream()))
    return d


def gemv_plan(fmt, n: int, k: int, m: int) -> dict:
    import ctypes
    out = (ctypes.c_int * 8)()
    _lib.check(_lib.lib().kyb_gemv_plan(_fmt(fmt), n, k, m, out))
    return dict(zip(("nt", "mst", "warps", "stages", "kbp", "ksplit", "smem", "grid"), list(out)))


def check_device_status() -> None:
    _lib.check(_lib.lib().kyb_check_device_status(_stream()))


def to_device_t16(fmt: str, raw_np: np.ndarray, n: int, k: int, device="cuda") -> torch.Tensor:
    """Host GGUF rows (numpy uint8 [n, row_bytes]) -> device T16, repacked on the device."""
    raw = torch.from_numpy(np.ascontiguousarray(raw_np)).to(device)
    return raw_to_t16(fmt, raw, n, k)
