"""Thin torch-tensor front end of the C ABI: pointers, sizes and the current CUDA stream go straight to libkyb.so."""
from __future__ import annotations

import numpy as np
import torch

from . import _lib, flags as F
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
    """Grow-only scratch buffer per (device, stream): the chunk sums of the GEMV's two-launch form live here."""
    key = (device.index, _stream())
    buf = _ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _ws[key] = torch.empty(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
    return buf


def release_workspaces(stream_id: int | None = None) -> None:
    """Drops the cached workspaces (of one stream id, or all): for callers that create and retire many streams."""
    for key in [k for k in _ws if stream_id is None or k[1] == stream_id]:
        del _ws[key]


def gemv(fmt, t16: torch.Tensor, n: int, k: int, x: torch.Tensor, gscale: float = 1.0, out: torch.Tensor | None = None, chained: bool = False,
         x2: torch.Tensor | None = None, limit: float | None = None) -> torch.Tensor:
    """y fp16 [m, n] = x fp16 [m, k] @ W^T for m <= 32, W in T16.
    chained: launch with programmatic stream serialization (the kernel sets up and prefetches weights while the preceding kernel of the stream drains, and waits
    for it before touching x or y): only when the weights were not written by the kernel directly before this call on the stream. Same bits either way.
    x2: gated input, the row fed to the product is fp16(silu(x row) * x2 row), formed while the rows are staged (optional clamp `limit`)."""
    _need_cuda(t16, x, x2)
    if x.dtype != torch.float16 or x.dim() != 2 or x.shape[1] != k:
        raise ValueError(f"x must be float16 [m, {k}], got {x.dtype} {tuple(x.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    if x2 is not None:
        if x2.dtype != torch.float16 or x2.shape != x.shape:
            raise ValueError("the gated form takes two float16 tensors of one shape")
        if x2.stride() != x.stride():
            x, x2 = x.contiguous(), x2.contiguous()
    m = x.shape[0]
    y = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    L = _lib.lib()
    need = L.kyb_gemv_workspace_bytes(_fmt(fmt), n, k, m)
    ws = workspace(x.device, need) if need else None
    wp, wn = (ws.data_ptr(), ws.numel()) if ws is not None else (None, 0)
    if x2 is not None:
        _lib.check(L.kyb_gemv_glu_t16(_fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), x2.data_ptr(), float(limit or 0.0), m, x.stride(0), float(gscale), y.data_ptr(), y.stride(0),
                                      wp, wn, 1 if chained else 0, _stream()))
        return y
    _lib.check(L.kyb_gemv_t16(_fmt(fmt), t16.data_ptr(), n, k, x.data_ptr(), m, x.stride(0), float(gscale), y.data_ptr(), y.stride(0), wp, wn, 1 if chained else 0, _stream()))
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
    return dict(zip(("nt", "aligned", "warps", "kc", "kbp", "ksplit", "smem", "grid"), list(out)))


def gemv_workspace_bytes(fmt, n: int, k: int, m: int) -> int:
    """Bytes of scratch the product needs (0: one launch; else chunk sums through the workspace and a finalize launch)."""
    return int(_lib.lib().kyb_gemv_workspace_bytes(_fmt(fmt), n, k, m))


def check_device_status() -> None:
    _lib.check(_lib.lib().kyb_check_device_status(_stream()))


def to_device_t16(fmt: str, raw_np: np.ndarray, n: int, k: int, device="cuda") -> torch.Tensor:
    """Host GGUF rows (numpy uint8 [n, row_bytes]) -> device T16, repacked on the device."""
    raw = torch.from_numpy(np.ascontiguousarray(raw_np)).to(device)
    return raw_to_t16(fmt, raw, n, k)


# ------------------------------------------------------------------------------------------------ routed experts
def _p(t):
    return None if t is None else t.data_ptr()


def moe_select(logits: torch.Tensor, E: int, K: int, norm: bool = True, has_shared: bool = False):
    """logits fp32 [T, >= E (+1)] -> (inds uint32-as-int32 [T*K], scs f32 [T*K], sgs f32 [T] or None)."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("router logits must be contiguous float32 [T, E(+1)]")
    T = logits.shape[0]
    inds = torch.empty(T * K, dtype=torch.int32, device=logits.device)
    scs = torch.empty(T * K, dtype=torch.float32, device=logits.device)
    sgs = torch.empty(T, dtype=torch.float32, device=logits.device) if has_shared else None
    _lib.check(_lib.lib().kyb_moe_select(logits.data_ptr(), logits.stride(0), T, E, K, int(norm), int(has_shared), inds.data_ptr(), scs.data_ptr(), _p(sgs), _stream()))
    return inds, scs, sgs


_ROUTER_PIECES: dict = {}


def _router_pieces(gw: torch.Tensor, sg: torch.Tensor | None):
    """The gate cut into three fp16 pieces per row for the tensor-core router, made once per (gate tensor, version) and kept (a few MB per gate)."""
    key = (gw.data_ptr(), gw._version, tuple(gw.shape), None if sg is None else (sg.data_ptr(), sg._version))
    hit = _ROUTER_PIECES.get(key)
    if hit is None:
        E, H = gw.shape
        rpad = int(_lib.lib().kyb_router_rpad(E, 0 if sg is None else 1))
        pieces = torch.empty((3 * rpad, H), dtype=torch.float16, device=gw.device)
        inv = torch.empty((rpad,), dtype=torch.float32, device=gw.device)
        _lib.check(_lib.lib().kyb_router_split(gw.data_ptr(), _p(sg), E, H, pieces.data_ptr(), inv.data_ptr(), _stream()))
        if len(_ROUTER_PIECES) >= 64:
            _ROUTER_PIECES.clear()
        hit = _ROUTER_PIECES[key] = (pieces, inv, rpad, gw, sg)              # the gate tensors are kept alive so that their addresses stay theirs
    return hit[0], hit[1], hit[2]


def router_logits(x: torch.Tensor, gw: torch.Tensor, sgw: torch.Tensor | None = None, tensor_cores: bool | None = None) -> torch.Tensor:
    """fp32 [T, E + 1] router logits of x [T, H] (fp32 / fp16 / bf16) on the fp32 gate gw [E, H]; column E = shared-expert gate logit (sgw [H]) or unwritten.
    tensor_cores: None = by size (fp16 activations, at least flags.ROUTER_TC_MIN_ROWS tokens: one tcgen05 GEMM on the gate cut into three fp16 pieces + a
    recombining launch; below that the fp32 kernels, whose two forms agree bit for bit); True / False force one path."""
    _need_cuda(x, gw)
    if gw.dtype != torch.float32 or x.dtype not in _DT or x.dim() != 2 or x.shape[1] != gw.shape[1]:
        raise ValueError("router_logits takes x [T, H] (fp32 / fp16 / bf16) and an fp32 gate [E, H]")
    x, gw = (x if x.stride(1) == 1 else x.contiguous()), gw.contiguous()
    sg = None if sgw is None else sgw.reshape(-1).to(torch.float32).contiguous()
    T, (E, H) = x.shape[0], gw.shape
    lg = torch.empty((T, E + 1), dtype=torch.float32, device=x.device)
    if sg is None:
        lg[:, E].zero_()                                                    # no shared expert: the column exists (fixed row pitch) and reads as 0
    if tensor_cores is None:
        tensor_cores = x.dtype == torch.float16 and T >= F.ROUTER_TC_MIN_ROWS and H % 64 == 0
    if tensor_cores:
        if x.dtype != torch.float16 or H % 64:
            raise ValueError("the tensor-core router takes float16 activations with H a multiple of 64")
        pieces, inv, rpad = _router_pieces(gw, sg)
        work = workspace(x.device, T * 3 * rpad * 4)
        _lib.check(_lib.lib().kyb_router_logits_tc(x.data_ptr(), x.stride(0), pieces.data_ptr(), inv.data_ptr(), T, E, 0 if sg is None else 1, H, work.data_ptr(), lg.data_ptr(),
                                                   lg.stride(0), _stream()))
        return lg
    _lib.check(_lib.lib().kyb_router_logits(x.data_ptr(), _DT[x.dtype], x.stride(0), gw.data_ptr(), _p(sg), T, E, H, lg.data_ptr(), lg.stride(0), _stream()))
    return lg


def dequant_rows(fmt, t16: torch.Tensor, n: int, k: int, rows: torch.Tensor, dtype=torch.float16, gscale: float = 1.0) -> torch.Tensor:
    """[len(rows), k] decoded rows of a T16 matrix, gathered by id (int tensor on the device, 0 <= id < n)."""
    _need_cuda(t16, rows)
    ids = rows.reshape(-1).to(torch.int32).contiguous()
    out = torch.empty((ids.numel(), k), dtype=dtype, device=t16.device)
    if ids.numel():
        _lib.check(_lib.lib().kyb_dequant_rows_t16(_fmt(fmt), t16.data_ptr(), n, k, ids.data_ptr(), ids.numel(), float(gscale), _DT[dtype], out.data_ptr(), k, _stream()))
    return out


def gather_flat(srcs, dsts, nbytes=None) -> None:
    """Copies srcs[i] into dsts[i] (equal byte counts, multiples of 16 bytes, 16-byte aligned) with one launch per 128 pairs. Entries are contiguous device tensors
    or raw device addresses (ints, e.g. peer-mapped pointers; then nbytes[i] gives the size)."""
    import ctypes as C
    n = len(srcs)
    if n == 0:
        return
    ptr = lambda t: t if isinstance(t, int) else t.data_ptr()
    sizes = []
    for i, (a, b) in enumerate(zip(srcs, dsts)):
        sz = None
        for t in (a, b):
            if isinstance(t, torch.Tensor):
                if not t.is_cuda or not t.is_contiguous():
                    raise ValueError("gather_flat copies contiguous CUDA tensors")
                tsz = t.numel() * t.element_size()
                if sz is not None and tsz != sz:
                    raise ValueError("gather_flat: source and destination differ in size")
                sz = tsz
        if sz is None:
            sz = int(nbytes[i])
        sizes.append(sz)
    for i in range(0, n, 128):
        m = min(128, n - i)
        S = (C.c_void_p * m)(*[ptr(t) for t in srcs[i:i + m]])
        D = (C.c_void_p * m)(*[ptr(t) for t in dsts[i:i + m]])
        B = (C.c_int64 * m)(*sizes[i:i + m])
        _lib.check(_lib.lib().kyb_gather_flat(S, D, B, m, _stream()))


def moe_plan(ids: torch.Tensor, E: int, topk: int, mt: int = 128, wts: torch.Tensor | None = None, rank: torch.Tensor | None = None):
    """Counting sort of the slots by expert. Returns dict(order, inv, tok, ids_s, wts_s, off, tb)."""
    _need_cuda(ids)
    ids = ids.reshape(-1).to(torch.int32).contiguous()
    P, dev = ids.numel(), ids.device
    mk = lambda n, dt: torch.empty(n, dtype=dt, device=dev)
    out = dict(order=mk(P, torch.int32), inv=mk(P, torch.int32), tok=mk(P, torch.int32), ids_s=mk(P, torch.int32),
               wts_s=mk(P, torch.float32) if wts is not None else None, off=mk(E + 1, torch.int32), tb=mk(E + 1, torch.int32))
    w = None if wts is None else wts.reshape(-1).to(torch.float32).contiguous()
    r = None if rank is None else rank.to(torch.int32).contiguous()
    _lib.check(_lib.lib().kyb_moe_plan(ids.data_ptr(), _p(w), _p(r), E, P, topk, mt, out["order"].data_ptr(), out["inv"].data_ptr(), out["tok"].data_ptr(),
                                       out["ids_s"].data_ptr(), _p(out["wts_s"]), out["off"].data_ptr(), out["tb"].data_ptr(), _stream()))
    return out


def gather_rows(x: torch.Tensor, src: torch.Tensor, div: int = 1, perm: torch.Tensor | None = None) -> torch.Tensor:
    """out[r] = x[src[r] // div] (fp16 rows), optional column permutation."""
    _need_cuda(x, src)
    if x.dtype != torch.float16 or x.stride(1) != 1:
        raise ValueError("gather_rows takes float16 rows")
    R, k = src.numel(), x.shape[1]
    out = torch.empty((R, k), dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().kyb_gather_rows(x.data_ptr(), x.stride(0), x.shape[0], src.data_ptr(), div, _p(perm), R, k, out.data_ptr(), k, _stream()))
    return out


def silu_mul(a: torch.Tensor, b: torch.Tensor, limit: float | None = None, perm: torch.Tensor | None = None) -> torch.Tensor:
    """fp16(silu(a) * b) computed in fp32 (optional clamp as the reference's swiglu_limit)."""
    _need_cuda(a, b)
    if a.shape != b.shape or a.dtype != torch.float16 or b.dtype != torch.float16 or a.stride() != b.stride() or a.stride(1) != 1:
        raise ValueError("silu_mul takes two float16 [rows, n] tensors of the same layout")
    rows, n = a.shape
    h = torch.empty((rows, n), dtype=torch.float16, device=a.device)
    _lib.check(_lib.lib().kyb_silu_mul(a.data_ptr(), b.data_ptr(), a.stride(0), rows, n, float(limit or 0.0), _p(perm), h.data_ptr(), n, _stream()))
    return h


def moe_combine(y: torch.Tensor, scs: torch.Tensor, K: int, sgs: torch.Tensor | None = None, shared: torch.Tensor | None = None, dtype=torch.float16) -> torch.Tensor:
    """y fp16 [T*K, H] (slot order), scs f32 [T*K] -> [T, H] weighted sum (+ gated shared expert)."""
    _need_cuda(y, scs)
    S, H = y.shape
    T = S // K
    o = torch.empty((T, H), dtype=dtype, device=y.device)
    _lib.check(_lib.lib().kyb_moe_combine(y.data_ptr(), y.stride(0), scs.data_ptr(), _p(sgs), _p(shared), 0 if shared is None else shared.stride(0), T, K, H,
                                          0 if dtype == torch.float32 else 1, o.data_ptr(), H, _stream()))
    return o


def moe_groups(eids: torch.Tensor, E: int):
    """Expert election for the gathered GEMV: slots of one expert are served 8 at a time. Returns the scratch triple (g_expert, g_slots, ngroups) that
    gemv_group takes as `groups`; one election serves every projection of a layer. Slots with an id outside [0, E) are in no group."""
    _need_cuda(eids)
    eids = eids.reshape(-1).to(torch.int32).contiguous()
    S = eids.numel()
    scratch = torch.empty(S * 9 + 1, dtype=torch.int32, device=eids.device)
    g_expert, g_slots, ngroups = scratch[:S], scratch[S:9 * S], scratch[9 * S:]
    _lib.check(_lib.lib().kyb_moe_groups(eids.data_ptr(), S, E, g_expert.data_ptr(), g_slots.data_ptr(), ngroups.data_ptr(), _stream()))
    return g_expert, g_slots, ngroups


def gemv_group(fmt, t16: torch.Tensor, n: int, k: int, E: int, x: torch.Tensor, eids: torch.Tensor, xrows: torch.Tensor | None = None, xdiv: int = 1,
               gs: torch.Tensor | None = None, out: torch.Tensor | None = None, groups=None, t16b: torch.Tensor | None = None, gsb: torch.Tensor | None = None,
               x2: torch.Tensor | None = None, limit: float | None = None) -> torch.Tensor:
    """y fp16 [S, n]: slot s = expert eids[s] applied to row xrows[s] (or s // xdiv) of x fp16 [*, k]; one weight read per expert and 8 slots.
    t16b (+ gsb): a second stack of the same shape in the same launch, y is [2 S, n] with its results in rows [S, 2 S). x2: gated input, the row fed to the
    product is fp16(silu(x row) * x2 row). groups: the election of moe_groups(eids, E) when the caller already has it."""
    _need_cuda(t16, x, eids, t16b, x2)
    if x.dtype != torch.float16 or x.stride(1) != 1 or x.shape[1] != k:
        raise ValueError(f"x must be float16 [rows, {k}]")
    if x2 is not None and (x2.dtype != torch.float16 or x2.shape != x.shape or x2.stride() != x.stride()):
        raise ValueError("the gated form takes two float16 tensors of one shape and layout")
    if t16b is not None and t16b.numel() != t16.numel():
        raise ValueError("the pair form takes two stacks of one shape and format")
    S = eids.numel()
    eids = eids.reshape(-1).to(torch.int32).contiguous()
    rows = S * (2 if t16b is not None else 1)
    y = out if out is not None else torch.empty((rows, n), dtype=torch.float16, device=x.device)
    if y.shape[0] != rows:
        raise ValueError(f"out must hold {rows} rows")
    g_expert, g_slots, ngroups = groups if groups is not None else moe_groups(eids, E)
    xr = None if xrows is None else xrows.reshape(-1).to(torch.int32).contiguous()
    _lib.check(_lib.lib().kyb_gemv_group_t16(_fmt(fmt), t16.data_ptr(), _p(t16b), n, k, E, x.data_ptr(), _p(x2), float(limit or 0.0), x.stride(0), eids.data_ptr(), _p(xr), xdiv, S,
                                             _p(gs), _p(gsb), y.data_ptr(), y.stride(0), g_expert.data_ptr(), g_slots.data_ptr(), ngroups.data_ptr(), _stream()))
    return y


def gemm_f16_grouped(a: torch.Tensor, b: torch.Tensor, n: int, E: int, tb: torch.Tensor, off: torch.Tensor, row_map: torch.Tensor | None = None,
                     gs: torch.Tensor | None = None, out: torch.Tensor | None = None, out_rows: int | None = None) -> torch.Tensor:
    """d [rows, n]: sorted rows a fp16 [s, k] of expert segments (off) times the fp16 expert stack b [E*n, k]; tile list tb (tiles of 128 rows)."""
    _need_cuda(a, b, tb, off)
    s, k = a.shape
    d = out if out is not None else torch.empty((out_rows or s, n), dtype=torch.float16, device=a.device)
    _lib.check(_lib.lib().kyb_gemm_f16_grouped(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), s, n, k, E, tb.data_ptr(), off.data_ptr(), _p(row_map), _p(gs),
                                               d.data_ptr(), d.stride(0), _stream()))
    return d


def gemm_kq(fmt, t16: torch.Tensor, n: int, k: int, a: torch.Tensor, gscale: float = 1.0, out: torch.Tensor | None = None, msub: int = 0,
            split: int | None = None) -> torch.Tensor:
    """d fp16 [m, n] = a fp16 [m, k] @ W^T with W decoded from its T16 tiles inside the GEMM (no fp16 copy of W in HBM).
    split: number of k-ranges (split-k through an fp32 workspace for products with fewer output tiles than SMs); None = the library's suggestion when msub is 0
    and `flags.GEMM_SPLIT_K` is on, 1 = never."""
    _need_cuda(t16, a)
    if a.dtype != torch.float16 or a.dim() != 2 or a.shape[1] != k:
        raise ValueError(f"gemm_kq takes float16 [m, {k}], got {a.dtype} {tuple(a.shape)}")
    if a.stride(1) != 1:
        a = a.contiguous()
    m = a.shape[0]
    d = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=a.device)
    L = _lib.lib()
    if split is None:
        split = L.kyb_gemm_kq_split(_fmt(fmt), n, k, m) if (msub == 0 and F.GEMM_SPLIT_K) else 1
    if split > 1:
        need = L.kyb_gemm_kq_split_bytes(n, m, split)
        ws = workspace(a.device, need)
        _lib.check(L.kyb_gemm_kq_splitk(_fmt(fmt), t16.data_ptr(), n, k, a.data_ptr(), a.stride(0), m, float(gscale), d.data_ptr(), d.stride(0), split, ws.data_ptr(),
                                        ws.numel(), _stream()))
        return d
    _lib.check(L.kyb_gemm_kq(_fmt(fmt), t16.data_ptr(), n, k, a.data_ptr(), a.stride(0), m, float(gscale), d.data_ptr(), d.stride(0), msub, _stream()))
    return d


def gemm_kq_ag(fmt, t16: torch.Tensor, n: int, k: int, a: torch.Tensor, peer_ptrs, ldd: int, col0: int, gscale: float = 1.0, msub: int = 0) -> None:
    """gemm_kq whose epilogue stores every tile into the [m, ldd] fp16 output matrix of every rank (peer_ptrs: peer-mapped base addresses, own rank included) at
    column col0: the all-gather of an N-sharded linear happens inside the GEMM. The caller synchronises the ranks around the call."""
    _need_cuda(t16, a)
    if a.dtype != torch.float16 or a.dim() != 2 or a.shape[1] != k:
        raise ValueError(f"gemm_kq_ag takes float16 [m, {k}], got {a.dtype} {tuple(a.shape)}")
    if a.stride(1) != 1:
        a = a.contiguous()
    out = _lib.PeerOut.of(peer_ptrs)
    _lib.check(_lib.lib().kyb_gemm_kq_ag(_fmt(fmt), t16.data_ptr(), n, k, a.data_ptr(), a.stride(0), a.shape[0], float(gscale), out, ldd, col0, msub, _stream()))


def gemm_kq_grouped(fmt, t16: torch.Tensor, n: int, k: int, E: int, a: torch.Tensor, tb: torch.Tensor, off: torch.Tensor, row_map: torch.Tensor | None = None,
                    gs: torch.Tensor | None = None, out: torch.Tensor | None = None, out_rows: int | None = None, mt: int = 256) -> torch.Tensor:
    """d [rows, n]: sorted rows a fp16 [s, k] of expert segments (off) times the T16 expert stack (E * n rows), decoded inside the GEMM; tile list tb of mt-row
    tiles (moe_plan with the same mt, 128 or 256)."""
    _need_cuda(t16, a, tb, off)
    s = a.shape[0]
    d = out if out is not None else torch.empty((out_rows or s, n), dtype=torch.float16, device=a.device)
    _lib.check(_lib.lib().kyb_gemm_kq_grouped(_fmt(fmt), t16.data_ptr(), n, k, E, a.data_ptr(), a.stride(0), s, tb.data_ptr(), off.data_ptr(), _p(row_map), _p(gs),
                                              d.data_ptr(), d.stride(0), mt, _stream()))
    return d


def gemm_kq_grouped_glu(fmt, t16_gate: torch.Tensor, t16_up: torch.Tensor, n: int, k: int, E: int, a: torch.Tensor, tb: torch.Tensor, off: torch.Tensor,
                        gs_gate: torch.Tensor | None = None, gs_up: torch.Tensor | None = None, limit: float | None = None, mt: int = 256) -> torch.Tensor:
    """h fp16 [s, n] = silu(a W_gate^T) * (a W_up^T) on sorted rows, the gate and up stacks of a routed layer in ONE grouped product with the gated activation in
    its epilogue (both products rounded to fp16 first, as the separate launches would store them)."""
    _need_cuda(t16_gate, t16_up, a, tb, off)
    s = a.shape[0]
    h = torch.empty((s, n), dtype=torch.float16, device=a.device)
    _lib.check(_lib.lib().kyb_gemm_kq_grouped_glu(_fmt(fmt), t16_gate.data_ptr(), t16_up.data_ptr(), n, k, E, a.data_ptr(), a.stride(0), s, tb.data_ptr(), off.data_ptr(),
                                                  _p(gs_gate), _p(gs_up), float(limit or 0.0), h.data_ptr(), h.stride(0), mt, _stream()))
    return h


# ------------------------------------------------------------------------------------------------ NVFP4 tensor-core path
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def nvfp4_sf_bytes(rows: int, k: int) -> int:
    return _lib.lib().kyb_nvfp4_sf_bytes(rows, k)


def nvfp4_quant_rows(x: torch.Tensor, swizzled: bool = True, plain: bool = True):
    """x fp16 / bf16 [rows, k] -> (codes uint8 [rows, k/2], plain scales uint8 [rows, k/16] or None, chunk-layout scales uint8 or None)."""
    _need_cuda(x)
    if x.dtype not in (torch.float16, torch.bfloat16) or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("nvfp4_quant_rows takes fp16 / bf16 [rows, k]")
    rows, k = x.shape
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    sp = torch.empty((rows, k // 16), dtype=torch.uint8, device=x.device) if plain else None
    ss = torch.empty(nvfp4_sf_bytes(rows, k), dtype=torch.uint8, device=x.device) if swizzled else None
    _lib.check(_lib.lib().kyb_nvfp4_quant_rows(x.data_ptr(), _DT[x.dtype], x.stride(0), rows, k, codes.data_ptr(), _p(sp), _p(ss), _stream()))
    return codes, sp, ss


def nvfp4_unpack_rows(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.float16) -> torch.Tensor:
    _need_cuda(codes, scales)
    rows, k = codes.shape[0], codes.shape[1] * 2
    out = torch.empty((rows, k), dtype=dtype, device=codes.device)
    _lib.check(_lib.lib().kyb_nvfp4_unpack_rows(codes.data_ptr(), scales.data_ptr(), rows, k, _DT[dtype], out.data_ptr(), k, _stream()))
    return out


def nvfp4_sf_swizzle(plain: torch.Tensor, k: int) -> torch.Tensor:
    """plain scale bytes [rows, k/16] -> chunk layout."""
    _need_cuda(plain)
    plain = plain.contiguous()
    rows = plain.shape[0]
    out = torch.empty(nvfp4_sf_bytes(rows, k), dtype=torch.uint8, device=plain.device)
    _lib.check(_lib.lib().kyb_nvfp4_sf_swizzle(plain.data_ptr(), rows, k, out.data_ptr(), 1, _stream()))
    return out


def nvfp4_sf_unswizzle(swz: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    out = torch.empty((rows, k // 16), dtype=torch.uint8, device=swz.device)
    _lib.check(_lib.lib().kyb_nvfp4_sf_swizzle(out.data_ptr(), rows, k, swz.data_ptr(), 0, _stream()))
    return out


def gemm_nvfp4_ag(a_codes, sfa, b_codes, sfb, m: int, n: int, k: int, peer_ptrs, ldd: int, col0: int, gscale: float = 1.0, dtype=torch.float16) -> None:
    """gemm_nvfp4 with the all-gather of an N-sharded linear folded into the epilogue (see gemm_kq_ag)."""
    _need_cuda(a_codes, sfa, b_codes, sfb)
    out = _lib.PeerOut.of(peer_ptrs)
    _lib.check(_lib.lib().kyb_gemm_nvfp4_ag(a_codes.data_ptr(), sfa.data_ptr(), b_codes.data_ptr(), sfb.data_ptr(), m, n, k, float(gscale), _DT[dtype], out, ldd, col0, _stream()))


def gemm_nvfp4(a_codes, sfa, b_codes, sfb, m: int, n: int, k: int, gscale: float = 1.0, dtype=torch.float16, out=None) -> torch.Tensor:
    """d [m, n] = gscale * dequant(A) dequant(B)^T on block-scaled tcgen05 (scales in the chunk layout)."""
    _need_cuda(a_codes, sfa, b_codes, sfb)
    d = out if out is not None else torch.empty((m, n), dtype=dtype, device=a_codes.device)
    _lib.check(_lib.lib().kyb_gemm_nvfp4(a_codes.data_ptr(), sfa.data_ptr(), b_codes.data_ptr(), sfb.data_ptr(), m, n, k, float(gscale), _DT[d.dtype], d.data_ptr(),
                                         d.stride(0), _stream()))
    return d
