"""Quantized linear modules on the device: torch mirror of kyojin_mlx/foreign_linear.py (`DevPack` :464-1167, `ForeignLinear`
:1211-1247, `SplitLinear` :1251-1268, `make_linear` :1271). Same names, argument order and shape conventions; tensors are torch CUDA
tensors, kernels are the sm_100a kernels behind include/kyb.h. There is no CPU path."""
from __future__ import annotations

import numpy as np
import torch

from . import flags as F
from . import foreign_pack as FP
from . import ops


class Split:
    """Members of a fused linear whose GGUF types differ (role of kyojin_mlx/foreign_linear.py `Split`): packs with one input width."""

    def __init__(self, packs):
        self.packs = list(packs)
        self.k = self.packs[0].k
        self.n = sum(p.n for p in self.packs)
        if any(p.k != self.k for p in self.packs):
            raise ValueError("Split: members differ in input width")


class DevPack:
    """The device arrays of one weight matrix, or of a stack of E expert matrices (E * n rows, expert e = rows [e n, (e + 1) n)),
    as kyojin_mlx/foreign_linear.py:493-559. One resident copy: the T16 bytes (same size as the stored blocks)."""

    def __init__(self, packs, device="cuda"):
        ps = packs if isinstance(packs, list) else [packs]
        p0 = ps[0]
        if any((p.fmt, p.n, p.k) != (p0.fmt, p0.n, p0.k) for p in ps):
            raise ValueError("experts differ in format / shape")
        self.fmt, self.n, self.k = p0.fmt, p0.n, p0.k
        self.E = len(ps) if isinstance(packs, list) else None
        if self.E and self.n % 16:
            raise ValueError("expert stacks need n % 16 == 0 (a 16-row tile must not straddle two experts)")
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ValueError("DevPack lives on a CUDA device (there is no CPU path)")
        parts = []
        for p in ps:                                                        # repack on the device, one expert at a time
            if p.fmt == "nvfp4":
                parts.append(torch.from_numpy(FP.to_t16(p)).to(dev))
            else:
                parts.append(ops.raw_to_t16(p.fmt, torch.from_numpy(np.ascontiguousarray(p.qs)).to(dev), p.n, p.k))
        self.t16 = parts[0] if len(parts) == 1 else torch.cat(parts)
        gs = [float(np.asarray(p.gscale, np.float32).reshape(-1)[0]) for p in ps]
        self.gscale = gs[0]
        self.gs = torch.tensor(gs, dtype=torch.float32, device=dev)       # one scale per expert (per-tensor scale of a single matrix)
        self.nrows = self.n * (self.E or 1)

    @classmethod
    def from_t16(cls, fmt: str, t16: torch.Tensor, n: int, k: int, E: int | None = None, gscale=1.0):
        """Wraps T16 bytes that are already on the device (synthetic benchmark weights, shards)."""
        self = cls.__new__(cls)
        self.fmt, self.n, self.k, self.E, self.t16 = fmt, n, k, E, t16
        self.gscale = float(gscale)
        self.gs = torch.full((E or 1,), float(gscale), dtype=torch.float32, device=t16.device)
        self.nrows = n * (E or 1)
        if t16.numel() != ops.t16_nbytes(fmt, self.nrows, k):
            raise ValueError(f"T16 buffer of {t16.numel()} bytes does not hold [{self.nrows}, {k}] {fmt}")
        return self

    @property
    def nbytes(self) -> int:
        return self.t16.numel()

    def arrays(self):
        """The resident device arrays (kyojin_mlx/foreign_linear.py:621-622)."""
        return [self.t16, self.gs]

    @classmethod
    def grouped(cls, devs):
        """One DevPack over the concatenated rows of same-input DevPacks (q | k | v, gate | up), members' rows one after the other
        (kyojin_mlx/foreign_linear.py:577-594). Members whose row count is not a multiple of 16 are re-tiled through the stored row form on the device.
        NVFP4 members must share one per-tensor scale (the kernels apply one scale per matrix)."""
        d0 = devs[0]
        if any((d.fmt, d.k, d.E) != (d0.fmt, d0.k, None) for d in devs):
            raise ValueError("grouped: one format, one k, no expert stacks")
        if any(d.gscale != d0.gscale for d in devs):
            raise ValueError("grouped: members differ in their per-tensor scale")
        n = sum(d.n for d in devs)
        if all(d.n % 16 == 0 for d in devs[:-1]):
            t16 = torch.cat([d.t16 for d in devs])
        else:
            raw = torch.cat([ops.t16_to_raw(d.fmt, d.t16, d.n, d.k) for d in devs])
            t16 = ops.raw_to_t16(d0.fmt, raw, n, d0.k)
        return cls.from_t16(d0.fmt, t16, n, d0.k, None, d0.gscale)

    def rows(self, n) -> "DevPack":
        """A DevPack over output rows of one matrix: n = an int (the first n rows) or a 1-D sequence of row ids, gathered in that order
        (kyojin_mlx/foreign_linear.py:596-619). The per-tensor scale stays."""
        if self.E:
            raise ValueError("rows: one matrix")
        if isinstance(n, int):
            if not 0 < n <= self.n:
                raise ValueError("rows: 0 < n <= N")
            if n % 16 == 0:
                return DevPack.from_t16(self.fmt, self.t16[:ops.t16_nbytes(self.fmt, n, self.k)].clone(), n, self.k, None, self.gscale)
            idx = torch.arange(n, device=self.t16.device)
        else:
            idx = torch.as_tensor(np.asarray(n).astype(np.int64), device=self.t16.device)
            if idx.dim() != 1 or not 0 < idx.numel() <= self.n:
                raise ValueError("rows: 1-D index, 0 < len <= N")
        raw = ops.t16_to_raw(self.fmt, self.t16, self.n, self.k).index_select(0, idx)
        return DevPack.from_t16(self.fmt, ops.raw_to_t16(self.fmt, raw.contiguous(), idx.numel(), self.k), idx.numel(), self.k, None, self.gscale)

    # ---- one matrix, x2 [R, k] fp16 -> [R, n] fp16 (row-count dispatch of foreign_linear.py:672-737)
    def apply(self, x2: torch.Tensor) -> torch.Tensor:
        if self.E:
            raise ValueError("apply() is for one matrix; expert stacks go through gather / ForeignSwitchGLU")
        R = x2.shape[0]
        if R == 0:
            return torch.empty((0, self.n), dtype=torch.float16, device=x2.device)
        if R <= F.GEMV_ROWS:
            # chained launches only once a plain launch of this matrix has run: whatever wrote the weights then lies further back in the stream
            chained, self._settled = F.GEMV_CHAINED and getattr(self, "_settled", False), True
            return ops.gemv(self.fmt, self.t16, self.n, self.k, x2, self.gscale, chained=chained)
        if R < F.GEMM_MIN_ROWS:
            return self._rows_chunked(x2)
        return self._prefill(x2)

    def _rows_chunked(self, x2):
        """A few more rows than one few-row launch takes: 32-row slices, one weight read each."""
        y = torch.empty((x2.shape[0], self.n), dtype=torch.float16, device=x2.device)
        for i in range(0, x2.shape[0], 32):
            ops.gemv(self.fmt, self.t16, self.n, self.k, x2[i:i + 32], self.gscale, out=y[i:i + 32])
        return y

    def _prefill(self, x2):
        """Prefill: one tcgen05 GEMM whose weight operand is decoded from the T16 tiles inside the kernel (fp16 weights in shared memory only, fp32
        accumulation); role of the reference's large-row path (foreign_linear.py:710 `x2 @ self.dequant().T`). The NVFP4 per-tensor scale is applied to the
        fp32 accumulator, not folded into the fp16 weights. KYB_PREFILL_TWO_STEP=1 runs the staged form instead (fp16 matrix in HBM, then the fp16 GEMM)."""
        from .layout import PREFILL_FUSED
        if F.PREFILL_TWO_STEP or self.fmt not in PREFILL_FUSED:
            return self._prefill_two_step(x2)
        return ops.gemm_kq(self.fmt, self.t16, self.n, self.k, x2, self.gscale)

    def _prefill_two_step(self, x2):
        w16 = ops.dequant(self.fmt, self.t16, self.n, self.k, torch.float16, 1.0)
        return ops.gemm_f16(x2, w16, self.gscale)

    # ---- NVFP4 W4A4: activations quantised on the fly with the weights' block rule, block-scaled tcgen05 GEMM (no counterpart kernel in the reference, whose
    # NVFP4 linear is W4A16; this serves the benchmark's NVFP4 prefill configuration)
    def _a4_operands(self):
        if getattr(self, "_a4", None) is None:
            if self.fmt != "nvfp4" or self.E:
                raise ValueError("apply_a4() is for one NVFP4 matrix")
            raw = ops.t16_to_raw("nvfp4", self.t16, self.n, self.k)                       # GGUF NVFP4 rows, back from T16 on the device
            blk = raw.reshape(self.n, self.k // 64, 36)
            sc = blk[:, :, 0:4].reshape(self.n, self.k // 16).contiguous()
            q = blk[:, :, 4:36].reshape(self.n, self.k // 64, 4, 8)
            codes = torch.cat([q & 15, q >> 4], dim=-1).reshape(self.n, self.k)          # byte j of a 16-sub-block = inputs j and j + 8
            qs = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
            self._a4 = (qs, ops.nvfp4_sf_swizzle(sc, self.k))
        return self._a4

    def apply_a4(self, x2: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
        """y = quant_nvfp4(x) W^T on the block-scaled tensor-core path; x fp16 / bf16 [R, k]. Needs n % 256 == 0 and k % 256 == 0."""
        qs, sfb = self._a4_operands()
        if x2.dtype not in (torch.float16, torch.bfloat16):
            x2 = x2.to(torch.bfloat16)
        acodes, _, asw = ops.nvfp4_quant_rows(x2.contiguous(), swizzled=True, plain=False)
        return ops.gemm_nvfp4(acodes, asw, qs, sfb, x2.shape[0], self.n, self.k, self.gscale, out_dtype)

    def dequant(self, dtype=torch.float16) -> torch.Tensor:
        """[rows, k] weights (fp16 saturated as foreign_linear.py:1050-1065, or float32 bit-equal to the reference decoder)."""
        if self.E and self.fmt == "nvfp4" and len(set(self.gs.tolist())) > 1:
            out = torch.empty((self.nrows, self.k), dtype=dtype, device=self.t16.device)
            for e in range(self.E):
                out[e * self.n:(e + 1) * self.n] = ops.dequant(self.fmt, self.t16, self.nrows, self.k, dtype, float(self.gs[e]), e * self.n, self.n)
            return out
        return ops.dequant(self.fmt, self.t16, self.nrows, self.k, dtype, self.gscale)

    # ---- routed-expert slots: slot s uses expert eids[s] and row xrows[s] of x (fp16 [T, k]) -> [S, n]   (foreign_linear.py:1068-1164)
    def gather(self, x, xrows, eids, groups=None):
        if not self.E or x.dtype != torch.float16:
            raise ValueError("gather() needs an expert stack and fp16 rows")
        return ops.gemv_group(self.fmt, self.t16, self.n, self.k, self.E, x, eids, xrows=xrows, gs=self._gs(), groups=groups)

    def _gs(self):
        return self.gs if self.fmt == "nvfp4" else None

    def pair_ok(self, o) -> bool:
        return bool(self.E) and (self.fmt, self.n, self.k, self.E) == (o.fmt, o.n, o.k, o.E)

    def gather_pair(self, o, x, xrows, eids, groups=None):
        """(self.gather(...), o.gather(...)): gate | up of one expert block on the same slots in ONE launch (foreign_linear.py:1119-1154)."""
        y = self.gather_pair_raw(o, x, xrows, eids, groups)
        S = eids.numel()
        return y[:S], y[S:]

    def gather_pair_raw(self, o, x, xrows, eids, groups=None, xdiv=1):
        """[2 S, n]: rows [0, S) = this stack, rows [S, 2 S) = stack o, on the same slots (the input of glu_rows)."""
        if not self.pair_ok(o):
            raise ValueError("gather_pair: two expert stacks of one format and shape")
        return ops.gemv_group(self.fmt, self.t16, self.n, self.k, self.E, x, eids, xrows=xrows, xdiv=xdiv, gs=self._gs(), groups=groups, t16b=o.t16, gsb=o._gs())

    def glu_ok(self) -> bool:
        return bool(self.E)

    def gather_glu(self, a, b, xrows, eids, act=None, limit=None, groups=None):
        """gather() of the down projection on the gated input silu(a) * b (a, b fp16 [S, k]; slot s reads row xrows[s]) (foreign_linear.py:1156-1164): the
        activation is formed while the rows are staged, one launch. Bit-identical to the activation kernel followed by gather()."""
        if act is not None:
            raise NotImplementedError("only the silu-gated activation is built")
        if not self.E or a.dtype != torch.float16:
            raise ValueError("gather_glu() needs an expert stack and fp16 rows")
        return ops.gemv_group(self.fmt, self.t16, self.n, self.k, self.E, a, eids, xrows=xrows, gs=self._gs(), groups=groups, x2=b, limit=limit)

    def apply_glu(self, a, b, limit=None):
        """One matrix on the gated input silu(a) * b (foreign_linear.py:960-977). Up to the decode row limit the activation is formed while the down product
        stages its rows (one launch, no round trip of the gated rows through HBM); more rows run the activation kernel and then the prefill product."""
        if self.E:
            raise ValueError("apply_glu() is for one matrix")
        if 0 < a.shape[0] <= F.GEMV_ROWS and a.dtype == torch.float16 and b.dtype == torch.float16:
            chained, self._settled = F.GEMV_CHAINED and getattr(self, "_settled", False), True
            return ops.gemv(self.fmt, self.t16, self.n, self.k, a, self.gscale, chained=chained, x2=b, limit=limit)
        return self.apply(ops.silu_mul(a, b, limit))

    def expert(self, e: int) -> "DevPack":
        """Row-range view of expert e (no copy), as foreign_linear.py:637-660."""
        if not self.E:
            raise ValueError("not an expert stack")
        tb = ops.t16_nbytes(self.fmt, self.n, self.k)
        return DevPack.from_t16(self.fmt, self.t16[e * tb:(e + 1) * tb], self.n, self.k, None, float(self.gs[e]))


class ForeignLinear(torch.nn.Module):
    """y = layer(x) for x (..., in_features); output fp16 by default, bias added when present. Arrays are private (not parameters).
    Mirrors kyojin_mlx/foreign_linear.py:1211-1247."""

    def __init__(self, pack, bias=None, out_dtype=torch.float16, in_perm=None, device="cuda"):
        super().__init__()
        if isinstance(pack, Split):
            raise TypeError("a Split (mixed GGUF types) is served by SplitLinear: build it with make_linear")
        self.dev = pack if isinstance(pack, DevPack) else DevPack(pack, device)
        self._in_perm = None if in_perm is None else torch.as_tensor(np.asarray(in_perm).astype(np.int64), device=self.dev.t16.device)
        self.in_features, self.out_features, self.fmt = self.dev.k, self.dev.n, self.dev.fmt
        self.out_dtype = out_dtype
        self._bias = None if bias is None else torch.as_tensor(bias).to(self.dev.t16.device, out_dtype)

    def forward(self, x: torch.Tensor, permuted: bool = False) -> torch.Tensor:
        shape = x.shape
        if shape[-1] != self.in_features:
            raise ValueError(f"input width {shape[-1]} != in_features {self.in_features}")
        x2 = x.reshape(-1, shape[-1])
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        if self._in_perm is not None and not permuted:
            x2 = x2.index_select(1, self._in_perm)
        y = self.dev.apply(x2)
        if y.dtype != self.out_dtype:
            y = y.to(self.out_dtype)
        if self._bias is not None:
            y = y + self._bias
        return y.reshape(*shape[:-1], self.out_features)


class SplitLinear(torch.nn.Module):
    """A fused linear whose members have different GGUF types: one ForeignLinear per member, outputs concatenated on the last axis
    (kyojin_mlx/foreign_linear.py:1251-1268)."""

    def __init__(self, split: Split, bias=None, out_dtype=torch.float16, in_perm=None, device="cuda"):
        super().__init__()
        if in_perm is not None:
            raise ValueError("SplitLinear: a column permutation over mixed-type members is not supported")
        cuts = np.cumsum([0] + [p.n for p in split.packs])
        self.members = torch.nn.ModuleList(ForeignLinear(p, None if bias is None else bias[a:b], out_dtype, None, device)
                                           for p, a, b in zip(split.packs, cuts[:-1], cuts[1:]))
        self.in_features, self.out_features, self.fmt, self.out_dtype = split.k, split.n, "split", out_dtype

    def forward(self, x, permuted: bool = False):
        if permuted:
            raise ValueError("SplitLinear: no permuted input")
        return torch.cat([m(x) for m in self.members], dim=-1)


def make_linear(pack, bias=None, out_dtype=torch.float16, in_perm=None, device="cuda"):
    """ForeignLinear for a Pack, SplitLinear for a Split (kyojin_mlx/foreign_linear.py:1271)."""
    return (SplitLinear if isinstance(pack, Split) else ForeignLinear)(pack, bias, out_dtype, in_perm, device)


class StoredEmbedding(torch.nn.Module):
    """Token embedding kept in its quantized blocks (one resident copy): the rows of the ids are decoded on the fly; `as_linear` (a tied head) runs the
    stored product (kyojin_mlx/foreign_linear.py:1170-1199)."""

    def __init__(self, pack, device="cuda"):
        super().__init__()
        self.dev = pack if isinstance(pack, DevPack) else DevPack(pack, device)
        self.num_embeddings, self.dims = self.dev.n, self.dev.k

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        d = self.dev
        return ops.dequant_rows(d.fmt, d.t16, d.n, d.k, ids.reshape(-1), torch.float16, d.gscale).reshape(*ids.shape, self.dims)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        return self.dev.apply(x.reshape(-1, shape[-1]).to(torch.float16)).reshape(*shape[:-1], self.num_embeddings)


def glu_rows(y, S: int, limit=None):
    """Gated activation over a [2 S, n] pair output (rows [0, S) = gate, [S, 2 S) = up), one launch (foreign_linear.py:1316-1319)."""
    return ops.silu_mul(y[:S], y[S:], limit)


class ForeignSwitchGLU(torch.nn.Module):
    """mlx-lm SwitchGLU drop-in: (x [.., H], inds [.., K]) -> [.., K, H] UNWEIGHTED per-slot outputs; silu(gate x) * (up x) -> down
    (kyojin_mlx/foreign_linear.py:1333-1514). Up to GATHER_MAX slots: gathered GEMV with expert election (an expert's bytes are read once per 8 slots).
    More slots (prefill): slots sorted by expert on the device, grouped tcgen05 GEMM over 128-row tiles of one expert, scatter back to slot order."""

    def __init__(self, gate: DevPack, up: DevPack, down: DevPack, limit: float | None = None, act_kind=None):
        super().__init__()
        if act_kind is not None:
            raise NotImplementedError("only the silu-gated activation is built")
        if not (gate.E and gate.E == up.E == down.E) or (gate.n, gate.k) != (up.n, up.k) or down.k != gate.n or down.n != gate.k:
            raise ValueError("gate / up / down must be expert stacks of matching shapes")
        self.g, self.u, self.d = gate, up, down
        self.limit = limit

    def forward(self, x, inds):
        lead, H = x.shape[:-1], x.shape[-1]
        K = inds.shape[-1]
        T = int(np.prod(lead)) if len(lead) else 1
        x2 = x.reshape(T, H).to(torch.float16)
        e32 = inds.reshape(-1).to(torch.int32)
        S = T * K
        if S <= max(F.GATHER_MAX, F.GATHER_PER_EXPERT * self.g.E):
            y = self._gather_path(x2, e32, K)
        else:
            from . import foreign_kqgmm as KQ
            y = KQ.mlp(self, x2, e32, K)
        return y.reshape(*lead, K, self.d.n)

    def _gather_path(self, x2, e32, K):
        """Three projections, two launches after one election: gate | up as a pair, then down with the gated activation formed while its rows are staged."""
        S = e32.numel()
        groups = ops.moe_groups(e32, self.g.E)
        if self.g.pair_ok(self.u):
            ab = self.g.gather_pair_raw(self.u, x2, None, e32, groups, xdiv=K)
            a, b = ab[:S], ab[S:]
        else:                                                                 # gate and up stored in different formats
            a = ops.gemv_group(self.g.fmt, self.g.t16, self.g.n, self.g.k, self.g.E, x2, e32, xdiv=K, gs=self.g._gs(), groups=groups)
            b = ops.gemv_group(self.u.fmt, self.u.t16, self.u.n, self.u.k, self.u.E, x2, e32, xdiv=K, gs=self.u._gs(), groups=groups)
        return self.d.gather_glu(a, b, None, e32, limit=self.limit, groups=groups)


# ------------------------------------------------------------------------------------------------ same-input groups and the fused dense gated MLP (installers)
class _Group:
    """One concatenated matrix serving several same-input linears: the first member called with an input runs the product, the others take their slice of it
    (role of kyojin_mlx/foreign_linear.py `_Group`)."""

    def __init__(self, dev: DevPack, cuts):
        self.dev, self.cuts = dev, list(cuts)
        self.x = self.ys = None


class GroupMember(torch.nn.Module):
    """Stand-in for one ForeignLinear of a same-input group: same call, same output (its own rows of the grouped product, bias, output type); mirrors
    kyojin_mlx/foreign_linear.py:1527-1577. The grouped product runs once per distinct input object; the group keeps only a weak reference to that input."""

    def __init__(self, grp: _Group, i: int, src: ForeignLinear):
        super().__init__()
        self._g, self._i = grp, i
        self.in_features, self.out_features, self.fmt = src.in_features, src.out_features, src.fmt
        self.out_dtype, self._bias = src.out_dtype, src._bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        import weakref
        g, shape = self._g, x.shape
        if g.x is None or g.x() is not x or g.ys[self._i] is None:
            x2 = x.reshape(-1, shape[-1])
            if x2.dtype != torch.float16:
                x2 = x2.to(torch.float16)
            y = g.dev.apply(x2)
            g.ys = [y[:, a:b] for a, b in zip(g.cuts[:-1], g.cuts[1:])]
            g.x = weakref.ref(x)
        y, g.ys[self._i] = g.ys[self._i], None                   # every member takes its slice once
        if y.dtype != self.out_dtype:
            y = y.to(self.out_dtype)
        if self._bias is not None:
            y = y + self._bias
        return y.reshape(*shape[:-1], self.out_features)


def trace_calls(model: torch.nn.Module, example_inputs=None):
    """One forward in which every ForeignLinear / GroupMember / ForeignSwitchGLU only records (id of its input object, id of the module) and returns zeros of its
    output shape -> the list of records (role of kyojin_mlx/foreign_linear.py:1596-1613). example_inputs: the arguments of the forward (default: one token id)."""
    calls, keep = [], []
    orig_l, orig_s = ForeignLinear.forward, ForeignSwitchGLU.forward

    def rec_l(self, x, permuted=False):
        calls.append((id(x), id(self)))
        keep.append(x)                                           # ids stay unique while the trace holds the tensors
        return torch.zeros((*x.shape[:-1], self.out_features), dtype=self.out_dtype, device=x.device)

    def rec_s(self, x, inds):
        return torch.zeros((*x.shape[:-1], inds.shape[-1], self.d.n), dtype=torch.float16, device=x.device)

    ForeignLinear.forward, ForeignSwitchGLU.forward = rec_l, rec_s
    try:
        with torch.no_grad():
            if example_inputs is None:
                dev = next((m.dev.t16.device for m in model.modules() if isinstance(m, ForeignLinear)), torch.device("cuda"))
                example_inputs = (torch.zeros((1, 1), dtype=torch.int64, device=dev),)
            model(*example_inputs)
    finally:
        ForeignLinear.forward, ForeignSwitchGLU.forward = orig_l, orig_s
    return calls


def find_groups(calls, names):
    """calls: [(input object id, module id)] of one forward; names: module id -> name. Lists of >= 2 distinct named modules that received the same input object,
    each called exactly once in the forward, in first-call order."""
    times = {}
    for _, mid in calls:
        times[mid] = times.get(mid, 0) + 1
    buckets = {}
    for xid, mid in calls:
        if times[mid] == 1 and mid in names:
            buckets.setdefault(xid, []).append(names[mid])
    return [members for members in buckets.values() if len(members) >= 2]


def group_ok(lins) -> bool:
    """The grouped rows must be what every member computes alone: plain ForeignLinears of one format, input width, output type and per-tensor scale, no input
    permutation, no expert stacks."""
    l0 = lins[0]
    if any(type(l) is not ForeignLinear or l.dev is None or l.dev.E is not None or l._in_perm is not None for l in lins):
        return False
    return all((l.fmt, l.in_features, l.out_dtype, l.dev.gscale) == (l0.fmt, l0.in_features, l0.out_dtype, l0.dev.gscale) for l in lins)


def _set_module(model, name, new):
    parent = model
    *path, leaf = name.split(".")
    for p in path:
        parent = getattr(parent, p)
    setattr(parent, leaf, new)


def group_same_input(model: torch.nn.Module, example_inputs=None, log=print) -> dict:
    """Replaces the ForeignLinears that read the same input (q | k | v, gate | up) by GroupMembers over one concatenated matrix, so that a decode step launches
    one product per group (kyojin_mlx/foreign_linear.py:1617-1655). Groups are built one at a time and the members' own arrays dropped before the next. A model
    whose trace fails is left as it is. Returns {"groups", "members", "launches_saved"}."""
    named = {n: m for n, m in model.named_modules() if type(m) is ForeignLinear}
    try:
        groups = find_groups(trace_calls(model, example_inputs), {id(m): n for n, m in named.items()})
    except Exception as e:                                                # noqa: BLE001 - a forward that needs other arguments: stay as served
        log(f"[foreign] same-input grouping skipped ({type(e).__name__}: {e})")
        return {"groups": 0, "members": 0, "launches_saved": 0}
    parts = []
    for g in groups:                                                      # a same-input set of mixed formats splits into one group per (format, k, out dtype)
        by = {}
        for n in g:
            by.setdefault((named[n].fmt, named[n].in_features, named[n].out_dtype), []).append(n)
        parts += [p for p in by.values() if len(p) >= 2]
    ngroups = members = saved = 0
    for g in parts:
        lins = [named[n] for n in g]
        if not group_ok(lins):
            continue
        grp = _Group(DevPack.grouped([l.dev for l in lins]), [0] + list(np.cumsum([l.out_features for l in lins])))
        for i, (n, l) in enumerate(zip(g, lins)):
            _set_module(model, n, GroupMember(grp, i, l))
            l.dev = None
        ngroups, members, saved = ngroups + 1, members + len(g), saved + len(g) - 1
    log(f"[foreign] {members} linears in {ngroups} same-input groups, {saved} fewer launches per decode step")
    return {"groups": ngroups, "members": members, "launches_saved": saved}


PROJ = ("gate_proj", "up_proj", "down_proj")


class _Probe(torch.nn.Module):
    def __init__(self, fn):
        super().__init__()
        self._fn = fn

    def forward(self, x):
        return self._fn(x)


def silu_gated(mod) -> bool:
    """True when the module's own forward is down(silu(gate(x)) * up(x)): probed on stand-in projections (gate = identity, up = ones, down = identity) against
    silu. A gated MLP with another activation keeps its call (the fused launch computes silu). Any failure of the probe = False."""
    import copy
    try:
        m = copy.copy(mod)
        m._modules = dict(mod._modules)
        m.gate_proj, m.up_proj, m.down_proj = _Probe(lambda x: x), _Probe(lambda x: torch.ones_like(x)), _Probe(lambda x: x)
        x = torch.linspace(-4.0, 4.0, 33).reshape(1, 1, 33)
        return bool(torch.allclose(type(mod).forward(m, x), torch.nn.functional.silu(x), atol=1e-5))
    except Exception:                                                     # noqa: BLE001
        return False


def _glu_call(self, x):
    """down(silu(gate(x)) * up(x)) for decode rows: the activation is formed while the down projection stages its rows, so the MLP is gate | up plus ONE launch
    (kyojin_mlx/foreign_linear.py:1882-1907). Any other case runs the module's own forward."""
    dn, g, u = self.down_proj, self.gate_proj, self.up_proj
    lead, H = x.shape[:-1], x.shape[-1]
    R = int(np.prod(lead)) if len(lead) else 1
    K = dn.in_features
    if dn.dev is None or R == 0 or R > F.GEMV_ROWS:
        return self._stock_call(x)
    x2 = x.reshape(-1, H)
    if x2.dtype != torch.float16:
        x2 = x2.to(torch.float16)
    if isinstance(g, GroupMember) and isinstance(u, GroupMember):
        grp = g._g
        if u._g is not grp or (g._i, u._i) != (0, 1) or grp.cuts != [0, K, 2 * K]:
            return self._stock_call(x)
        y = grp.dev.apply(x2)                                             # [R, 2 K]: gate | up in one launch
        out = dn.dev.apply_glu(y[:, :K], y[:, K:])
    else:
        if type(g) is not ForeignLinear or type(u) is not ForeignLinear or g.dev is None or u.dev is None:
            return self._stock_call(x)
        out = dn.dev.apply_glu(g(x).reshape(R, K), u(x).reshape(R, K))
    return out.reshape(*lead, dn.out_features)


def install_dense_glu(model: torch.nn.Module, log=print) -> int:
    """Swaps the forward of every gated MLP (gate_proj / up_proj / down_proj, silu-gated by probe) whose down projection is a plain fp16 ForeignLinear for the fused
    call above (kyojin_mlx/foreign_linear.py:1934-1953). Returns the number of modules changed."""
    n = 0
    for _, mod in list(model.named_modules()):
        g, u, dn = (getattr(mod, k, None) for k in PROJ)
        if type(dn) is not ForeignLinear or getattr(mod.__class__, "_dense_glu", False) or not silu_gated(mod):
            continue
        ok = lambda l: (type(l) is ForeignLinear and l.dev is not None) or type(l) is GroupMember
        if not (ok(g) and ok(u)) or dn._bias is not None or dn._in_perm is not None or dn.out_dtype != torch.float16:
            continue
        if any(l.out_dtype != torch.float16 or l._bias is not None or l.out_features != dn.in_features for l in (g, u)):
            continue
        cls = mod.__class__
        mod.__class__ = type("Glu" + cls.__name__, (cls,), {"forward": _glu_call, "_stock_call": cls.forward, "_dense_glu": True})
        n += 1
    if n:
        log(f"[foreign] {n} gated MLPs form silu * mul inside the down projection's launch")
    return n
