"""Multi-GPU plumbing of the quantized linear over torch.distributed (NCCL on GPUs; the index / split logic is backend-agnostic and runs on gloo for tests).
The reference is single-device; this is new design for an 8 x B200 box:

* dense linears: the output dimension n is column-sharded in whole 16-row tiles (a T16 shard is a contiguous byte range), activations are replicated, every
  rank runs its shard and the output slices are all-gathered;
* routed experts: expert-parallel. Experts are split in contiguous ranges, tokens stay data-parallel; routed slots are sent to the rank that owns their expert
  with one all-to-all, run through that rank's local expert stack, and sent back with the mirrored all-to-all; the owner combines them with the routing weights.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------ dense: n-sharding
def shard_rows(n: int, world: int, rank: int, align: int = 16):
    """Rows [row0, row0 + rows) of rank `rank`: contiguous, whole `align`-row tiles, sizes differ by at most one tile."""
    tiles = (n + align - 1) // align
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    nt = base + (1 if rank < extra else 0)
    row0 = t0 * align
    return row0, max(0, min(n, (t0 + nt) * align) - row0)


def shard_t16(fmt: str, t16: torch.Tensor, n: int, k: int, world: int, rank: int):
    """The byte range of a T16 matrix that holds rank's rows (no copy): returns (view, row0, rows)."""
    from .layout import TILE_BYTES
    row0, rows = shard_rows(n, world, rank)
    per_tile_row = (k // 256) * TILE_BYTES[fmt]
    return t16[(row0 // 16) * per_tile_row:((row0 + rows + 15) // 16) * per_tile_row], row0, rows


class ShardedLinear:
    """y [m, n] = all-gather over ranks of x @ W[shard]^T. `local` is any callable x -> y_local (a ForeignLinear on this rank's shard)."""

    def __init__(self, local, n: int, group=None):
        self.local, self.n, self.group = local, n, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.splits = [shard_rows(n, self.world, r)[1] for r in range(self.world)]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        m = y.shape[0]
        if len(set(self.splits)) == 1:                                      # equal shards: one all-gather into [world, m, n / world]
            out = torch.empty((self.world * m, self.splits[0]), dtype=y.dtype, device=y.device)
            dist.all_gather_into_tensor(out, y.contiguous(), group=self.group)
            return out.view(self.world, m, -1).permute(1, 0, 2).reshape(m, self.n)
        mx = max(self.splits)                                               # uneven shards: pad the slices to the widest, gather, cut
        pad = torch.zeros((m, mx), dtype=y.dtype, device=y.device)
        pad[:, :y.shape[1]] = y
        out = torch.empty((self.world * m, mx), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(out, pad, group=self.group)
        out = out.view(self.world, m, mx)
        return torch.cat([out[r, :, :s] for r, s in enumerate(self.splits)], dim=1)


class PeerGather:
    """All-gather of the output slices of a whole decode step: every rank stores its (small) local outputs into ALL ranks' gathered buffers with ONE copy launch
    (plain 16-byte stores to peer-mapped symmetric memory over NVLink) followed by ONE device-side barrier, instead of one NCCL all-gather per product. The
    staged form (`begin` / `store` / `finish`) sends parts of the step early, on a second stream, and keeps the single barrier.
    shapes[i] = (m, n_local) of product i (the same on every rank; pad uneven shards); dtype float16. gathered(i) is this rank's [world, m, n_local] view, valid
    until the call after next (two buffer sets alternate)."""

    def __init__(self, shapes, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shapes = [tuple(s) for s in shapes]
        self.bytes = [m * n * 2 for m, n in self.shapes]
        if any(b % 16 for b in self.bytes):
            raise ValueError("every local output must be a multiple of 16 bytes")
        self.offs, tot = [], 0
        for b in self.bytes:
            self.offs.append(tot)
            tot += (self.world * b + 255) // 256 * 256
        self.bufs = [symm.empty(tot, dtype=torch.uint8, device=device) for _ in range(2)]
        self.hdls = [symm.rendezvous(b, self.group) for b in self.bufs]
        self.turn, self.last = 0, 0

    def __call__(self, outs) -> None:
        """outs[i]: this rank's contiguous fp16 [m, n_local] result of product i (on the current stream)."""
        from . import ops
        i, self.turn = self.turn, self.turn ^ 1
        hdl = self.hdls[i]
        srcs, dsts, sizes = [], [], []
        for o, off, b in zip(outs, self.offs, self.bytes):
            if o.numel() * o.element_size() != b or not o.is_contiguous():
                raise ValueError("output does not match its registered shape")
            for base in hdl.buffer_ptrs:
                srcs.append(o)
                dsts.append(int(base) + off + self.rank * b)
                sizes.append(b)
        ops.gather_flat(srcs, dsts, sizes)
        hdl.barrier()
        self.last = i

    def begin(self) -> None:
        """Staged form: takes the next buffer set. `store` then sends some of the step's outputs (no barrier), `finish` ends the step with the one barrier.
        A caller can issue each `store` on a second stream as soon as its outputs exist, so that the NVLink transfers run under the products that follow."""
        self.last, self.turn = self.turn, self.turn ^ 1

    def store(self, indices, outs) -> None:
        """Copies this rank's outputs `outs` of the products `indices` into every rank's buffers of the current set (one launch, no barrier)."""
        from . import ops
        hdl = self.hdls[self.last]
        srcs, dsts, sizes = [], [], []
        for i, o in zip(indices, outs):
            b = self.bytes[i]
            if o.numel() * o.element_size() != b or not o.is_contiguous():
                raise ValueError("output does not match its registered shape")
            for base in hdl.buffer_ptrs:
                srcs.append(o)
                dsts.append(int(base) + self.offs[i] + self.rank * b)
                sizes.append(b)
        ops.gather_flat(srcs, dsts, sizes)

    def finish(self) -> None:
        """One device-side barrier: every rank's stores of the step have landed. (Stream order must put every `store` of the step before this call.)"""
        self.hdls[self.last].barrier()

    def gathered(self, i: int) -> torch.Tensor:
        m, n = self.shapes[i]
        b = self.bytes[i]
        return self.bufs[self.last][self.offs[i]:self.offs[i] + self.world * b].view(torch.float16).reshape(self.world, m, n)


class FusedShardedLinear:
    """N-sharded prefill linear whose GEMM writes every output tile into the output matrix of EVERY rank (peer stores over NVLink from the epilogue), so the
    all-gather overlaps the tensor-core work tile by tile; one device-side barrier per call tells the ranks that all tiles have landed. `dev` is this rank's DevPack
    shard (rows [row0, row0 + dev.n) of the [n_total, k] matrix, shard_rows with whole 16-row tiles). a4 = True runs the NVFP4 W4A4 path (activations quantised on
    the fly). Outputs live in two alternating symmetric-memory buffers of max_rows rows: the tensor returned by call c is valid until call c + 2, and the
    consumer must read it on the stream of the call. Rows <= 32 (decode) are served by ShardedLinear (GEMV + NCCL all-gather): they are latency-bound either way."""

    def __init__(self, dev, n_total: int, max_rows: int, group=None, a4: bool = False, out_dtype=torch.float16, msub: int = 0):
        import torch.distributed._symmetric_memory as symm
        self.dev, self.n, self.group, self.a4, self.out_dtype = dev, n_total, group or dist.group.WORLD, a4, out_dtype
        self.msub = msub                                                     # K-quant GEMM: activation blocks per work item (1: the peer stores of a tile overlap the next tile's MMAs)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        align = 256 if a4 else 16
        self.col0, rows = shard_rows(n_total, self.world, self.rank, align)
        if rows != dev.n:
            raise ValueError(f"this rank's shard has {dev.n} rows, shard_rows gives {rows}")
        if n_total % 8:
            raise ValueError("the gathered width must be a multiple of 8")
        self.bufs = [symm.empty((max_rows, n_total), dtype=out_dtype, device=dev.t16.device) for _ in range(2)]
        self.hdls = [symm.rendezvous(b, self.group) for b in self.bufs]
        self.turn = 0

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        from . import ops
        m = x.shape[0]
        i, self.turn = self.turn, self.turn ^ 1
        buf, hdl = self.bufs[i], self.hdls[i]
        if m > buf.shape[0]:
            raise ValueError(f"{m} rows exceed the buffer of {buf.shape[0]}")
        ptrs = list(hdl.buffer_ptrs)
        d = self.dev
        if self.a4:
            qs, sfb = d._a4_operands()
            if x.dtype not in (torch.float16, torch.bfloat16):
                x = x.to(torch.bfloat16)
            codes, _, asw = ops.nvfp4_quant_rows(x.contiguous(), swizzled=True, plain=False)
            ops.gemm_nvfp4_ag(codes, asw, qs, sfb, m, d.n, d.k, ptrs, self.n, self.col0, d.gscale, self.out_dtype)
        else:
            if self.out_dtype != torch.float16:
                raise ValueError("the K-quant GEMM writes float16")
            ops.gemm_kq_ag(d.fmt, d.t16, d.n, d.k, x.to(torch.float16), ptrs, self.n, self.col0, d.gscale, self.msub)
        hdl.barrier()                                                        # every rank's tiles have landed in every buffer
        return buf[:m]


# ------------------------------------------------------------------------------------------------ routed experts: expert parallelism
def expert_range(E: int, world: int, rank: int):
    base, extra = divmod(E, world)
    e0 = rank * base + min(rank, extra)
    return e0, base + (1 if rank < extra else 0)


def owner_of(e: torch.Tensor, E: int, world: int) -> torch.Tensor:
    """Rank that owns each expert id (contiguous ranges, the first E % world ranks hold one more)."""
    base, extra = divmod(E, world)
    cut = extra * (base + 1)
    return torch.where(e < cut, e // (base + 1), extra + (e - cut) // max(base, 1))


def ep_moe(x: torch.Tensor, inds: torch.Tensor, scs: torch.Tensor, E: int, local_experts, group=None, out_dtype=torch.float32, slot_dtype=None,
           slot_width: int | None = None) -> torch.Tensor:
    """Expert-parallel routed layer. x [T, H] (this rank's tokens), inds [T, K] global expert ids, scs [T, K] routing weights.
    local_experts(rows [S, H], local_ids [S]) -> [S, H_out]: this rank's expert stack applied slot by slot (unweighted), e.g. a ForeignSwitchGLU with K = 1.
    Returns [T, H_out] = sum_k scs[t, k] * expert(inds[t, k])(x[t]). Split sizes are exchanged first (one small all-to-all; the sizes are read on the host).
    slot_dtype / slot_width: dtype and width H_out of what local_experts returns. Every rank must exchange the same element type and width, also a rank that
    receives no slot and so never calls local_experts; give them whenever they differ from x (default: the dtype and width of x)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T, K = inds.shape
    e = inds.reshape(-1).to(torch.int64)
    dest = owner_of(e, E, world)
    order = torch.argsort(dest, stable=True)                                # slots grouped by destination rank
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    e0_of = torch.tensor([expert_range(E, world, r)[0] for r in range(world)], device=e.device)
    send_rows = x[order // K].contiguous()
    send_ids = (e[order] - e0_of[dest[order]]).to(torch.int32).contiguous()
    recv_rows = torch.empty((sum(rc), x.shape[1]), dtype=x.dtype, device=x.device)
    recv_ids = torch.empty(sum(rc), dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=group)
    dist.all_to_all_single(recv_ids, send_ids, rc, sc, group=group)
    sd, sw = slot_dtype or x.dtype, slot_width or x.shape[1]
    y_recv = local_experts(recv_rows, recv_ids) if recv_rows.shape[0] else torch.empty((0, sw), dtype=sd, device=x.device)
    if y_recv.dtype != sd or y_recv.shape[1] != sw:
        raise ValueError(f"local_experts returned {y_recv.dtype} [*, {y_recv.shape[1]}], the exchange was declared as {sd} [*, {sw}] (slot_dtype / slot_width)")
    y_back = torch.empty((send_rows.shape[0], y_recv.shape[1]), dtype=y_recv.dtype, device=x.device)
    dist.all_to_all_single(y_back, y_recv.contiguous(), sc, rc, group=group)
    y_slots = torch.empty_like(y_back)
    y_slots[order] = y_back                                                  # back to slot order (t K + k)
    if y_slots.is_cuda and y_slots.dtype == torch.float16 and out_dtype in (torch.float16, torch.float32):
        from . import ops
        return ops.moe_combine(y_slots, scs.reshape(-1).to(torch.float32).contiguous(), K, dtype=out_dtype)
    w = scs.reshape(T, K, 1).to(torch.float32)
    return (y_slots.reshape(T, K, -1).to(torch.float32) * w).sum(1).to(out_dtype)
