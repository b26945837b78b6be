"""GGUF file reader -> packs for the device kernels: the role of kyojin_mlx/foreign_gguf.py `GgufFile` (:186-308) and of the loader half of
kyojin_mlx/foreign_linear.py `_read_gguf` (:2240-2328), for the formats this package has kernels for (Q4_K, Q3_K, Q6_K, NVFP4; F32 / F16 / BF16 tensors are returned
as arrays). The container format is the public GGUF layout (little endian, versions 2 and 3): magic, version, tensor count, key count, typed key / value pairs,
tensor infos (name, dimensions with the fastest first, ggml type id, offset), then the data section aligned to `general.alignment` (default 32).
Tensor bytes are memory-mapped (zero copy); `load_linear` / `load_experts` hand them to foreign_pack.to_pack and the T16 repack on the device.
A split shard set (gguf-split: <name>-00001-of-0000N.gguf ...) opened through its FIRST shard reads as one logical file: key / value pairs of shard 1, the tensors
of every shard, bytes mapped from the shard that holds the tensor; any gap in the set is an error, never a partial load (kyojin_mlx/foreign_gguf.py:247-285).
Not built: the two layouts of type id 43 (that id is not in the type table here, so such tensors are refused by name)."""
from __future__ import annotations

import glob
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np


# ggml type id -> (name, block elements, block bytes): the public ggml type table (sizes are needed to size every tensor of a file, also the ones without a kernel here)
TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36),
    10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
    16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50), 20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110),
    22: ("IQ2_S", 256, 82), 23: ("IQ4_XS", 256, 136), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 34: ("TQ1_0", 256, 54), 35: ("TQ2_0", 256, 66), 39: ("MXFP4", 32, 17), 40: ("NVFP4", 64, 36),
}
KERNEL_TYPES = ("Q4_K", "Q3_K", "Q6_K", "NVFP4", "Q5_K", "Q8_0", "Q2_K", "IQ4_XS")          # stored formats the CUDA kernels read (after the lossless T16 repack)


class GgufError(ValueError):
    pass


class GgufTypeError(GgufError):
    pass


# ---- container layout (public GGUF specification): "GGUF", u32 version, u64 tensor count, u64 pair count, the pairs, the tensor records, padding, data
_U32, _U64 = struct.Struct("<I"), struct.Struct("<Q")
# value kind -> numpy dtype of a scalar of that kind (kinds 8 = string and 9 = array are handled apart)
_KIND_DTYPE = {0: "u1", 1: "i1", 2: "<u2", 3: "<i2", 4: "<u4", 5: "<i4", 6: "<f4", 7: "u1", 10: "<u8", 11: "<i8", 12: "<f8"}
_MAX_RECORDS = 1 << 20            # tensors or pairs per file
_MAX_RANK = 4                     # ggml tensors have at most four dimensions


@dataclass
class TensorInfo:
    """One tensor record: `ne` as stored (fastest dimension first), ggml type id, offset inside the data section. `shape` is `ne` reversed (rows first);
    `nbytes` is 0 and `known` False for a type id outside the table (the file stays readable, reading that tensor is refused)."""
    name: str
    ne: tuple
    type: int
    offset: int

    def __post_init__(self):
        entry = TYPES.get(self.type)
        self.known = entry is not None
        self.tname = entry[0] if entry else f"ID{self.type}"
        self.nbytes = 0
        if entry:
            _, per_block, block_bytes = entry
            count = 1
            for d in self.ne:
                count *= d
            inner = self.ne[0] if self.ne else 1
            if inner % per_block:
                raise GgufError(f"{self.name}: {self.tname} stores blocks of {per_block} values, the innermost dimension is {inner}")
            self.nbytes = count // per_block * block_bytes

    @property
    def shape(self):
        return self.ne[::-1]

    @property
    def row_bytes(self):
        _, per_block, block_bytes = TYPES[self.type]
        return (self.ne[0] if self.ne else 1) // per_block * block_bytes


class _Scan:
    """Forward-only decoder over the header bytes."""

    def __init__(self, view, label):
        self.view, self.at, self.label = view, 0, label

    def _span(self, n):
        lo, hi = self.at, self.at + n
        if n < 0 or hi > len(self.view):
            raise GgufError(f"{self.label}: the header ends inside a field at byte {lo}")
        self.at = hi
        return lo

    def u32(self):
        return _U32.unpack_from(self.view, self._span(4))[0]

    def u64(self):
        return _U64.unpack_from(self.view, self._span(8))[0]

    def text(self):
        n = self.u64()
        lo = self._span(n)
        return str(self.view[lo:lo + n], "utf-8", "replace")

    def scalars(self, kind, count):
        """`count` values of a fixed-size kind, decoded in one piece."""
        dt = np.dtype(_KIND_DTYPE[kind])
        lo = self._span(dt.itemsize * count)
        vals = np.frombuffer(self.view, dtype=dt, count=count, offset=lo)
        return vals.astype(bool) if kind == 7 else vals

    def value(self, kind, depth=0):
        if kind in _KIND_DTYPE:
            return self.scalars(kind, 1)[0].item()
        if kind == 8:
            return self.text()
        if kind == 9 and depth < 4:
            inner, count = self.u32(), self.u64()
            if count > len(self.view):                       # every item takes at least one byte
                raise GgufError(f"{self.label}: an array claims {count} items, more than the file has bytes")
            if inner in _KIND_DTYPE:
                return self.scalars(inner, count).tolist()
            return [self.value(inner, depth + 1) for _ in range(count)]
        raise GgufError(f"{self.label}: value kind {kind} is not part of the GGUF specification")


def _parse_header(view, label):
    """-> (version, pairs, tensor records in file order, offset of the data section)."""
    if len(view) < 24 or bytes(view[:4]) != b"GGUF":
        raise GgufError(f"{label}: the GGUF signature is missing")
    sc = _Scan(view, label)
    sc.at = 4
    version = sc.u32()
    if version not in (2, 3):
        raise GgufError(f"{label}: container version {version}; versions 2 and 3 (little endian) are understood")
    n_tensors, n_pairs = sc.u64(), sc.u64()
    if max(n_tensors, n_pairs) > _MAX_RECORDS:
        raise GgufError(f"{label}: {n_tensors} tensors / {n_pairs} pairs is beyond what a header can hold")
    pairs = {}
    for _ in range(n_pairs):
        key = sc.text()
        pairs[key] = sc.value(sc.u32())
    records = {}
    for _ in range(n_tensors):
        name, rank = sc.text(), sc.u32()
        if rank > _MAX_RANK:
            raise GgufError(f"{label}: {name} has rank {rank}")
        ne = tuple(sc.u64() for _ in range(rank))
        type_id, offset = sc.u32(), sc.u64()
        if name in records:
            raise GgufError(f"{label}: {name} is listed twice")
        records[name] = TensorInfo(name, ne, type_id, offset)
    align = pairs.get("general.alignment", 32)
    if not isinstance(align, int) or align < 1 or align & (align - 1):
        raise GgufError(f"{label}: general.alignment = {align!r} is not a power of two")
    data_start = -(-sc.at // align) * align
    for rec in records.values():
        if data_start + rec.offset + rec.nbytes > len(view):
            raise GgufError(f"{label}: {rec.name} needs bytes [{rec.offset}, {rec.offset + rec.nbytes}) of a data section that ends at {len(view) - data_start}")
    return version, pairs, records, data_start


class _Shard:
    """One file on disk: its memory map and parsed header."""

    def __init__(self, path):
        self.path = os.fspath(path)
        self.map = None
        with open(self.path, "rb") as fh:
            if os.fstat(fh.fileno()).st_size:
                self.map = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)       # the map outlives the descriptor
        try:
            self.version, self.kv, self.tensors, self.data_start = _parse_header(memoryview(self.map) if self.map is not None else memoryview(b""), self.path)
        except BaseException:
            self.release()
            raise

    def release(self):
        if self.map is not None:
            try:
                self.map.close()
            except BufferError:                               # arrays handed out by raw() still point into the map; it is unmapped when they go
                pass
            self.map = None

    def bytes_of(self, rec):
        return np.frombuffer(self.map, dtype=np.uint8, count=rec.nbytes, offset=self.data_start + rec.offset)


def _split_position(path):
    """(stem, index, total) of a gguf-split file name `<stem>-IIIII-of-TTTTT.gguf`, or None."""
    base = os.path.basename(path)
    if not base.endswith(".gguf"):
        return None
    parts = base[:-5].rsplit("-", 3)
    if len(parts) != 4 or parts[2] != "of" or not (len(parts[1]) == len(parts[3]) == 5 and parts[1].isdigit() and parts[3].isdigit()):
        return None
    return parts[0], int(parts[1]), int(parts[3])


class GgufFile:
    """One GGUF file or split set: `kv` (dict), `tensors` (name -> TensorInfo), `raw(name)` (uint8 view [rows.., row bytes]), `array(name)` for F32 / F16 / BF16 tensors."""

    def __init__(self, path):
        self.path = os.fspath(path)
        first = _Shard(self.path)
        self._shards = [first]
        self._home = {name: first for name in first.tensors}          # tensor name -> shard whose data section holds it
        self.version, self.kv, self.tensors, self.data_start = first.version, first.kv, dict(first.tensors), first.data_start
        try:
            total = int(self.kv.get("split.count") or 1)
            if total > 1:
                self._open_rest_of_set(total)
        except BaseException:
            self.close()
            raise

    def _open_rest_of_set(self, total):
        """The file announces a split set of `total` files: it has to be number 1 by key and by name; files 2..total are found beside it, checked and merged."""
        here = int(self.kv.get("split.no", 0))
        pos = _split_position(self.path)
        if here != 0:
            raise GgufError(f"{self.path} is part {here + 1} of a {total}-file set; a set is opened through its part 1")
        if pos is None or pos[1:] != (1, total):
            raise GgufError(f"{self.path} announces a {total}-file set, so its name has to end in -00001-of-{total:05d}.gguf")
        folder = os.path.dirname(os.path.abspath(self.path))
        present = {}
        for cand in glob.glob(os.path.join(glob.escape(folder), glob.escape(pos[0]) + "-*-of-*.gguf")):
            p = _split_position(cand)
            if p and p[0] == pos[0] and p[2] == total:
                present[p[1]] = cand
        absent = [i for i in range(2, total + 1) if i not in present]
        if absent:
            raise GgufError(f"{self.path}: parts {absent} of {total} were not found in {folder}; nothing is loaded from an incomplete set")
        for i in range(2, total + 1):
            part = _Shard(present[i])
            self._shards.append(part)
            if (part.kv.get("split.no"), part.kv.get("split.count")) != (i - 1, total):
                raise GgufError(f"{part.path} describes itself as part {part.kv.get('split.no')!r} of {part.kv.get('split.count')!r}, its name says {i - 1} of {total}")
            clash = self.tensors.keys() & part.tensors.keys()
            if clash:
                raise GgufError(f"{part.path} repeats tensors of an earlier part: {sorted(clash)[:3]}")
            self.tensors.update(part.tensors)
            self._home.update({name: part for name in part.tensors})
        declared = self.kv.get("split.tensors.count")
        if declared is not None and declared != len(self.tensors):
            raise GgufError(f"{self.path}: the set's parts list {len(self.tensors)} tensors, the first part promises {declared}")

    def close(self):
        for sh in self._shards:
            sh.release()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def raw(self, name) -> np.ndarray:
        """uint8 view of the tensor's bytes, shape [rows.., row_bytes] (zero copy)."""
        rec = self.tensors[name]
        if not rec.known:
            raise GgufTypeError(f"{name}: ggml type id {rec.type} has no entry in this reader's type table, so its size is unknown")
        flat = self._home[name].bytes_of(rec)
        return flat.reshape(rec.shape[:-1] + (rec.row_bytes,)) if rec.ne else flat

    def array(self, name) -> np.ndarray:
        """F32 / F16 / BF16 (as float32) / integer tensors as numpy arrays of their shape."""
        ti = self.tensors[name]
        dt = {"F32": "<f4", "F16": "<f2", "F64": "<f8", "I8": "i1", "I16": "<i2", "I32": "<i4", "I64": "<i8"}.get(ti.tname)
        flat = self.raw(name).reshape(-1)
        if dt is not None:
            return flat.view(dt).reshape(ti.shape)
        if ti.tname == "BF16":
            return (flat.view("<u2").astype(np.uint32) << 16).view(np.float32).reshape(ti.shape)
        raise GgufTypeError(f"tensor {name}: {ti.tname} is a block format; use load_pack / load_linear")

    # ---- quantized matrices -> packs / device modules
    def load_pack(self, name):
        """foreign_pack.Pack of a 2-D tensor [n, k] of a kernel format."""
        from . import foreign_pack as FP
        ti = self.tensors[name]
        if ti.tname not in KERNEL_TYPES:
            raise GgufTypeError(f"tensor {name}: {ti.tname} has no kernel in this package (kernel formats: {', '.join(KERNEL_TYPES)})")
        if len(ti.ne) != 2:
            raise GgufError(f"tensor {name}: {len(ti.ne)} dimensions; load_pack reads matrices, load_experts reads stacks")
        return FP.to_pack(ti.tname, np.array(self.raw(name)), ti.ne[0])        # a private, writable copy: the map may be closed afterwards

    def load_expert_packs(self, name):
        """List of E packs of a stacked expert tensor ne = [k, n, E] (expert e = rows [e n, (e + 1) n) of the flattened stack, kyojin_mlx/foreign_linear.py:2278-2280)."""
        from . import foreign_pack as FP
        ti = self.tensors[name]
        if ti.tname not in KERNEL_TYPES:
            raise GgufTypeError(f"tensor {name}: {ti.tname} has no kernel in this package")
        if len(ti.ne) != 3:
            raise GgufError(f"tensor {name}: an expert stack has three dimensions [k, n, E], got {ti.ne}")
        raw = self.raw(name)                                  # [E, n, row bytes]
        return [FP.to_pack(ti.tname, np.array(raw[e]), ti.ne[0]) for e in range(ti.ne[2])]

    def load_linear(self, name, bias=None, device="cuda"):
        """ForeignLinear on `device` for a matrix of a kernel format (y = x W^T, W = the stored [n, k])."""
        from .foreign_linear import make_linear
        return make_linear(self.load_pack(name), bias, device=device)

    def load_experts(self, name, device="cuda"):
        """DevPack of an expert stack (one resident T16 copy of all experts)."""
        from .foreign_linear import DevPack
        return DevPack(self.load_expert_packs(name), device)
