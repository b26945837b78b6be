"""GGUF file reader -> packs for the device kernels: the role of kyojin_mlx/foreign_gguf.py `GgufFile` (:186-308) and of the loader half of
kyojin_mlx/foreign_linear.py `_read_gguf` (:2240-2328), for the formats this package has kernels for (Q4_K, Q3_K, Q6_K, NVFP4; F32 / F16 / BF16 tensors are returned
as arrays). The container format is the public GGUF layout (little endian, versions 2 and 3): magic, version, tensor count, key count, typed key / value pairs,
tensor infos (name, dimensions with the fastest first, ggml type id, offset), then the data section aligned to `general.alignment` (default 32).
Tensor bytes are memory-mapped (zero copy); `load_linear` / `load_experts` hand them to foreign_pack.to_pack and the T16 repack on the device.
A split shard set (gguf-split: <name>-00001-of-0000N.gguf ...) opened through its FIRST shard reads as one logical file: key / value pairs of shard 1, the tensors
of every shard, bytes mapped from the shard that holds the tensor; any gap in the set is an error, never a partial load (kyojin_mlx/foreign_gguf.py:247-285).
Not built: the two layouts of type id 43 (that id is not in the type table here, so such tensors are refused by name)."""
from __future__ import annotations

import mmap
import os
import re
import struct

import numpy as np

MAGIC = b"GGUF"
ALIGN_DEFAULT = 32

# ggml type id -> (name, block elements, block bytes): the public ggml type table (sizes are needed to size every tensor of a file, also the ones without a kernel here)
TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36),
    10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
    16: ("IQ2_XXS", 256, 66), 17: ("IQ2_XS", 256, 74), 18: ("IQ3_XXS", 256, 98), 19: ("IQ1_S", 256, 50), 20: ("IQ4_NL", 32, 18), 21: ("IQ3_S", 256, 110),
    22: ("IQ2_S", 256, 82), 23: ("IQ4_XS", 256, 136), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
    29: ("IQ1_M", 256, 56), 30: ("BF16", 1, 2), 34: ("TQ1_0", 256, 54), 35: ("TQ2_0", 256, 66), 39: ("MXFP4", 32, 17), 40: ("NVFP4", 64, 36),
}
KERNEL_TYPES = ("Q4_K", "Q3_K", "Q6_K", "NVFP4")          # stored formats the CUDA kernels read (after the lossless T16 repack)


_SHARD_NAME = re.compile(r"^(.*)-(\d{5})-of-(\d{5})\.gguf$")


class GgufError(ValueError):
    pass


class GgufTypeError(GgufError):
    pass


class TensorInfo:
    """name, ne (fastest dimension first, as stored), ggml type id / name, offset in the data section, byte count; shape = ne reversed (rows first)."""
    __slots__ = ("name", "ne", "type", "offset", "nbytes", "tname", "known")

    def __init__(self, name, ne, type_, offset):
        self.name, self.ne, self.type, self.offset = name, tuple(int(d) for d in ne), int(type_), int(offset)
        self.known = self.type in TYPES
        if not self.known:                                  # the file stays readable; reading THIS tensor fails
            self.tname, self.nbytes = f"ID{self.type}", 0
            return
        self.tname, be, bb = TYPES[self.type]
        n = int(np.prod(self.ne, dtype=np.int64)) if self.ne else 1
        if n % be or (self.ne and self.ne[0] % be):
            raise GgufError(f"tensor {name}: row length {self.ne[0] if self.ne else n} is not a multiple of the {self.tname} block of {be}")
        self.nbytes = n // be * bb

    @property
    def shape(self):
        return tuple(reversed(self.ne))


class _Cursor:
    def __init__(self, buf, pos):
        self.b, self.p = buf, pos

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.p + size > len(self.b):
            raise GgufError("truncated header")
        v = struct.unpack_from(fmt, self.b, self.p)[0]
        self.p += size
        return v

    def string(self):
        n = self.take("<Q")
        if n > 1 << 30 or self.p + n > len(self.b):
            raise GgufError("implausible string length in the header")
        s = bytes(self.b[self.p:self.p + n]).decode("utf-8", errors="replace")
        self.p += n
        return s

    _SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}

    def value(self, t):
        if t in self._SCALAR:
            return self.take(self._SCALAR[t])
        if t == 7:
            return bool(self.take("<B"))
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            if n > 1 << 28:
                raise GgufError("implausible array length in the header")
            return [self.value(et) for _ in range(n)]
        raise GgufError(f"unknown key / value type {t}")


class GgufFile:
    """One GGUF file: `kv` (dict), `tensors` (name -> TensorInfo), `raw(name)` (uint8 view [rows.., row bytes]), `array(name)` for F32 / F16 / BF16 tensors."""

    def __init__(self, path, _member=False):
        self.path = str(path)
        self._owner, self._members = {}, []                  # tensor name -> shard that holds it (split sets); the other shards
        self._f = open(self.path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        if size < 24 or self._mm[:4] != MAGIC:
            self.close()
            raise GgufError(f"{path}: not a GGUF file")
        c = _Cursor(memoryview(self._mm), 4)
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"{path}: GGUF version {self.version} (this reader: 2 and 3, little endian)")
        nt, nkv = c.take("<Q"), c.take("<Q")
        if nt > 1 << 22 or nkv > 1 << 22:
            raise GgufError("implausible tensor / key count")
        self.kv = {}
        for _ in range(nkv):
            k = c.string()
            self.kv[k] = c.value(c.take("<I"))
        self.tensors = {}
        for _ in range(nt):
            name = c.string()
            nd = c.take("<I")
            if nd > 8:
                raise GgufError(f"tensor {name}: {nd} dimensions")
            ne = [c.take("<Q") for _ in range(nd)]
            t, off = c.take("<I"), c.take("<Q")
            if name in self.tensors:
                raise GgufError(f"duplicate tensor {name}")
            self.tensors[name] = TensorInfo(name, ne, t, off)
        al = int(self.kv.get("general.alignment", ALIGN_DEFAULT))
        if al <= 0 or al & (al - 1):
            raise GgufError(f"general.alignment {al}")
        self.data_start = (c.p + al - 1) // al * al
        for ti in self.tensors.values():
            if self.data_start + ti.offset + ti.nbytes > size:
                raise GgufError(f"tensor {ti.name}: data past the end of the file")
        if not _member and int(self.kv.get("split.count", 1) or 1) > 1:
            self._attach_shards()

    def _attach_shards(self):
        """This file is shard 1 of a split set: open and check the others (count, numbering, no duplicate tensor, tensor total)."""
        n, no = int(self.kv["split.count"]), int(self.kv.get("split.no", 0))
        m = _SHARD_NAME.match(os.path.basename(self.path))
        if no != 0:
            raise GgufError(f"{self.path}: shard split.no={no} of {n}: open the FIRST shard (-00001-of-{n:05d}.gguf)")
        if not m or int(m.group(2)) != 1 or int(m.group(3)) != n:
            raise GgufError(f"{self.path}: split.count={n} but the file name is not <name>-00001-of-{n:05d}.gguf")
        folder, base = os.path.dirname(os.path.realpath(self.path)), m.group(1)
        members = [self]
        try:
            for i in range(2, n + 1):
                f = os.path.join(folder, f"{base}-{i:05d}-of-{n:05d}.gguf")
                if not os.path.isfile(f):
                    raise GgufError(f"{self.path}: shard {i} of {n} is missing ({os.path.basename(f)})")
                s = GgufFile(f, _member=True)
                members.append(s)
                if int(s.kv.get("split.count", 0) or 0) != n or int(s.kv.get("split.no", -1)) != i - 1:
                    raise GgufError(f"{f}: split.no={s.kv.get('split.no')} split.count={s.kv.get('split.count')}, expected {i - 1} / {n}")
            for s in members:
                for name, ti in s.tensors.items():
                    if s is not self:
                        if name in self.tensors:
                            raise GgufError(f"duplicate tensor {name} across shards ({os.path.basename(s.path)})")
                        self.tensors[name] = ti
                    self._owner[name] = s
            want = self.kv.get("split.tensors.count")
            if want is not None and int(want) != len(self.tensors):
                raise GgufError(f"{self.path}: shard set holds {len(self.tensors)} tensors, split.tensors.count says {want}")
        except BaseException:
            for s in members[1:]:
                s.close()
            raise
        self._members = members[1:]

    def close(self):
        for s in self._members:
            s.close()
        self._members = []
        mm, self._mm = self._mm, None
        try:
            if mm is not None:
                mm.close()
        except BufferError:                                  # views handed out by raw() are still alive: the map goes with them
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def raw(self, name) -> np.ndarray:
        """uint8 view of the tensor's bytes, shape [rows.., row_bytes] (zero copy)."""
        ti = self.tensors[name]
        if not ti.known:
            raise GgufTypeError(f"tensor {name}: ggml type id {ti.type} is not in the type table of this reader")
        _, be, bb = TYPES[ti.type]
        src = self._owner.get(name, self)
        a = np.frombuffer(src._mm, dtype=np.uint8, count=ti.nbytes, offset=src.data_start + ti.offset)
        return a.reshape(ti.shape[:-1] + (ti.ne[0] // be * bb,)) if ti.ne else a

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
