"""Loader and ctypes signatures of libkyb.so, the C-ABI CUDA library (include/kyb.h).

The library is built in-tree (kyojin_mac_b200/libkyb.so) by `build()` with nvcc for sm_100a. There is no fallback: if the
library cannot be loaded every operator raises KybUnavailable."""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO_PATH = os.path.join(HERE, "libkyb.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]

OK, EINVAL, ECUDA, ETIMEOUT, EUNSUPPORTED, EWORKSPACE = 0, -1, -2, -3, -4, -5


class KybError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"kyb status {status}: {msg}")
        self.status = status


class KybUnavailable(RuntimeError):
    pass


def _nvcc() -> str:
    for p in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc"):
        if p and os.path.exists(p):
            return p
    return "nvcc"


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers() -> list[str]:
    return glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(os.path.dirname(HERE), "include", "kyb.h")]


def _stale() -> bool:
    if not os.path.exists(SO_PATH):
        return True
    t = os.path.getmtime(SO_PATH)
    return any(os.path.getmtime(d) > t for d in sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu under csrc/ for sm_100a (cross-compiles without a GPU) and links libkyb.so.

    One object per source under kyojin_mac_b200/build/, compiled in parallel; an object is rebuilt when its source or any
    header is newer."""
    if not force and not _stale():
        return SO_PATH
    from concurrent.futures import ThreadPoolExecutor
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    hdr_t = max(os.path.getmtime(h) for h in _headers())
    flags = [f for f in NVCC_FLAGS if f != "-shared"]
    jobs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [_nvcc()] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", obj, src]
        return src, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 4))) as pool:
        for src, r in pool.map(compile_one, jobs):
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n" + r.stdout + r.stderr)
            if verbose:
                print(r.stderr)
    objs = [os.path.join(objdir, os.path.basename(s)[:-3] + ".o") for s in sources()]
    r = subprocess.run([_nvcc(), "-shared", "-o", SO_PATH + ".tmp"] + objs + ["-lcuda"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    os.replace(SO_PATH + ".tmp", SO_PATH)
    return SO_PATH


_lock = threading.Lock()
_lib = None

_vp, _i64, _sz, _int, _f32 = C.c_void_p, C.c_int64, C.c_size_t, C.c_int, C.c_float


class PeerOut(C.Structure):
    """kyb_peer_out: base address of the output matrix on every rank (peer-mapped), and the rank count."""
    _fields_ = [("ptr", C.c_void_p * 8), ("count", C.c_int)]

    @classmethod
    def of(cls, ptrs):
        if not 1 <= len(ptrs) <= 8:
            raise ValueError("1..8 peer outputs")
        o = cls()
        for i, p in enumerate(ptrs):
            o.ptr[i] = int(p)
        o.count = len(ptrs)
        return o


_pp = C.POINTER(PeerOut)
SIGNATURES = {
    "kyb_version": (_int, []),
    "kyb_status_string": (C.c_char_p, [_int]),
    "kyb_last_error": (C.c_char_p, []),
    "kyb_t16_nbytes": (_sz, [_int, _i64, _i64]),
    "kyb_raw_row_bytes": (_sz, [_int, _i64]),
    "kyb_repack_raw_to_t16": (_int, [_int, _vp, _i64, _i64, _vp, _vp]),
    "kyb_repack_t16_to_raw": (_int, [_int, _vp, _i64, _i64, _vp, _vp]),
    "kyb_dequant_t16": (_int, [_int, _vp, _i64, _i64, _i64, _i64, _f32, _int, _vp, _i64, _vp]),
    "kyb_gemv_workspace_bytes": (_sz, [_int, _i64, _i64, _i64]),
    "kyb_gemv_t16": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _vp, _sz, _int, _vp]),
    "kyb_gemv_glu_t16": (_int, [_int, _vp, _i64, _i64, _vp, _vp, _f32, _i64, _i64, _f32, _vp, _i64, _vp, _sz, _int, _vp]),
    "kyb_gemv_chunks": (_int, [_i64, _i64]),
    "kyb_gemv_partial_t16": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp]),
    "kyb_gemv_finalize": (_int, [_vp, _int, _i64, _i64, _f32, _vp, _i64, _vp]),
    "kyb_gemm_kq": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _int, _vp]),
    "kyb_gemm_kq_split": (_int, [_int, _i64, _i64, _i64]),
    "kyb_gemm_kq_split_bytes": (C.c_size_t, [_i64, _i64, _int]),
    "kyb_gemm_kq_splitk": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _int, _vp, C.c_size_t, _vp]),
    "kyb_gemm_kq_ag": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _f32, _pp, _i64, _i64, _int, _vp]),
    "kyb_gemm_nvfp4_ag": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _pp, _i64, _i64, _vp]),
    "kyb_gemm_kq_grouped": (_int, [_int, _vp, _i64, _i64, _int, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _int, _vp]),
    "kyb_gemm_kq_grouped_glu": (_int, [_int, _vp, _vp, _i64, _i64, _int, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _f32, _vp, _i64, _int, _vp]),
    "kyb_dequant_rows_t16": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _f32, _int, _vp, _i64, _vp]),
    "kyb_router_rpad": (_i64, [_int, _int]),
    "kyb_router_split": (_int, [_vp, _vp, _int, _i64, _vp, _vp, _vp]),
    "kyb_router_logits_tc": (_int, [_vp, _i64, _vp, _vp, _i64, _int, _int, _i64, _vp, _vp, _i64, _vp]),
    "kyb_gemm_f16_tn_f32": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _f32, _vp, _i64, _vp]),
    "kyb_router_logits": (_int, [_vp, _int, _i64, _vp, _vp, _i64, _int, _i64, _vp, _i64, _vp]),
    "kyb_gather_flat": (_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int64), _int, _vp]),
    "kyb_q4mma": (_int, [_vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp]),
    "kyb_gemv_t16_static": (_int, [_int, _vp, _i64, _i64, _vp, _i64, _i64, _f32, _vp, _i64, _int, _vp]),
    "kyb_gemm_f16_tn": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _f32, _vp, _i64, _vp]),
    "kyb_gemm_f16_grouped": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "kyb_nvfp4_sf_bytes": (_sz, [_i64, _i64]),
    "kyb_nvfp4_quant_rows": (_int, [_vp, _int, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "kyb_nvfp4_unpack_rows": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _i64, _vp]),
    "kyb_fp4_quant_block32": (_int, [_vp, _int, _i64, _i64, _i64, _vp, _vp, _vp]),
    "kyb_fp4_unpack_block32": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _i64, _vp]),
    "kyb_nvfp4_sf_swizzle": (_int, [_vp, _i64, _i64, _vp, _int, _vp]),
    "kyb_gemm_nvfp4": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp, _i64, _vp]),
    "kyb_moe_select": (_int, [_vp, _i64, _i64, _int, _int, _int, _int, _vp, _vp, _vp, _vp]),
    "kyb_moe_plan": (_int, [_vp, _vp, _vp, _int, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "kyb_gather_rows": (_int, [_vp, _i64, _i64, _vp, _int, _vp, _i64, _i64, _vp, _i64, _vp]),
    "kyb_silu_mul": (_int, [_vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp, _i64, _vp]),
    "kyb_moe_combine": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _int, _i64, _int, _vp, _i64, _vp]),
    "kyb_moe_groups": (_int, [_vp, _i64, _int, _vp, _vp, _vp, _vp]),
    "kyb_gemv_group_t16": (_int, [_int, _vp, _vp, _i64, _i64, _int, _vp, _vp, _f32, _i64, _vp, _vp, _int, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp]),
    "kyb_gemv_plan": (_int, [_int, _i64, _i64, _i64, C.POINTER(C.c_int)]),
    "kyb_check_device_status": (_int, [_vp]),
    "kyb_selftest_wait_timeout": (_int, [_int, _vp]),
}


def lib():
    """The loaded library (ctypes.CDLL with typed entry points). Raises KybUnavailable when it is missing: no CPU path exists."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(SO_PATH):
                raise KybUnavailable(f"{SO_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                                     "(kyojin_mac_b200 has no CPU fallback)")
            try:
                h = C.CDLL(SO_PATH)
            except OSError as e:
                raise KybUnavailable(f"cannot load {SO_PATH}: {e}") from e
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(h, name)
                fn.restype, fn.argtypes = res, args
            _lib = h
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise KybError(status, lib().kyb_last_error().decode("utf-8", "replace") or lib().kyb_status_string(status).decode())
