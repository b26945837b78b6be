"""numpy restatement of the routed-expert layer around the quantized products (TEST INFRASTRUCTURE, see oracle/__init__.py).

Parity unpinned: the reference implements these steps as Metal kernels / MLX ops (kyojin_mlx/foreign_moe.py:77-119, foreign_linear.py:1353-1361,
foreign_kqgmm.py:169-196, moe_sort.py) that cannot run here; this file restates their arithmetic and the tests check it against independent
fp64 formulations (argsort of an fp64 softmax, bincount plans) the way the reference's own tests do (tests/test_foreign_moe.py:95-118,
tests/test_moe_sort.py:13-23)."""
from __future__ import annotations

import numpy as np

from .kq_numpy import sat_f16


def select(logits, K: int, norm: bool = True, E: int | None = None):
    """fp32 softmax over the first E columns, K rounds of arg-max (value descending, lowest index on ties), weights top / sum(top) when norm;
    sgs = sigmoid of column E when present. (kyojin_mlx/foreign_moe.py:77-104)"""
    L = np.asarray(logits, np.float32)
    E = L.shape[1] if E is None else E
    p = L[:, :E] - L[:, :E].max(-1, keepdims=True)
    p = np.exp(p).astype(np.float32)
    p = (p * (np.float32(1.0) / p.sum(-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    T = L.shape[0]
    inds = np.zeros((T, K), np.uint32)
    top = np.zeros((T, K), np.float32)
    q = p.copy()
    for k in range(K):
        i = q.argmax(-1)                                   # first maximum = lowest index on ties
        inds[:, k] = i
        top[:, k] = q[np.arange(T), i]
        q[np.arange(T), i] = -1.0
    ts = np.zeros(T, np.float32)
    for k in range(K):
        ts = (ts + top[:, k]).astype(np.float32)
    scs = (top / ts[:, None]).astype(np.float32) if norm else top
    sgs = (1.0 / (1.0 + np.exp(-L[:, E].astype(np.float32)))).astype(np.float32) if L.shape[1] > E else None
    return inds.reshape(-1), scs.reshape(-1), sgs


def glu(a, b, limit=None):
    """fp16(silu(f32 a) * f32 b), optional clamp (kyojin_mlx/foreign_linear.py:1353-1361)."""
    a, b = np.asarray(a).astype(np.float32), np.asarray(b).astype(np.float32)
    if limit is not None:
        a, b = np.minimum(a, np.float32(limit)), np.clip(b, -np.float32(limit), np.float32(limit))
    return sat_f16(a * (np.float32(1.0) / (np.float32(1.0) + np.exp(-a))) * b)


def combine(y, scs, K: int, sgs=None, shared=None, out16=True):
    """sum_k f32(y[t K + k]) * scs[t K + k] (+ sgs[t] * shared[t]) (kyojin_mlx/foreign_moe.py:112-119)."""
    y = np.asarray(y).astype(np.float32)
    S, H = y.shape
    acc = np.zeros((S // K, H), np.float32)
    w = np.asarray(scs, np.float32).reshape(S // K, K)
    for k in range(K):
        acc = acc + y.reshape(S // K, K, H)[:, k] * w[:, k:k + 1]
    if shared is not None:
        acc = acc + np.asarray(sgs, np.float32)[:, None] * np.asarray(shared).astype(np.float32)
    return sat_f16(acc) if out16 else acc.astype(np.float32)


def host_plan(ids, E: int, mt: int):
    """Expert segment starts and tile starts of a slot list (numpy bincount plan, tests/test_moe_sort.py:13-23)."""
    cnt = np.bincount(np.asarray(ids).reshape(-1), minlength=E)
    off = np.concatenate([[0], np.cumsum(cnt)]).astype(np.uint32)
    tb = np.concatenate([[0], np.cumsum((cnt + mt - 1) // mt)]).astype(np.uint32)
    return cnt, off, tb


def routed_layer(x, inds, Wg, Wu, Wd, K: int, ref_path: bool, limit=None):
    """Unweighted per-slot outputs [T*K, H] of a routed SwiGLU layer from dequantised expert weights W* [E, n, k].
    ref_path False: fp64 throughout, no intermediate rounding (the accuracy reference). True: the reference's rounding points (fp16 a, b, h, y with
    fp32 accumulation: gate / up products rounded to fp16, the gated activation rounded to fp16, the down product rounded to fp16; kyojin_mlx/foreign_linear.py:1353-1361, :1448)."""
    x = np.asarray(x)
    T = x.shape[0]
    e = np.asarray(inds).reshape(T, K)
    dt = np.float32 if ref_path else np.float64
    out = np.zeros((T * K, Wd.shape[1]), np.float16 if ref_path else np.float64)
    for ex in np.unique(e):
        t, k = np.nonzero(e == ex)
        xs = x[t].astype(dt)
        wg, wu, wd = (W[ex].astype(np.float16).astype(dt) if ref_path else W[ex].astype(dt) for W in (Wg, Wu, Wd))
        a, b = xs @ wg.T, xs @ wu.T
        if ref_path:
            h = glu(sat_f16(a), sat_f16(b), limit).astype(dt)
            y = sat_f16(h @ wd.T)
        else:
            if limit is not None:
                a, b = np.minimum(a, limit), np.clip(b, -limit, limit)
            h = a / (1.0 + np.exp(-a)) * b
            y = h @ wd.T
        out[t * K + k] = y
    return out
