"""The CPU implementation that the benchmark times beside the GPU path - TEST / BENCHMARK INFRASTRUCTURE, never imported by the package.

When the reference package is installed beside the repository (`baseline/_ref`, the offline `pip install --target` of the reference; it is git-ignored and
travels to the GPU box with the working tree) or is reachable through $KYOJIN_REF, its own numpy dequantiser `kyojin_mlx.foreign_gguf.dequant`
(kyojin_mlx/foreign_gguf.py:376-394) is what runs: kind "reference". Otherwise the numpy restatement of this directory runs: kind "port" (it is bit-equal to the
reference decoder on the golden vectors, so the arithmetic timed is the same)."""
from __future__ import annotations

import os
import sys

import numpy as np

from . import kq_numpy as O

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_dequant():
    """(dequant(tname, raw, k) -> float32 [n, k], kind, description)."""
    for cand in (os.environ.get("KYOJIN_REF"), os.path.join(_ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "kyojin_mlx")):
            if cand not in sys.path:
                sys.path.insert(0, cand)
            try:
                from kyojin_mlx import foreign_gguf as G
                return G.dequant, "reference", f"kyojin_mlx.foreign_gguf.dequant of the reference package under {os.path.relpath(cand, _ROOT)}"
            except Exception:                                # noqa: BLE001 - an unusable install falls back to the port
                pass
    return (lambda tname, raw, k: O.dequant(tname, raw, k)), "port", "numpy restatement oracle/kq_numpy.py of the reference's CPU decoder"


def linear_cpu():
    """(linear(tname, raw, k, x) -> float32 [m, n], kind, description): the reference's large-row CPU path, dequantise per call then x @ W.T in float32
    (kyojin_mlx/foreign_linear.py:710)."""
    deq, kind, impl = reference_dequant()

    def linear(tname, raw, k, x):
        return np.asarray(x).astype(np.float32) @ deq(tname, raw, k).T

    return linear, kind, impl
