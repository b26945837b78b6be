"""Regenerates the golden fixtures of this directory from the reference checkout.

Run once in a container that has the reference source tree (it is NOT needed to run the tests):
    python tests/golden/make_golden.py /path/to/reference
Writes
  kquant_ggml.npz  - the Q4_K / Q3_K / Q6_K / Q5_K / Q8_0 / Q2_K / IQ4_XS entries of the reference's tests/data/gguf_ggml_ref.npz
                     (raw blocks + ggml's own float32 dequantised values, llama.cpp pin recorded in `pin`)
  ref_dequant.npz  - seeded random blocks of Q4_K / Q3_K / Q6_K / NVFP4 / Q5_K / Q8_0 / Q2_K / IQ4_XS with the output of the reference
                     decoder kyojin_mlx.foreign_gguf.dequant, the reference's pack-form NVFP4 arrays
                     (foreign_gguf.to_pack) and kyojin_mlx.foreign_pack.dequant of them with a gscale.
"""
import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from kyojin_mlx import foreign_gguf as GF, foreign_pack as FP, foreign_synth as SY
    here = os.path.dirname(os.path.abspath(__file__))

    src = np.load(os.path.join(ref_root, "tests", "data", "gguf_ggml_ref.npz"))
    keep = {"pin": src["pin"]}
    for t in ("Q4_K", "Q3_K", "Q6_K", "Q5_K", "Q8_0", "Q2_K", "IQ4_XS"):
        keep[t + "_raw"], keep[t + "_ref"] = src[t + "_raw"], src[t + "_ref"]
    np.savez_compressed(os.path.join(here, "kquant_ggml.npz"), **keep)

    out = {}
    for i, (t, n, k) in enumerate((("Q4_K", 6, 512), ("Q3_K", 6, 512), ("Q6_K", 6, 512), ("NVFP4", 6, 256), ("Q5_K", 6, 512), ("Q8_0", 6, 512), ("Q2_K", 6, 512), ("IQ4_XS", 6, 512))):
        rng = np.random.default_rng(100 + i)
        raw = SY.random_blocks(t, n, k, rng)
        if t == "NVFP4":                                   # also the scale codes the decoder special-cases
            raw = raw.copy()
            blk = raw.reshape(n, k // 64, 36)
            blk[0, 0, 0:4] = (0x00, 0x7F, 0x01, 0x7E)      # zero, NaN code (-> 0), smallest subnormal, largest finite
            blk[1, 0, 0:4] = (0x07, 0x08, 0x80, 0xFF)      # largest subnormal, smallest normal, signed codes
        out[t + "_raw"], out[t + "_k"] = raw, np.int64(k)
        out[t + "_f32"] = GF.dequant(t, raw, k)
        # BASELINE-style scales: d, dmin = fp16(|N(0, 1e-3)|)
        if t != "NVFP4":
            raw2 = rng.integers(0, 256, raw.shape, dtype=np.uint8).reshape(n, k // 256, -1)
            SY.set_scales(t, raw2, np.abs(rng.normal(0.0, 1e-3, (n, k // 256))))
            raw2 = raw2.reshape(n, -1)
            out[t + "_raw_small"] = raw2
            out[t + "_f32_small"] = GF.dequant(t, raw2, k)
    p = GF.to_pack("NVFP4", out["NVFP4_raw"], int(out["NVFP4_k"]))
    out["NVFP4_pack_qs"], out["NVFP4_pack_meta"] = p.qs, p.meta
    p.gscale = np.float32(0.0123)
    out["NVFP4_pack_gscale"] = np.float32(p.gscale)
    out["NVFP4_pack_f32"] = FP.dequant(p)
    out["NVFP4_pack_f32_nog"] = FP.dequant(p, g=False)
    np.savez_compressed(os.path.join(here, "ref_dequant.npz"), **out)
    print("wrote", sorted(out))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KYOJIN_REFERENCE", "."))
