"""CPU oracle of the dequant-fused quantized linear (TEST INFRASTRUCTURE, not product code).

Everything under this directory restates, in numpy, the arithmetic of the reference's CPU
implementation (kyojin_mlx/foreign_gguf.py, foreign_pack.py, fp4pack.py, fp4tile.py,
foreign_moe.py, foreign_kqgmm.py). It exists to CHECK the CUDA kernels and to provide the
timed CPU baseline of the benchmark. Only the test suite, the smoke check and the benchmark's
CPU legs may import it; the shipped package never does and has no CPU fallback.

Parity pins:
  * K-quant decoders (Q4_K, Q3_K, Q6_K): pinned bit-for-bit on ggml's own dequantised output
    (the reference's tests/data/gguf_ggml_ref.npz, llama.cpp pin 29c720ea, re-exported as
    tests/golden/kquant_ggml.npz) and on outputs of the reference decoder run on seeded random
    blocks (tests/golden/ref_dequant.npz, written by tests/golden/make_golden.py).
  * NVFP4 (GGUF blocks and the qs/meta/gscale pack): pinned on outputs of the reference decoders
    (same fixture file); the reference holds no ggml golden vector for this type.
  * fp4pack.pack / router select / glu / combine / slot plan: the reference implements these with
    MLX array ops that cannot run without MLX, so the restatements are "parity unpinned": checked
    only through their algebraic properties and against independent fp64 formulations.
"""
