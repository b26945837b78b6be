"""kyojin_mac_b200: the dequant-fused quantized linear of kyojin-mac (GGUF K-quants + NVFP4) for NVIDIA B200 (sm_100a).

Host code is Python/PyTorch over a C-ABI CUDA library (kyojin_mac_b200/csrc, declared in include/kyb.h). There is no CPU
fallback: every operator raises if the CUDA library is missing."""
__version__ = "0.1.0"
