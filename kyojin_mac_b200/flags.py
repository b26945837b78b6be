"""Dispatch thresholds of the quantized linear (role of the row-count constants of kyojin_mlx/foreign_linear.py:38-94), each
overridable through the environment at import time. There is no backend switch: every path is sm_100a CUDA."""
import os


def _int(name: str, default: int) -> int:
    v = os.environ.get(name, "")
    return int(v) if v else default


GEMV_ROWS = _int("KYB_GEMV_ROWS", 32)        # rows served by the decode GEMV / few-row tensor-core kernel (one weight read per 32 rows)
GEMM_MIN_ROWS = _int("KYB_GEMM_MIN_ROWS", 64)  # from here the prefill GEMM (tcgen05) runs
GATHER_MAX = _int("KYB_GATHER_MAX", 256)     # routed-expert slots up to here take the gathered GEMV path (reference: 128, foreign_linear.py:87)
GATHER_PER_EXPERT = _int("KYB_GATHER_PER_EXPERT", 4)   # ... or up to this many slots per expert of the stack: with election an expert's bytes are read once per 8 of its slots, so a decode batch that spreads over many experts (64 tokens x top-8 over 256 experts) stays bandwidth-bound on the bytes it touches
PREFILL_TWO_STEP = _int("KYB_PREFILL_TWO_STEP", 0) != 0   # 1: prefill = fp16 copy of the weights in HBM, then the fp16 GEMM (the reference's form); 0: weights decoded inside the GEMM
GEMV_CHAINED = _int("KYB_GEMV_CHAINED", 1) != 0   # decode products of a module are launched with programmatic stream serialization from their second call on (the weights are settled by then): consecutive products overlap launch and pipeline fill
ROUTER_TC_MIN_ROWS = _int("KYB_ROUTER_TC_MIN_ROWS", 512)   # fp16 token batches from this size compute the router logits on the tensor cores (gate cut into three fp16 pieces); below it the fp32 kernels run
GEMM_SPLIT_K = _int("KYB_GEMM_SPLIT_K", 1) != 0   # prefill products with fewer 256 x 256 output tiles than SMs cut k into ranges (fp32 partial sums in a workspace, added in k order); 0: never
