"""kairos_engine_b200 — the Gemma-4-26B-A4B MoE feed-forward hot path of kairos-engine as
hand-written sm_100a CUDA behind a C ABI (include/sp_engine/moe_backend.h). CUDA only."""
from .engine import (FLAVOUR_DECODE, FLAVOUR_PREFILL, GEMMA4_26B_A4B, MoeEngine, MoeExt, gelu_mul, gemv_q4b,
                     q4b_dequantize, q4b_quantize)
from ._lib import SpMoeError

__all__ = ["MoeEngine", "MoeExt", "SpMoeError", "FLAVOUR_DECODE", "FLAVOUR_PREFILL", "GEMMA4_26B_A4B",
           "q4b_quantize", "q4b_dequantize", "gelu_mul", "gemv_q4b"]
