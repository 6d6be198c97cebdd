"""gigaslop_b200: B200 (sm_100a) implementation of gigaslop's quantized-GEMM hot path.

The product is ``libgigaslop_b200.so`` (hand-written CUDA, C ABI declared in
``include/gigaslop_b200/``); this package is the thin PyTorch-facing host layer.
"""
from ._lib import LIB_PATH, device_status, lib  # noqa: F401
from .ops import (  # noqa: F401
    quantize_tensor, fp8_quantize_per_token, gemm_i8_i32, gemm_i8, gemm_fp8, gemm_i8_rotary, quantize_gemm_i8_rotary,
    gemm_fp8_rotary, dual_gemm_i8_silu, dual_gemm_fp8_silu, mxfp8_quantize, dual_gemm_fp8_silu_mxfp8,
    gemm_f16, fp8_down_proj, fp8_factored_gemm, factored_lstm_step, mx_scales_to_tiled, gemm_mxfp8, dual_gemm_mxfp8_silu,
)

from .lstm import lstm_layer, lstm_scratch, lstm_stack  # noqa: F401,E402

__version__ = "0.1.0"
