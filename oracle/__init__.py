"""CPU oracle for the quantized-GEMM hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, in plain PyTorch-on-CPU, the
host-side reference math that the gigaslop kernels are checked against.  It is
imported by the test-suite, by the smoke check and by the CPU-baseline leg of
the benchmark; the product package never imports it and has no CPU fallback.

Every function cites the reference file:line it follows (paths are relative to
the reference project root).  Pinning status:

* INT8 quantiser, int32 GEMM, dequant GEMM, rotary, SwiGLU, FP8 quantisers,
  FP8 GEMM, factored GEMM and the factored LSTM step are pinned by golden
  vectors produced by running the reference's own functions
  (``tests/golden/make_golden.py``).
* MXFP8 block scaling and the full-rank sigmoid/tanh LSTM have no reference
  implementation (kernel source absent / semantics only described in prose):
  **parity unpinned** for those two.
"""
from .quant import (  # noqa: F401
    quantize_tensor, quantize_per_row_cpp, fp8_quantize_per_token,
    fp8_quantize_per_token_kernel, fp8_quantize_per_channel, fp8_quantize_scalar,
    e4m3_encode, e4m3_decode,
)
from .gemm import (  # noqa: F401
    gemm_i32, gemm_dequant_ref, gemm_dequant_exact, rotary_ref, rotary_exact,
    dual_gemm_silu_ref, dual_gemm_silu_model, naive_fp8_gemm_ref,
    fp8_gemm_f16_ref, fp8_gemm_model, fp8_rotary_ref, fp8_dual_silu_ref,
    rope_tables,
)
from .mx import (  # noqa: F401
    mx_block_quantize, mx_dequantize, mx_dual_silu_ref, mx_gemm_ref, e8m0_decode,
)
from .lstm import (  # noqa: F401
    factored_gemm_ref, down_proj_ref, factored_lstm_step_ref,
    lstm_fullrank_step_ref, lstm_fullrank_recurrent_ref, lstm_fullrank_layer_ref, lstm_fullrank_stack_ref,
)
