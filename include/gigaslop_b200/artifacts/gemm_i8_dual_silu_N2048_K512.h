/* Drop-in for the reference's exported `gemm_i8_dual_silu_N2048_K512.h` (cute/export_dual_gemm_i8_silu.py:53-63). */
#pragma once
#define GSB200_DUAL_PREFIX gemm_i8_dual_silu_N2048_K512
#include "gemm_i8_dual_silu_template.h"
