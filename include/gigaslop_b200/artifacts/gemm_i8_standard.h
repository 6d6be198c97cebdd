/* Drop-in for the reference's exported `gemm_i8_standard.h` (prefix gemm_i8_std, cute/export_gemm_i8.py:16-28):
 * W8A8 GEMM with per-token x per-channel dequant to fp16. */
#pragma once
#define GSB200_STD_PREFIX gemm_i8_std
#include "gemm_i8_std_template.h"
