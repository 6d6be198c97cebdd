/* Drop-in for the reference's exported `gemm_i8_rotary_N1536_K512_H8D64R64S2048.h`
 * (cute/export_configs/gemm_i8_rotary.toml; consumer: cute/main_rotary.cpp:28-30). */
#pragma once
#define GSB200_ROT_PREFIX gemm_i8_rotary_N1536_K512_H8D64R64S2048
#define GSB200_ROT_NHEAD 8
#define GSB200_ROT_HEAD_DIM 64
#define GSB200_ROT_ROTARY_DIM 64
#define GSB200_ROT_SEQ_TABLE 2048
#include "gemm_i8_rotary_template.h"
