/* Drop-in for the reference's exported `gemm_i8_dual_silu_N2048_K512.h` (cute/export_dual_gemm_i8_silu.py:53-63).
 * Wrapper arguments = the kernel's __call__: mA, mB_gate, mB_up, mC, mScaleA, mScaleB_gate, mScaleB_up
 * (cute/ampere_dual_gemm_i8_silu.py:52-61,469-471). */
#pragma once
#include "../cute_dsl_abi.h"

GSB200_DECL_MODULE_(gemm_i8_dual_silu_N2048_K512)
GSB200_DECL_STRIDED_(gemm_i8_dual_silu_N2048_K512, mA)
GSB200_DECL_STRIDED_(gemm_i8_dual_silu_N2048_K512, mB_gate)
GSB200_DECL_STRIDED_(gemm_i8_dual_silu_N2048_K512, mB_up)
GSB200_DECL_STRIDED_(gemm_i8_dual_silu_N2048_K512, mC)
GSB200_DECL_POINTER_(gemm_i8_dual_silu_N2048_K512, mScaleA)
GSB200_DECL_POINTER_(gemm_i8_dual_silu_N2048_K512, mScaleB_gate)
GSB200_DECL_POINTER_(gemm_i8_dual_silu_N2048_K512, mScaleB_up)

static inline int32_t cute_dsl_gemm_i8_dual_silu_N2048_K512_wrapper(
    gemm_i8_dual_silu_N2048_K512_Kernel_Module_t* module, gemm_i8_dual_silu_N2048_K512_Tensor_mA_t* mA,
    gemm_i8_dual_silu_N2048_K512_Tensor_mB_gate_t* mB_gate, gemm_i8_dual_silu_N2048_K512_Tensor_mB_up_t* mB_up,
    gemm_i8_dual_silu_N2048_K512_Tensor_mC_t* mC, gemm_i8_dual_silu_N2048_K512_Tensor_mScaleA_t* mScaleA,
    gemm_i8_dual_silu_N2048_K512_Tensor_mScaleB_gate_t* mScaleB_gate,
    gemm_i8_dual_silu_N2048_K512_Tensor_mScaleB_up_t* mScaleB_up) {
  (void)module;
  const int32_t M = mA->dynamic_shapes[0], K = mA->dynamic_shapes[1], L = mA->dynamic_shapes[2];
  const int32_t N = mB_gate->dynamic_shapes[0];
  if (mB_gate->dynamic_shapes[1] != K || mB_up->dynamic_shapes[0] != N || mB_up->dynamic_shapes[1] != K ||
      mB_up->dynamic_strides[0] != mB_gate->dynamic_strides[0] || mC->dynamic_shapes[0] != M || mC->dynamic_shapes[1] != N)
    return GSB200_ERR_BAD_ARG;
  for (int32_t l = 0; l < L; ++l) {
    int32_t rc = gsb200_dual_gemm_i8_silu_f16(
        (const int8_t*)GSB200_BATCH_PTR_(mA, l, 1), mA->dynamic_strides[0], (const int8_t*)GSB200_BATCH_PTR_(mB_gate, l, 1),
        (const int8_t*)GSB200_BATCH_PTR_(mB_up, l, 1), mB_gate->dynamic_strides[0], GSB200_BATCH_PTR_(mC, l, 2),
        mC->dynamic_strides[0], (const float*)mScaleA->data + (int64_t)l * M, (const float*)mScaleB_gate->data + (int64_t)l * N,
        (const float*)mScaleB_up->data + (int64_t)l * N, M, N, K, 0, (gsb200_stream_t)0);
    if (rc != 0) return rc;
  }
  return 0;
}
