/* Drop-in for the reference's exported `gemm_i8_standard.h` (prefix gemm_i8_std, cute/export_gemm_i8.py:16-28):
 * W8A8 GEMM with per-token x per-channel dequant to fp16.  Argument order = the kernel's __call__:
 * mA, mB, mC, mScaleA, mScaleB (cute/main.cpp:125). */
#pragma once
#include "../cute_dsl_abi.h"

GSB200_DECL_MODULE_(gemm_i8_std)
GSB200_DECL_STRIDED_(gemm_i8_std, mA)
GSB200_DECL_STRIDED_(gemm_i8_std, mB)
GSB200_DECL_STRIDED_(gemm_i8_std, mC)
GSB200_DECL_POINTER_(gemm_i8_std, mScaleA)
GSB200_DECL_POINTER_(gemm_i8_std, mScaleB)

static inline int32_t cute_dsl_gemm_i8_std_wrapper(gemm_i8_std_Kernel_Module_t* module, gemm_i8_std_Tensor_mA_t* mA,
                                                   gemm_i8_std_Tensor_mB_t* mB, gemm_i8_std_Tensor_mC_t* mC,
                                                   gemm_i8_std_Tensor_mScaleA_t* mScaleA,
                                                   gemm_i8_std_Tensor_mScaleB_t* mScaleB) {
  (void)module;
  const int32_t M = mA->dynamic_shapes[0], K = mA->dynamic_shapes[1], L = mA->dynamic_shapes[2];
  const int32_t N = mB->dynamic_shapes[0];
  if (mB->dynamic_shapes[1] != K || mC->dynamic_shapes[0] != M || mC->dynamic_shapes[1] != N) return GSB200_ERR_BAD_ARG;
  for (int32_t l = 0; l < L; ++l) {
    /* scale vectors are [M, L] / [N, L] with unit stride along M / N (cute/ampere_gemm_i8_quant_rmem.py:233-234) */
    int32_t rc = gsb200_gemm_i8_f16((const int8_t*)GSB200_BATCH_PTR_(mA, l, 1), mA->dynamic_strides[0],
                                    (const int8_t*)GSB200_BATCH_PTR_(mB, l, 1), mB->dynamic_strides[0],
                                    GSB200_BATCH_PTR_(mC, l, 2), mC->dynamic_strides[0],
                                    (const float*)mScaleA->data + (int64_t)l * M, (const float*)mScaleB->data + (int64_t)l * N,
                                    M, N, K, 0, (gsb200_stream_t)0);
    if (rc != 0) return rc;
  }
  return 0;
}
