/* Body shared by the W8A8 dequant GEMM drop-ins (the reference exports one, prefix gemm_i8_std,
 * cute/export_gemm_i8.py:16-28).  Define GSB200_STD_PREFIX before including.  Wrapper arguments = the kernel's
 * __call__: mA, mB, mC, mScaleA, mScaleB (cute/main.cpp:125). */
#include "../cute_dsl_abi.h"

#define GSB200_STD_(s) GSB200_CAT_(GSB200_STD_PREFIX, s)

GSB200_DECL_MODULE_(GSB200_STD_PREFIX)
GSB200_DECL_STRIDED_(GSB200_STD_PREFIX, mA)
GSB200_DECL_STRIDED_(GSB200_STD_PREFIX, mB)
GSB200_DECL_STRIDED_(GSB200_STD_PREFIX, mC)
GSB200_DECL_POINTER_(GSB200_STD_PREFIX, mScaleA)
GSB200_DECL_POINTER_(GSB200_STD_PREFIX, mScaleB)

static inline int32_t GSB200_CAT_(cute_dsl_, GSB200_STD_(_wrapper))(GSB200_STD_(_Kernel_Module_t)* module, GSB200_STD_(_Tensor_mA_t)* mA,
                                                   GSB200_STD_(_Tensor_mB_t)* mB, GSB200_STD_(_Tensor_mC_t)* mC,
                                                   GSB200_STD_(_Tensor_mScaleA_t)* mScaleA,
                                                   GSB200_STD_(_Tensor_mScaleB_t)* mScaleB) {
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

#undef GSB200_STD_
#undef GSB200_STD_PREFIX
