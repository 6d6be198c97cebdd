/* Body shared by the `gemm_i8_rotary_N<N>_K<K>_H<h>D<d>R<r>S<s>.h` drop-ins (name pattern:
 * cute/export_gemm_i8_rotary.py:65-67).  Define GSB200_ROT_PREFIX, GSB200_ROT_NHEAD, GSB200_ROT_HEAD_DIM,
 * GSB200_ROT_ROTARY_DIM and GSB200_ROT_SEQ_TABLE before including.  Wrapper arguments = the kernel's
 * __call__: mA, mB, mC, mScaleA, mScaleB, mSin, mCos, int32 seqlen (cute/main_rotary.cpp:158); nhead, head_dim,
 * rotary_dim and the sin/cos table extent are baked per header, M and seqlen (<= table) are runtime. */
#include "../cute_dsl_abi.h"

#define GSB200_ROT_(s) GSB200_CAT_(GSB200_ROT_PREFIX, s)

GSB200_DECL_MODULE_(GSB200_ROT_PREFIX)
GSB200_DECL_STRIDED_(GSB200_ROT_PREFIX, mA)
GSB200_DECL_STRIDED_(GSB200_ROT_PREFIX, mB)
GSB200_DECL_STRIDED_(GSB200_ROT_PREFIX, mC)
GSB200_DECL_POINTER_(GSB200_ROT_PREFIX, mScaleA)
GSB200_DECL_POINTER_(GSB200_ROT_PREFIX, mScaleB)
GSB200_DECL_POINTER_(GSB200_ROT_PREFIX, mSin)
GSB200_DECL_POINTER_(GSB200_ROT_PREFIX, mCos)

static inline int32_t GSB200_CAT_(cute_dsl_, GSB200_ROT_(_wrapper))(
    GSB200_ROT_(_Kernel_Module_t) * module, GSB200_ROT_(_Tensor_mA_t) * mA, GSB200_ROT_(_Tensor_mB_t) * mB,
    GSB200_ROT_(_Tensor_mC_t) * mC, GSB200_ROT_(_Tensor_mScaleA_t) * mScaleA, GSB200_ROT_(_Tensor_mScaleB_t) * mScaleB,
    GSB200_ROT_(_Tensor_mSin_t) * mSin, GSB200_ROT_(_Tensor_mCos_t) * mCos, int32_t seqlen) {
  (void)module;
  const int32_t M = mA->dynamic_shapes[0], K = mA->dynamic_shapes[1], L = mA->dynamic_shapes[2];
  const int32_t N = mB->dynamic_shapes[0];
  if (mB->dynamic_shapes[1] != K || mC->dynamic_shapes[0] != M || mC->dynamic_shapes[1] != N) return GSB200_ERR_BAD_ARG;
  if (seqlen < 1 || seqlen > GSB200_ROT_SEQ_TABLE) return GSB200_ERR_BAD_ARG;
  for (int32_t l = 0; l < L; ++l) {
    int32_t rc = gsb200_gemm_i8_rotary_f16(
        (const int8_t*)GSB200_BATCH_PTR_(mA, l, 1), mA->dynamic_strides[0], (const int8_t*)GSB200_BATCH_PTR_(mB, l, 1),
        mB->dynamic_strides[0], GSB200_BATCH_PTR_(mC, l, 2), mC->dynamic_strides[0],
        (const float*)mScaleA->data + (int64_t)l * M, (const float*)mScaleB->data + (int64_t)l * N,
        (const float*)mSin->data, (const float*)mCos->data, M, N, K, GSB200_ROT_NHEAD, GSB200_ROT_HEAD_DIM,
        GSB200_ROT_ROTARY_DIM, seqlen, 0, 0, (gsb200_stream_t)0);
    if (rc != 0) return rc;
  }
  return 0;
}

#undef GSB200_ROT_
#undef GSB200_ROT_PREFIX
#undef GSB200_ROT_NHEAD
#undef GSB200_ROT_HEAD_DIM
#undef GSB200_ROT_ROTARY_DIM
#undef GSB200_ROT_SEQ_TABLE
