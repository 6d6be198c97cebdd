/* Body shared by the `gemm_i8_dual_silu_N<N>_K<K>.h` drop-ins (name pattern: cute/export_dual_gemm_i8_silu.py:53-63).
 * Define GSB200_DUAL_PREFIX before including.  Wrapper arguments = the kernel's __call__: mA, mB_gate, mB_up, mC,
 * mScaleA, mScaleB_gate, mScaleB_up (cute/ampere_dual_gemm_i8_silu.py:52-61,469-471); every extent is read from the
 * descriptors at run time. */
#include "../cute_dsl_abi.h"

#define GSB200_DUAL_(s) GSB200_CAT_(GSB200_DUAL_PREFIX, s)

GSB200_DECL_MODULE_(GSB200_DUAL_PREFIX)
GSB200_DECL_STRIDED_(GSB200_DUAL_PREFIX, mA)
GSB200_DECL_STRIDED_(GSB200_DUAL_PREFIX, mB_gate)
GSB200_DECL_STRIDED_(GSB200_DUAL_PREFIX, mB_up)
GSB200_DECL_STRIDED_(GSB200_DUAL_PREFIX, mC)
GSB200_DECL_POINTER_(GSB200_DUAL_PREFIX, mScaleA)
GSB200_DECL_POINTER_(GSB200_DUAL_PREFIX, mScaleB_gate)
GSB200_DECL_POINTER_(GSB200_DUAL_PREFIX, mScaleB_up)

static inline int32_t GSB200_CAT_(cute_dsl_, GSB200_DUAL_(_wrapper))(
    GSB200_DUAL_(_Kernel_Module_t)* module, GSB200_DUAL_(_Tensor_mA_t)* mA,
    GSB200_DUAL_(_Tensor_mB_gate_t)* mB_gate, GSB200_DUAL_(_Tensor_mB_up_t)* mB_up,
    GSB200_DUAL_(_Tensor_mC_t)* mC, GSB200_DUAL_(_Tensor_mScaleA_t)* mScaleA,
    GSB200_DUAL_(_Tensor_mScaleB_gate_t)* mScaleB_gate,
    GSB200_DUAL_(_Tensor_mScaleB_up_t)* mScaleB_up) {
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

#undef GSB200_DUAL_
#undef GSB200_DUAL_PREFIX
