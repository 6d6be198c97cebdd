/*
 * CUDA twins of the header-only HIP wrappers the reference generates for its FP8 kernels
 * (fly/export_fp8_*.py, fly/export_f16_down_proj.py): same type names, function names and argument order,
 * `hipDeviceptr_t` -> `const void*` / `void*`, `hipStream_t` -> `cudaStream_t`.  As in the reference the shapes
 * other than M are compile-time constants: define the FP8_*_N / _K / ... macros you need before including this
 * file (defaults = the deployed export configs).  Differences, all stated in INTEGRATION.md:
 *   - weights are K-major [N, K], not the RDNA WMMA pre-shuffle (convert once with gigaslop_b200.layout);
 *   - <x>_Module_Load takes the .hsaco path for source compatibility and ignores it (the code is in
 *     libgigaslop_b200); it validates the current device instead;
 *   - M does not have to be a multiple of a tile size.
 * Return convention as in the reference: 0 ok, -1 bad argument, otherwise the CUDA error code.
 */
#ifndef GIGASLOP_B200_FP8_WRAPPERS_H_
#define GIGASLOP_B200_FP8_WRAPPERS_H_

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "gigaslop_b200.h"

#ifndef FP8_GEMM_N
#define FP8_GEMM_N 1536            /* fly/export_configs/rdna_fp8_gemm.toml */
#endif
#ifndef FP8_GEMM_K
#define FP8_GEMM_K 512
#endif
#ifndef FP8_GEMM_ROTARY_N
#define FP8_GEMM_ROTARY_N 1536
#endif
#ifndef FP8_GEMM_ROTARY_K
#define FP8_GEMM_ROTARY_K 512
#endif
#ifndef FP8_GEMM_ROTARY_HALF
#define FP8_GEMM_ROTARY_HALF 32
#endif
#ifndef FP8_GEMM_ROTARY_NHEAD
#define FP8_GEMM_ROTARY_NHEAD 8
#endif
#ifndef FP8_DUAL_SILU_N
#define FP8_DUAL_SILU_N 2048       /* fly/export_configs/rdna_fp8_dual_gemm_silu.toml */
#endif
#ifndef FP8_DUAL_SILU_K
#define FP8_DUAL_SILU_K 512
#endif
#ifndef FP8_DUAL_MXFP8_N
#define FP8_DUAL_MXFP8_N 2048
#endif
#ifndef FP8_DUAL_MXFP8_K
#define FP8_DUAL_MXFP8_K 512
#endif
#ifndef FP8_PTQ_K
#define FP8_PTQ_K 512
#endif
#ifndef FP8_DOWN_PROJ_C
#define FP8_DOWN_PROJ_C 1024       /* fly/export_configs/rdna_fp8_down_proj.toml */
#endif
#ifndef FP8_DOWN_PROJ_R
#define FP8_DOWN_PROJ_R 128
#endif
#ifndef F16_DOWN_PROJ_C
#define F16_DOWN_PROJ_C 1024
#endif
#ifndef F16_DOWN_PROJ_R
#define F16_DOWN_PROJ_R 128
#endif
#ifndef FP8_FAC_GEMM_C
#define FP8_FAC_GEMM_C 1024        /* fly/export_configs/rdna_fp8_factored_gemm.toml */
#endif
#ifndef FP8_FAC_GEMM_R
#define FP8_FAC_GEMM_R 128
#endif
#ifndef FP8_FAC_GEMM_N
#define FP8_FAC_GEMM_N 4096
#endif
#ifndef FP8_FACTORED_LSTM_H
#define FP8_FACTORED_LSTM_H 1024   /* fly/export_configs/rdna_fp8_factored_lstm.toml */
#endif
#ifndef FP8_FACTORED_LSTM_K_HH
#define FP8_FACTORED_LSTM_K_HH 128
#endif
#ifndef FP8_FACTORED_LSTM_R
#define FP8_FACTORED_LSTM_R 128
#endif
#define FP8_FACTORED_LSTM_OUT_SCALE (1.0f / 448.0f)

#define GSB200_FP8_MODULE_(name)                                                         \
  typedef struct { void* module; void* func; } name##_Module_t;                          \
  static inline int name##_Module_Load(name##_Module_t* m, const char* hsaco_path) {     \
    (void)hsaco_path;                                                                    \
    m->module = 0; m->func = 0;                                                          \
    return gsb200_init();                                                                \
  }                                                                                      \
  static inline void name##_Module_Unload(name##_Module_t* m) { m->module = 0; m->func = 0; }

GSB200_FP8_MODULE_(fp8_ptq)
GSB200_FP8_MODULE_(fp8_gemm)
GSB200_FP8_MODULE_(fp8_gemm_rotary)
GSB200_FP8_MODULE_(fp8_dual_silu)
GSB200_FP8_MODULE_(fp8_dual_mxfp8)
GSB200_FP8_MODULE_(fp8_down_proj)
GSB200_FP8_MODULE_(f16_down_proj)
GSB200_FP8_MODULE_(fp8_factored_lstm)
GSB200_FP8_MODULE_(fp8_fac_gemm)

/* fly/export_fp8_dual_gemm_silu.py:311-329 */
static inline int fp8_ptq_wrapper(const fp8_ptq_Module_t* m, void* d_out_fp8, void* d_out_scale, const void* d_inp,
                                  int32_t M, cudaStream_t stream) {
  (void)m;
  return gsb200_ptq_fp8(d_inp, GSB200_F16, FP8_PTQ_K, (uint8_t*)d_out_fp8, FP8_PTQ_K, (float*)d_out_scale, M, FP8_PTQ_K,
                        0, (gsb200_stream_t)stream);
}

/* fly/export_fp8_gemm.py:222-237 (output fp16) */
static inline int fp8_gemm_wrapper(const fp8_gemm_Module_t* m, void* d_C, const void* d_A, const void* d_B_nk,
                                   const void* d_scale_a, const void* d_scale_b, int32_t M, cudaStream_t stream) {
  (void)m;
  return gsb200_gemm_fp8_f16((const uint8_t*)d_A, FP8_GEMM_K, (const uint8_t*)d_B_nk, FP8_GEMM_K, d_C, FP8_GEMM_N,
                             (const float*)d_scale_a, (const float*)d_scale_b, M, FP8_GEMM_N, FP8_GEMM_K, 0,
                             (gsb200_stream_t)stream);
}

/* fly/export_fp8_gemm_rotary.py:204-222 */
static inline int fp8_gemm_rotary_wrapper(const fp8_gemm_rotary_Module_t* m, void* d_C, const void* d_A,
                                          const void* d_B_nk, const void* d_scale_a, const void* d_scale_b,
                                          const void* d_sin, const void* d_cos, int32_t M, int32_t seqlen,
                                          cudaStream_t stream) {
  (void)m;
  return gsb200_gemm_fp8_rotary_f16((const uint8_t*)d_A, FP8_GEMM_ROTARY_K, (const uint8_t*)d_B_nk, FP8_GEMM_ROTARY_K, d_C,
                                    FP8_GEMM_ROTARY_N, (const float*)d_scale_a, (const float*)d_scale_b,
                                    (const float*)d_sin, (const float*)d_cos, M, FP8_GEMM_ROTARY_N, FP8_GEMM_ROTARY_K,
                                    FP8_GEMM_ROTARY_NHEAD, 2 * FP8_GEMM_ROTARY_HALF, 2 * FP8_GEMM_ROTARY_HALF, seqlen, 0, 0,
                                    (gsb200_stream_t)stream);
}

/* fly/export_fp8_dual_gemm_silu.py:226-255 */
static inline int fp8_dual_silu_wrapper(const fp8_dual_silu_Module_t* m, void* d_C, const void* d_A,
                                        const void* d_B_gate_nk, const void* d_B_up_nk, const void* d_scale_a,
                                        const void* d_scale_b_gate, const void* d_scale_b_up, int32_t M,
                                        cudaStream_t stream) {
  (void)m;
  return gsb200_dual_gemm_fp8_silu_f16((const uint8_t*)d_A, FP8_DUAL_SILU_K, (const uint8_t*)d_B_gate_nk,
                                       (const uint8_t*)d_B_up_nk, FP8_DUAL_SILU_K, d_C, FP8_DUAL_SILU_N,
                                       (const float*)d_scale_a, (const float*)d_scale_b_gate, (const float*)d_scale_b_up,
                                       M, FP8_DUAL_SILU_N, FP8_DUAL_SILU_K, 0, (gsb200_stream_t)stream);
}

/* fly/export_fp8_dual_gemm_silu_mxfp8.py:206-236: out_fp8 [M,N] + out_scale uint8 [M,N/32] */
static inline int fp8_dual_silu_mxfp8_wrapper(const fp8_dual_mxfp8_Module_t* m, void* d_out_fp8, void* d_out_scale,
                                              const void* d_A, const void* d_B_gate_nk, const void* d_B_up_nk,
                                              const void* d_scale_a, const void* d_scale_b_gate,
                                              const void* d_scale_b_up, int32_t M, cudaStream_t stream) {
  (void)m;
  return gsb200_dual_gemm_fp8_silu_mxfp8((const uint8_t*)d_A, FP8_DUAL_MXFP8_K, (const uint8_t*)d_B_gate_nk,
                                         (const uint8_t*)d_B_up_nk, FP8_DUAL_MXFP8_K, (uint8_t*)d_out_fp8, FP8_DUAL_MXFP8_N,
                                         (uint8_t*)d_out_scale, FP8_DUAL_MXFP8_N / 32, (const float*)d_scale_a,
                                         (const float*)d_scale_b_gate, (const float*)d_scale_b_up, M, FP8_DUAL_MXFP8_N,
                                         FP8_DUAL_MXFP8_K, 0, (gsb200_stream_t)stream);
}

/* fly/export_fp8_down_proj.py:144-155: x_down_f16[M,R] = (x_fp8 . dn_fp8) * sx[m] * s_dn; any M */
static inline int fp8_down_proj_wrapper(const fp8_down_proj_Module_t* m, void* d_x_down, const void* d_x,
                                        const void* d_scale_x, const void* d_dn_rc, const void* d_scale_dn, int32_t M,
                                        cudaStream_t stream) {
  (void)m;
  return gsb200_gemm_fp8_f16((const uint8_t*)d_x, FP8_DOWN_PROJ_C, (const uint8_t*)d_dn_rc, FP8_DOWN_PROJ_C, d_x_down,
                             FP8_DOWN_PROJ_R, (const float*)d_scale_x, (const float*)d_scale_dn, M, FP8_DOWN_PROJ_R,
                             FP8_DOWN_PROJ_C, GSB200_FLAG_SCALAR_SCALE_B, (gsb200_stream_t)stream);
}

/* fly/export_f16_down_proj.py:128-137 */
static inline int f16_down_proj_wrapper(const f16_down_proj_Module_t* m, void* d_x_down, const void* d_x,
                                        const void* d_dn_rc, int32_t M, cudaStream_t stream) {
  (void)m;
  return gsb200_gemm_f16_f16(d_x, F16_DOWN_PROJ_C, d_dn_rc, F16_DOWN_PROJ_C, d_x_down, F16_DOWN_PROJ_R, 0, 0, M,
                             F16_DOWN_PROJ_R, F16_DOWN_PROJ_C, 0, (gsb200_stream_t)stream);
}

/* fly/export_fp8_factored_gemm.py:178-203: ih_f16[M,N] = f16((x_fp8 . dn_fp8) * sx[m] * s_dn) . up_f16 + bias; any M.
 * dn is taken K-major [R,C] and up K-major [N,R] instead of the RDNA pre-shuffles. */
static inline int fp8_fac_gemm_wrapper(const fp8_fac_gemm_Module_t* m, void* d_ih_out, const void* d_x,
                                       const void* d_scale_x, const void* d_dn_rc, const void* d_scale_dn,
                                       const void* d_up_nr, const void* d_bias, int32_t M, cudaStream_t stream) {
  (void)m;
  return gsb200_fac_gemm_fp8_f16((const uint8_t*)d_x, FP8_FAC_GEMM_C, (const float*)d_scale_x, (const uint8_t*)d_dn_rc,
                                 FP8_FAC_GEMM_C, (const float*)d_scale_dn, d_up_nr, FP8_FAC_GEMM_R, (const float*)d_bias,
                                 d_ih_out, FP8_FAC_GEMM_N, M, FP8_FAC_GEMM_C, FP8_FAC_GEMM_R, FP8_FAC_GEMM_N,
                                 (gsb200_stream_t)stream);
}

/* fly/export_fp8_factored_lstm.py:158-182 */
static inline int fp8_factored_lstm_wrapper(const fp8_factored_lstm_Module_t* m, void* d_h_fp8_out, void* d_c_inout,
                                            const void* d_hh_down, const void* d_up_hh_nk, const void* d_bias_hh,
                                            const void* d_x_down, const void* d_up_ih_nk, const void* d_bias_ih,
                                            int32_t B, cudaStream_t stream) {
  (void)m;
  return gsb200_factored_lstm_step((uint8_t*)d_h_fp8_out, (float*)d_c_inout, d_hh_down, d_up_hh_nk, (const float*)d_bias_hh,
                                   d_x_down, d_up_ih_nk, (const float*)d_bias_ih, B, FP8_FACTORED_LSTM_H,
                                   FP8_FACTORED_LSTM_K_HH, FP8_FACTORED_LSTM_R, (gsb200_stream_t)stream);
}

#endif /* GIGASLOP_B200_FP8_WRAPPERS_H_ */
