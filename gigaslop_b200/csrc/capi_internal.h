// Declarations shared by the translation units of libgigaslop_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "gigaslop_b200/gigaslop_b200.h"

namespace gsb {

// Map a CUDA error to the C-ABI status convention (print, never abort).
inline int32_t cuda_status(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return GSB200_OK;
  fprintf(stderr, "gigaslop_b200: %s: %s (%s)\n", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return static_cast<int32_t>(e);
}

int32_t launch_ptq_mx(const void* x, int x_dtype, long long ldx, uint8_t* q, long long ldq, uint8_t* scales,
                      long long lds, long long M, int K, cudaStream_t st);
int32_t launch_ptq(const void* x, int x_dtype, long long ldx, void* q, long long ldq, float* scale, long long M,
                   int K, int fmt, cudaStream_t st);

struct GemmArgs {
  int kind;                      // KIND_I8 / KIND_F8
  int epi;                       // EPI_*
  const void* A; long long lda;
  const void* B0; const void* B1; long long ldb;
  void* C; long long ldc;
  uint8_t* out_scale; long long ld_scale;   // MXFP8 output: E8M0 scales [M, N/32]
  const float* scale_a; const float* scale_b0; const float* scale_b1;
  const float* sin_tab; const float* cos_tab;
  long long M; int N; int K;
  int nhead, head_dim, rotary_dim, seqlen; long long row_offset;
  int flags;
};
int32_t launch_gemm(const GemmArgs& a, cudaStream_t st);
int32_t ensure_device();          // validates the current device once, returns GSB200_OK / error
int sm_count();                   // SMs of the current device (cached)
int32_t read_clear_status(uint32_t out[4]);
int32_t set_spin_budget(uint32_t clocks);
int32_t selftest_wait_timeout(cudaStream_t st);

}  // namespace gsb
