// C++ consumer of the CUDA twins of the reference's fp8_*_wrapper headers.  Mirrors the all-ones known-answer
// check of fly/main_rdna_fp8_gemm.cpp:136-205: A = B = fp8(1.0), unit scales -> every C element equals K.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <vector>

#define FP8_GEMM_N 512
#define FP8_GEMM_K 512
#include "fp8_wrappers.h"

int main() {
  const int M = 200, N = FP8_GEMM_N, K = FP8_GEMM_K;
  fp8_gemm_Module_t mod;
  if (fp8_gemm_Module_Load(&mod, "unused.hsaco") != 0) { std::printf("module load failed\n"); return 2; }
  std::vector<uint8_t> a((size_t)M * K, 0x38), b((size_t)N * K, 0x38);   // 0x38 = E4M3 1.0
  std::vector<float> sa(M, 1.0f), sb(N, 1.0f);
  std::vector<__half> c((size_t)M * N);
  void *d_a, *d_b, *d_c, *d_sa, *d_sb;
  cudaMalloc(&d_a, a.size()); cudaMalloc(&d_b, b.size()); cudaMalloc(&d_c, c.size() * 2);
  cudaMalloc(&d_sa, M * 4); cudaMalloc(&d_sb, N * 4);
  cudaMemcpy(d_a, a.data(), a.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(d_b, b.data(), b.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(d_sa, sa.data(), M * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d_sb, sb.data(), N * 4, cudaMemcpyHostToDevice);
  cudaStream_t st;
  cudaStreamCreate(&st);
  int rc = fp8_gemm_wrapper(&mod, d_c, d_a, d_b, d_sa, d_sb, M, st);
  cudaStreamSynchronize(st);
  cudaMemcpy(c.data(), d_c, c.size() * 2, cudaMemcpyDeviceToHost);
  int bad = 0;
  for (size_t i = 0; i < c.size(); ++i) bad += std::fabs(__half2float(c[i]) - (float)K) > 0.5f;
  std::printf("fp8_gemm_wrapper rc=%d mismatches=%d\n", rc, bad);
  fp8_gemm_Module_Unload(&mod);
  return (rc == 0 && bad == 0) ? 0 : 1;
}
