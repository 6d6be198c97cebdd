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
  if (rc != 0 || bad != 0) return 1;

  // fp8_fac_gemm_wrapper (fly/export_fp8_factored_gemm.py:178-203), known answer: x = 1, dn = 1 (scale 1/8),
  // sx = 1/8 -> x_down = C/64 = 16; up = 1/4, bias = 3 -> ih = 16 * R / 4 + 3 = 515.
  {
    const int Mf = 300, C = FP8_FAC_GEMM_C, R = FP8_FAC_GEMM_R, Nf = FP8_FAC_GEMM_N;
    fp8_fac_gemm_Module_t fm;
    if (fp8_fac_gemm_Module_Load(&fm, "unused.hsaco") != 0) { std::printf("module load failed\n"); return 2; }
    std::vector<uint8_t> x((size_t)Mf * C, 0x38), dn((size_t)R * C, 0x38);
    std::vector<float> sx(Mf, 0.125f), sdn(1, 0.125f), bias(Nf, 3.0f);
    std::vector<__half> up((size_t)Nf * R, __float2half(0.25f)), ih((size_t)Mf * Nf);
    void *d_x, *d_dn, *d_sx, *d_sdn, *d_up, *d_bias, *d_ih;
    cudaMalloc(&d_x, x.size()); cudaMalloc(&d_dn, dn.size()); cudaMalloc(&d_sx, Mf * 4); cudaMalloc(&d_sdn, 4);
    cudaMalloc(&d_up, up.size() * 2); cudaMalloc(&d_bias, Nf * 4); cudaMalloc(&d_ih, ih.size() * 2);
    cudaMemcpy(d_x, x.data(), x.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_dn, dn.data(), dn.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_sx, sx.data(), Mf * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_sdn, sdn.data(), 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_up, up.data(), up.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(d_bias, bias.data(), Nf * 4, cudaMemcpyHostToDevice);
    const int rc2 = fp8_fac_gemm_wrapper(&fm, d_ih, d_x, d_sx, d_dn, d_sdn, d_up, d_bias, Mf, st);
    cudaStreamSynchronize(st);
    cudaMemcpy(ih.data(), d_ih, ih.size() * 2, cudaMemcpyDeviceToHost);
    int bad2 = 0;
    for (size_t i = 0; i < ih.size(); ++i) bad2 += std::fabs(__half2float(ih[i]) - 515.0f) > 0.5f;
    std::printf("fp8_fac_gemm_wrapper rc=%d mismatches=%d\n", rc2, bad2);
    fp8_fac_gemm_Module_Unload(&fm);
    if (rc2 != 0 || bad2 != 0) return 1;
  }
  return 0;
}
