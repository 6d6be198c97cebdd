// Consumer of headers written by gigaslop_b200.export_headers for shapes the repository does not ship:
// rotary N=768 (4 heads), K=256, table of 512 rows, and the dual SwiGLU GEMM N=256, K=128.  Written like the
// reference's cute/main_rotary.cpp: per-prefix module type, Module_Load, descriptor structs, wrapper call.
// With a GPU (argv[1] == "run") it checks a known answer; without, it only has to compile and link.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "gemm_i8_rotary_N768_K256_H4D64R64S512.h"
#include "gemm_i8_dual_silu_N256_K128.h"

extern "C" void _mlir_gemm_i8_rotary_N768_K256_H4D64R64S512_cuda_init(void**);   // as cute/main.cpp:14-15 declares its own

int main(int argc, char** argv) {
  if (argc < 2 || std::strcmp(argv[1], "run") != 0) { std::printf("linked\n"); return 0; }
  const int M = 200, N = 768, K = 256;
  gemm_i8_rotary_N768_K256_H4D64R64S512_Kernel_Module_t mod;
  gemm_i8_rotary_N768_K256_H4D64R64S512_Kernel_Module_Load(&mod);
  std::vector<int8_t> a((size_t)M * K, 1), b((size_t)N * K, 2);
  std::vector<float> sa(M, 0.5f), sb(N, 0.25f), sn(512 * 32, 0.0f), cs(512 * 32, 1.0f);   // identity rotation
  std::vector<__half> c((size_t)M * N);
  void *d_a, *d_b, *d_c, *d_sa, *d_sb, *d_sn, *d_cs;
  cudaMalloc(&d_a, a.size()); cudaMalloc(&d_b, b.size()); cudaMalloc(&d_c, c.size() * 2);
  cudaMalloc(&d_sa, M * 4); cudaMalloc(&d_sb, N * 4); cudaMalloc(&d_sn, sn.size() * 4); cudaMalloc(&d_cs, cs.size() * 4);
  cudaMemcpy(d_a, a.data(), a.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(d_b, b.data(), b.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(d_sa, sa.data(), M * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d_sb, sb.data(), N * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d_sn, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d_cs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice);
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mA_t mA{d_a, {M, K, 1}, {K, (int64_t)M * K}};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mB_t mB{d_b, {N, K, 1}, {K, (int64_t)N * K}};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mC_t mC{d_c, {M, N, 1}, {N, (int64_t)M * N}};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mScaleA_t mSa{d_sa};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mScaleB_t mSb{d_sb};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mSin_t mSn{d_sn};
  gemm_i8_rotary_N768_K256_H4D64R64S512_Tensor_mCos_t mCs{d_cs};
  int rc = cute_dsl_gemm_i8_rotary_N768_K256_H4D64R64S512_wrapper(&mod, &mA, &mB, &mC, &mSa, &mSb, &mSn, &mCs, 300);
  cudaDeviceSynchronize();
  cudaMemcpy(c.data(), d_c, c.size() * 2, cudaMemcpyDeviceToHost);
  int bad = 0;
  const float expect = 2.0f * K * 0.5f * 0.25f;      // acc = 2K, scales 1/2 and 1/4, identity rotation
  for (size_t i = 0; i < c.size(); ++i) bad += std::fabs(__half2float(c[i]) - expect) > 0.05f;
  std::printf("generated rotary header: rc=%d mismatches=%d\n", rc, bad);
  if (rc != 0 || bad != 0) return 1;

  // dual SwiGLU header: gate = up = K * 1 * 2 * (1/64) * (1/4) = 1 for K = 128 -> silu(1) * 1 = 0.7311
  {
    const int Md = 130, Nd = 256, Kd = 128;
    gemm_i8_dual_silu_N256_K128_Kernel_Module_t dm;
    gemm_i8_dual_silu_N256_K128_Kernel_Module_Load(&dm);
    std::vector<int8_t> x((size_t)Md * Kd, 1), w((size_t)Nd * Kd, 2);
    std::vector<float> sx(Md, 1.0f / 64), sw(Nd, 0.25f);
    std::vector<__half> o((size_t)Md * Nd);
    void *d_x, *d_wg, *d_wu, *d_o, *d_sx, *d_sg, *d_su;
    cudaMalloc(&d_x, x.size()); cudaMalloc(&d_wg, w.size()); cudaMalloc(&d_wu, w.size()); cudaMalloc(&d_o, o.size() * 2);
    cudaMalloc(&d_sx, Md * 4); cudaMalloc(&d_sg, Nd * 4); cudaMalloc(&d_su, Nd * 4);
    cudaMemcpy(d_x, x.data(), x.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_wg, w.data(), w.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_wu, w.data(), w.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_sx, sx.data(), Md * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_sg, sw.data(), Nd * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_su, sw.data(), Nd * 4, cudaMemcpyHostToDevice);
    gemm_i8_dual_silu_N256_K128_Tensor_mA_t tA{d_x, {Md, Kd, 1}, {Kd, (int64_t)Md * Kd}};
    gemm_i8_dual_silu_N256_K128_Tensor_mB_gate_t tG{d_wg, {Nd, Kd, 1}, {Kd, (int64_t)Nd * Kd}};
    gemm_i8_dual_silu_N256_K128_Tensor_mB_up_t tU{d_wu, {Nd, Kd, 1}, {Kd, (int64_t)Nd * Kd}};
    gemm_i8_dual_silu_N256_K128_Tensor_mC_t tC{d_o, {Md, Nd, 1}, {Nd, (int64_t)Md * Nd}};
    gemm_i8_dual_silu_N256_K128_Tensor_mScaleA_t tSa{d_sx};
    gemm_i8_dual_silu_N256_K128_Tensor_mScaleB_gate_t tSg{d_sg};
    gemm_i8_dual_silu_N256_K128_Tensor_mScaleB_up_t tSu{d_su};
    int rc2 = cute_dsl_gemm_i8_dual_silu_N256_K128_wrapper(&dm, &tA, &tG, &tU, &tC, &tSa, &tSg, &tSu);
    cudaDeviceSynchronize();
    cudaMemcpy(o.data(), d_o, o.size() * 2, cudaMemcpyDeviceToHost);
    int bad2 = 0;
    for (size_t i = 0; i < o.size(); ++i) bad2 += std::fabs(__half2float(o[i]) - 0.7311f) > 0.01f;
    std::printf("generated dual-silu header: rc=%d mismatches=%d\n", rc2, bad2);
    if (rc2 != 0 || bad2 != 0) return 1;
  }
  return 0;
}
