// Declarations shared by the translation units of libgigaslop_b200.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
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
  // fused activation quantiser (KIND_I8 + EPI_ROTARY, K <= 512): fp16 activations instead of A / scale_a
  const __half* x_f16; long long ldx; float* scale_a_out;
  int sm_cap;                    // > 0: this launch uses at most so many CTAs (beside the process-wide cap)
};
int32_t launch_gemm(const GemmArgs& a, cudaStream_t st);
struct LstmLayerArgs {
  const __half* ih; long long ld_ih;        // [T*B, 4H] fp16 hoisted input projection, row = t*B + b
  const uint8_t* w_hh; long long ld_w;      // [4H, H] E4M3, K-major
  const float* s_hh; const float* bias;     // [4H]; bias may be null
  const uint8_t* h0; const __half* c0;      // [B, H] initial state or null
  __half* h_out; uint8_t* h8_out; __half* c_last;
  long long T, B; int H; int reverse;
};
size_t lstm_scratch_bytes(long long B, int H);
int32_t launch_lstm_layer(const LstmLayerArgs& a, void* scratch, size_t scratch_bytes, cudaStream_t st);
int32_t launch_lstm_layer_static(const LstmLayerArgs& a, cudaStream_t st);
size_t lstm_stack_workspace_bytes(long long T, long long B, int H, int overlap);
int32_t launch_lstm_stack(const uint8_t* x, long long ldx, const float* sx, int C, const gsb200_lstm_layer_t* layers,
                          int n_layers, int reverse_first, __half* h_out, long long T, long long B, int H,
                          int time_blocks, void* ws, size_t ws_bytes, cudaStream_t st, cudaStream_t aux);
int32_t launch_factored_lstm_step(uint8_t* h_out, float* c, const __half* hh_down, const __half* up_hh,
                                  const float* bias_hh, const __half* x_down, const __half* up_ih, const float* bias_ih,
                                  long long B, int H, int K_hh, int R, cudaStream_t st);
size_t mx_tiled_scale_bytes(long long rows, int K);
int32_t launch_mx_scales_to_tiled(const uint8_t* src, long long ld, long long rows, int K, uint8_t* dst, cudaStream_t st);
int32_t launch_mx_gemm(bool dual, const uint8_t* A, long long lda, const uint8_t* sfa, const uint8_t* B0,
                       const uint8_t* B1, long long ldb, const uint8_t* sfb0, const uint8_t* sfb1, void* C,
                       long long ldc, long long M, int N, int K, cudaStream_t st);
int32_t launch_tensor_peak_probe(int kind, int n, int mmas, long long* clocks, int* ctas_out, cudaStream_t st);
int32_t ensure_device();          // validates the current device once, returns GSB200_OK / error
int sm_count();                   // SMs of the current device (cached), capped by set_sm_limit
int sm_count_physical();          // SMs of the current device, whatever the cap
void set_gemm_variant(int epilogue_warps, int cta_pairs);   // -1 = by shape
void set_sm_limit(int sms);       // process-wide cap for the grids of the persistent GEMM kernels (0 = none)
// Tiled 2-D tensor map of a row-major [rows, cols] tensor (served from a per-thread table when the same
// arguments come again); false if the driver refuses it.
bool tmap_2d(CUtensorMap* m, CUtensorMapDataType dt, int esz, const void* base, uint64_t rows, uint64_t cols,
             uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swz);
unsigned long long tmap_encode_count();   // tensor maps actually encoded since the library was loaded
int32_t read_clear_status(uint32_t out[4]);
int32_t set_spin_budget(uint32_t clocks);
int32_t selftest_wait_timeout(cudaStream_t st);

}  // namespace gsb
