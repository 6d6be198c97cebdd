// extern "C" surface of libgigaslop_b200 (see include/gigaslop_b200/gigaslop_b200.h).
#include "capi_internal.h"
#include "gemm_kernel.cuh"

using namespace gsb;

static inline cudaStream_t S(gsb200_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" {

const char* gsb200_version(void) { return "gigaslop_b200 0.1 (sm_100a)"; }

int32_t gsb200_init(void) { return ensure_device(); }

int32_t gsb200_device_status(uint32_t out[4]) {
  if (!out) return GSB200_ERR_BAD_ARG;
  return read_clear_status(out);
}

int32_t gsb200_set_spin_budget(uint32_t clocks) { return set_spin_budget(clocks); }

int32_t gsb200_set_gemm_variant(int32_t epilogue_warps, int32_t cta_pairs) {
  if ((epilogue_warps != -1 && epilogue_warps != 8 && epilogue_warps != 12) || cta_pairs < -1 || cta_pairs > 1) return GSB200_ERR_BAD_ARG;
  set_gemm_variant(epilogue_warps, cta_pairs);
  return GSB200_OK;
}
int32_t gsb200_set_sm_limit(int32_t sms) {
  if (sms < 0) return GSB200_ERR_BAD_ARG;
  set_sm_limit(sms);
  return GSB200_OK;
}

int32_t gsb200_selftest_wait_timeout(gsb200_stream_t stream) { return selftest_wait_timeout(S(stream)); }

int32_t gsb200_tensor_peak_probe(int32_t kind, int32_t n, int32_t mmas, int64_t* clocks, int32_t* ctas_out,
                                 gsb200_stream_t stream) {
  int ctas = 0;
  const int32_t rc = launch_tensor_peak_probe(kind, n, mmas, reinterpret_cast<long long*>(clocks), &ctas, S(stream));
  if (ctas_out) *ctas_out = ctas;
  return rc;
}

int64_t gsb200_tensor_map_encodes(void) { return static_cast<int64_t>(tmap_encode_count()); }

int32_t gsb200_ptq_int8(const void* x, int32_t x_dtype, int64_t ldx, int8_t* q, int64_t ldq, float* scale, int64_t M,
                        int32_t K, gsb200_stream_t stream) {
  return launch_ptq(x, x_dtype, ldx, q, ldq, scale, M, K, 0, S(stream));
}

int32_t gsb200_ptq_fp8(const void* x, int32_t x_dtype, int64_t ldx, uint8_t* q, int64_t ldq, float* scale, int64_t M,
                       int32_t K, int32_t torch_formulation, gsb200_stream_t stream) {
  return launch_ptq(x, x_dtype, ldx, q, ldq, scale, M, K, torch_formulation ? 2 : 1, S(stream));
}

int32_t gsb200_ptq_mxfp8(const void* x, int32_t x_dtype, int64_t ldx, uint8_t* q, int64_t ldq, uint8_t* scales,
                         int64_t ld_scales, int64_t M, int32_t K, gsb200_stream_t stream) {
  return launch_ptq_mx(x, x_dtype, ldx, q, ldq, scales, ld_scales, M, K, S(stream));
}

static GemmArgs base_args(int kind, int epi, const void* A, int64_t lda, const void* B0, const void* B1, int64_t ldb,
                          void* C, int64_t ldc, const float* sa, const float* sb0, const float* sb1, int64_t M,
                          int32_t N, int32_t K, int32_t flags) {
  GemmArgs a{};
  a.kind = kind; a.epi = epi;
  a.A = A; a.lda = lda; a.B0 = B0; a.B1 = B1; a.ldb = ldb; a.C = C; a.ldc = ldc;
  a.scale_a = sa; a.scale_b0 = sb0; a.scale_b1 = sb1;
  a.M = M; a.N = N; a.K = K; a.flags = flags;
  return a;
}

int32_t gsb200_gemm_i8_i32(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, int32_t* C, int64_t ldc,
                           int64_t M, int32_t N, int32_t K, gsb200_stream_t stream) {
  return launch_gemm(base_args(KIND_I8, EPI_I32, A, lda, B, nullptr, ldb, C, ldc, nullptr, nullptr, nullptr, M, N, K, 0),
                     S(stream));
}

int32_t gsb200_gemm_i8_f16(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, void* C, int64_t ldc,
                           const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K, int32_t flags,
                           gsb200_stream_t stream) {
  return launch_gemm(base_args(KIND_I8, EPI_DEQUANT, A, lda, B, nullptr, ldb, C, ldc, scale_a, scale_b, nullptr, M, N,
                               K, flags),
                     S(stream));
}

static int32_t rotary_common(int kind, const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
                             const float* scale_a, const float* scale_b, const float* sin_tab, const float* cos_tab,
                             int64_t M, int32_t N, int32_t K, int32_t nhead, int32_t head_dim, int32_t rotary_dim,
                             int32_t seqlen, int64_t row_offset, int32_t flags, gsb200_stream_t stream) {
  GemmArgs a = base_args(kind, EPI_ROTARY, A, lda, B, nullptr, ldb, C, ldc, scale_a, scale_b, nullptr, M, N, K, flags);
  a.sin_tab = sin_tab; a.cos_tab = cos_tab;
  a.nhead = nhead; a.head_dim = head_dim; a.rotary_dim = rotary_dim; a.seqlen = seqlen; a.row_offset = row_offset;
  return launch_gemm(a, S(stream));
}

int32_t gsb200_gemm_i8_rotary_f16(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, void* C, int64_t ldc,
                                  const float* scale_a, const float* scale_b, const float* sin_tab,
                                  const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                  int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                  int32_t flags, gsb200_stream_t stream) {
  return rotary_common(KIND_I8, A, lda, B, ldb, C, ldc, scale_a, scale_b, sin_tab, cos_tab, M, N, K, nhead, head_dim,
                       rotary_dim, seqlen, row_offset, flags, stream);
}

int32_t gsb200_ptq_gemm_i8_rotary_f16(const void* x_f16, int64_t ldx, const int8_t* B, int64_t ldb, void* C, int64_t ldc,
                                      float* scale_a_out, const float* scale_b, const float* sin_tab,
                                      const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                      int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                      int32_t flags, gsb200_stream_t stream) {
  if (!x_f16) return GSB200_ERR_BAD_ARG;
  GemmArgs a = base_args(KIND_I8, EPI_ROTARY, nullptr, 0, B, nullptr, ldb, C, ldc, nullptr, scale_b, nullptr, M, N, K, flags);
  a.sin_tab = sin_tab; a.cos_tab = cos_tab;
  a.nhead = nhead; a.head_dim = head_dim; a.rotary_dim = rotary_dim; a.seqlen = seqlen; a.row_offset = row_offset;
  a.x_f16 = static_cast<const __half*>(x_f16); a.ldx = ldx; a.scale_a_out = scale_a_out;
  return launch_gemm(a, S(stream));
}

int32_t gsb200_dual_gemm_i8_silu_f16(const int8_t* A, int64_t lda, const int8_t* B_gate, const int8_t* B_up,
                                     int64_t ldb, void* C, int64_t ldc, const float* scale_a,
                                     const float* scale_b_gate, const float* scale_b_up, int64_t M, int32_t N,
                                     int32_t K, int32_t flags, gsb200_stream_t stream) {
  return launch_gemm(base_args(KIND_I8, EPI_SILU, A, lda, B_gate, B_up, ldb, C, ldc, scale_a, scale_b_gate, scale_b_up,
                               M, N, K, flags),
                     S(stream));
}

int32_t gsb200_gemm_fp8_f16(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb, void* C, int64_t ldc,
                            const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K, int32_t flags,
                            gsb200_stream_t stream) {
  return launch_gemm(base_args(KIND_F8, EPI_DEQUANT, A, lda, B, nullptr, ldb, C, ldc, scale_a, scale_b, nullptr, M, N,
                               K, flags),
                     S(stream));
}

int32_t gsb200_gemm_fp8_rotary_f16(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb, void* C, int64_t ldc,
                                   const float* scale_a, const float* scale_b, const float* sin_tab,
                                   const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                   int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                   int32_t flags, gsb200_stream_t stream) {
  return rotary_common(KIND_F8, A, lda, B, ldb, C, ldc, scale_a, scale_b, sin_tab, cos_tab, M, N, K, nhead, head_dim,
                       rotary_dim, seqlen, row_offset, flags, stream);
}

int32_t gsb200_dual_gemm_fp8_silu_f16(const uint8_t* A, int64_t lda, const uint8_t* B_gate, const uint8_t* B_up,
                                      int64_t ldb, void* C, int64_t ldc, const float* scale_a,
                                      const float* scale_b_gate, const float* scale_b_up, int64_t M, int32_t N,
                                      int32_t K, int32_t flags, gsb200_stream_t stream) {
  return launch_gemm(base_args(KIND_F8, EPI_SILU, A, lda, B_gate, B_up, ldb, C, ldc, scale_a, scale_b_gate, scale_b_up,
                               M, N, K, flags),
                     S(stream));
}

int32_t gsb200_dual_gemm_fp8_silu_mxfp8(const uint8_t* A, int64_t lda, const uint8_t* B_gate, const uint8_t* B_up,
                                        int64_t ldb, uint8_t* out_fp8, int64_t ld_out, uint8_t* out_scale,
                                        int64_t ld_scale, const float* scale_a, const float* scale_b_gate,
                                        const float* scale_b_up, int64_t M, int32_t N, int32_t K, int32_t flags,
                                        gsb200_stream_t stream) {
  GemmArgs a = base_args(KIND_F8, EPI_SILU_MX, A, lda, B_gate, B_up, ldb, out_fp8, ld_out, scale_a, scale_b_gate,
                         scale_b_up, M, N, K, flags);
  a.out_scale = out_scale; a.ld_scale = ld_scale;
  return launch_gemm(a, S(stream));
}

int32_t gsb200_gemm_f16_f16(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
                            const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K, int32_t flags,
                            gsb200_stream_t stream) {
  // the kernel family counts K and the operand strides in bytes
  return launch_gemm(base_args(KIND_F16, EPI_DEQUANT, A, 2 * lda, B, nullptr, 2 * ldb, C, ldc, scale_a, scale_b, nullptr,
                               M, N, 2 * K, flags),
                     S(stream));
}

int32_t gsb200_fac_gemm_fp8_f16(const uint8_t* x, int64_t ldx, const float* scale_x, const uint8_t* dn_rc, int64_t lddn,
                                const float* scale_dn, const void* up_nr, int64_t ldup, const float* bias, void* ih,
                                int64_t ldih, int64_t M, int32_t C, int32_t R, int32_t N, gsb200_stream_t stream) {
  if (M == 0) return GSB200_OK;
  if (!x || !scale_x || !dn_rc || !scale_dn || !up_nr || !bias || !ih) return GSB200_ERR_BAD_ARG;
  if (R <= 0 || R % 8 != 0 || N < R || ldih < N) return GSB200_ERR_BAD_ARG;
  if (R > 256) return GSB200_ERR_UNSUPPORTED;          // the second GEMM keeps a row block's x_down (2R bytes per row) resident
  // 1. x_down[M,R] = f16((x . dn^T) * sx[m] * s_dn), written into the first R columns of each output row
  int32_t rc = launch_gemm(base_args(KIND_F8, EPI_DEQUANT, x, ldx, dn_rc, nullptr, lddn, ih, ldih, scale_x, scale_dn,
                                     nullptr, M, R, C, GSB200_FLAG_SCALAR_SCALE_B),
                           S(stream));
  if (rc != GSB200_OK) return rc;
  // 2. ih[M,N] = f16(x_down . up^T + bias), reading x_down from where step 1 left it: the activation-stationary
  //    schedule has a CTA read a row block's x_down completely before it writes that row block's output, and no
  //    other CTA touches those rows
  return launch_gemm(base_args(KIND_F16, EPI_BIAS, ih, 2 * ldih, up_nr, nullptr, 2 * ldup, ih, ldih, nullptr, bias,
                               nullptr, M, N, 2 * R, 0),
                     S(stream));
}

int32_t gsb200_factored_lstm_step(uint8_t* h_fp8_out, float* c_inout, const void* hh_down, const void* up_hh,
                                  const float* bias_hh, const void* x_down, const void* up_ih, const float* bias_ih,
                                  int64_t B, int32_t H, int32_t K_hh, int32_t R, gsb200_stream_t stream) {
  return launch_factored_lstm_step(h_fp8_out, c_inout, static_cast<const __half*>(hh_down),
                                   static_cast<const __half*>(up_hh), bias_hh, static_cast<const __half*>(x_down),
                                   static_cast<const __half*>(up_ih), bias_ih, B, H, K_hh, R, S(stream));
}

int64_t gsb200_mx_tiled_scale_bytes(int64_t rows, int32_t K) {
  if (rows <= 0 || K <= 0 || K % 128 != 0) return 0;
  return static_cast<int64_t>(mx_tiled_scale_bytes(rows, K));
}

int32_t gsb200_mx_scales_to_tiled(const uint8_t* scales, int64_t ld, int64_t rows, int32_t K, uint8_t* tiled,
                                  gsb200_stream_t stream) {
  return launch_mx_scales_to_tiled(scales, ld, rows, K, tiled, S(stream));
}

int32_t gsb200_gemm_mxfp8_f16(const uint8_t* A, int64_t lda, const uint8_t* sfa_tiled, const uint8_t* B, int64_t ldb,
                              const uint8_t* sfb_tiled, void* C, int64_t ldc, int64_t M, int32_t N, int32_t K,
                              gsb200_stream_t stream) {
  return launch_mx_gemm(false, A, lda, sfa_tiled, B, nullptr, ldb, sfb_tiled, nullptr, C, ldc, M, N, K, S(stream));
}

int32_t gsb200_dual_gemm_mxfp8_silu_f16(const uint8_t* A, int64_t lda, const uint8_t* sfa_tiled, const uint8_t* B_gate,
                                        const uint8_t* B_up, int64_t ldb, const uint8_t* sfb_gate_tiled,
                                        const uint8_t* sfb_up_tiled, void* C, int64_t ldc, int64_t M, int32_t N,
                                        int32_t K, gsb200_stream_t stream) {
  return launch_mx_gemm(true, A, lda, sfa_tiled, B_gate, B_up, ldb, sfb_gate_tiled, sfb_up_tiled, C, ldc, M, N, K,
                        S(stream));
}

int64_t gsb200_lstm_scratch_bytes(int64_t B, int32_t H) {
  if (B <= 0 || H <= 0) return 0;
  return static_cast<int64_t>(lstm_scratch_bytes(B, H));
}

int32_t gsb200_lstm_layer_fp8(const void* ih, int64_t ld_ih, const uint8_t* w_hh, int64_t ld_w, const float* s_hh,
                              const float* bias, const uint8_t* h0, const void* c0, void* h_out, uint8_t* h8_out,
                              void* c_last, int64_t T, int64_t B, int32_t H, int32_t reverse, void* scratch,
                              int64_t scratch_bytes, gsb200_stream_t stream) {
  LstmLayerArgs a{};
  a.ih = static_cast<const __half*>(ih); a.ld_ih = ld_ih; a.w_hh = w_hh; a.ld_w = ld_w; a.s_hh = s_hh; a.bias = bias;
  a.h0 = h0; a.c0 = static_cast<const __half*>(c0); a.h_out = static_cast<__half*>(h_out); a.h8_out = h8_out;
  a.c_last = static_cast<__half*>(c_last); a.T = T; a.B = B; a.H = H; a.reverse = reverse;
  return launch_lstm_layer(a, scratch, scratch_bytes < 0 ? 0 : static_cast<size_t>(scratch_bytes), S(stream));
}

int32_t gsb200_lstm_layer_fp8_static(const void* ih, int64_t ld_ih, const uint8_t* w_hh, int64_t ld_w,
                                     const float* s_hh, const float* bias, const uint8_t* h0, const void* c0,
                                     void* h_out, uint8_t* h8_out, void* c_last, int64_t T, int64_t B, int32_t H,
                                     int32_t reverse, gsb200_stream_t stream) {
  LstmLayerArgs a{};
  a.ih = static_cast<const __half*>(ih); a.ld_ih = ld_ih; a.w_hh = w_hh; a.ld_w = ld_w; a.s_hh = s_hh; a.bias = bias;
  a.h0 = h0; a.c0 = static_cast<const __half*>(c0); a.h_out = static_cast<__half*>(h_out); a.h8_out = h8_out;
  a.c_last = static_cast<__half*>(c_last); a.T = T; a.B = B; a.H = H; a.reverse = reverse;
  return launch_lstm_layer_static(a, S(stream));
}

int64_t gsb200_lstm_stack_workspace_bytes(int64_t T, int64_t B, int32_t H, int32_t overlap) {
  return static_cast<int64_t>(lstm_stack_workspace_bytes(T, B, H, overlap));
}

int32_t gsb200_lstm_stack_fp8(const uint8_t* x, int64_t ldx, const float* sx, int32_t C,
                              const gsb200_lstm_layer_t* layers, int32_t n_layers, int32_t reverse_first, void* h_out,
                              int64_t T, int64_t B, int32_t H, int32_t time_blocks, void* workspace,
                              int64_t workspace_bytes, gsb200_stream_t stream, gsb200_stream_t aux_stream) {
  return launch_lstm_stack(x, ldx, sx, C, layers, n_layers, reverse_first, static_cast<__half*>(h_out), T, B, H,
                           time_blocks, workspace, workspace_bytes < 0 ? 0 : static_cast<size_t>(workspace_bytes),
                           S(stream), S(aux_stream));
}

}  // extern "C"

// ---- module hooks named by the reference's generated headers -------------------------------------------
// `<prefix>_Kernel_Module_Load` calls `_mlir_<prefix>_cuda_init` once and `_mlir_<prefix>_cuda_load_to_device`
// once per visible device (cute/main.cpp:14-15,95-96).  Here "init" has nothing to load and "load to device"
// validates the device and sets the kernels' shared-memory attributes on it.
namespace {
void module_init(void** args) {
  // args = { cudaLibrary_t** library, cudaError_t* ret }
  if (!args) return;
  if (args[0]) **reinterpret_cast<cudaLibrary_t**>(args[0]) = nullptr;
  if (args[1]) *reinterpret_cast<cudaError_t*>(args[1]) = cudaSuccess;
}
void module_load_to_device(void** args) {
  // args = { cudaLibrary_t** library, int32_t* device_id, cudaError_t* ret }
  if (!args || !args[1] || !args[2]) return;
  const int dev = *reinterpret_cast<int32_t*>(args[1]);
  cudaError_t* ret = reinterpret_cast<cudaError_t*>(args[2]);
  int prev = 0;
  *ret = cudaGetDevice(&prev);
  if (*ret != cudaSuccess) return;
  *ret = cudaSetDevice(dev);
  if (*ret != cudaSuccess) return;
  const int32_t rc = ensure_device();
  cudaSetDevice(prev);
  *ret = rc == GSB200_OK ? cudaSuccess : (rc > 0 ? static_cast<cudaError_t>(rc) : cudaErrorInvalidDevice);
}
}  // namespace

#define GSB200_MODULE_HOOKS(P)                                                          \
  extern "C" void _mlir_##P##_cuda_init(void** a) { module_init(a); }                   \
  extern "C" void _mlir_##P##_cuda_load_to_device(void** a) { module_load_to_device(a); }

// generic pair for headers written by gigaslop_b200.export_headers (they alias their prefix's hook names to these)
extern "C" void gsb200_module_cuda_init(void** a) { module_init(a); }
extern "C" void gsb200_module_cuda_load_to_device(void** a) { module_load_to_device(a); }

GSB200_MODULE_HOOKS(gemm_i8_std)
GSB200_MODULE_HOOKS(gemm_i8_rotary_N1536_K512_H8D64R64S1024)
GSB200_MODULE_HOOKS(gemm_i8_rotary_N1536_K512_H8D64R64S2048)
GSB200_MODULE_HOOKS(gemm_i8_dual_silu_N2048_K512)

#ifdef GSB200_GEMM_PROF
// Profiling builds only: copy out (and clear) the per-CTA role timers of the GEMM kernels.
extern "C" int32_t gsb200_debug_gemm_prof(long long* out /* [160][16] */) {
  cudaError_t e = cudaMemcpyFromSymbol(out, gsb::g_gemm_prof, sizeof(long long) * 160 * 16);
  if (e != cudaSuccess) return -1;
  static long long zeros[160 * 16];
  e = cudaMemcpyToSymbol(gsb::g_gemm_prof, zeros, sizeof(zeros));
  return e == cudaSuccess ? 0 : -1;
}
#endif
