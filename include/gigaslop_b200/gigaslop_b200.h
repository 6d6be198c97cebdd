/*
 * gigaslop_b200 -- plain C ABI of the B200 (sm_100a) quantized-GEMM library.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, allocates nothing and returns a status:
 *   0   success (kernel enqueued)
 *  <0   argument / capability error (GSB200_ERR_*), nothing was launched
 *  >0   the cudaError_t of a failed CUDA call (also printed to stderr)
 * All matrices are row-major; A is [M,K], weights are K-major [N,K] (the layout of
 * an nn.Linear weight), outputs are [M,N].  Leading dimensions are in elements.
 * Alignment: base pointers 16 bytes, lda/ldb multiples of 16 (bytes of 8-bit
 * data), ldc a multiple of 8 (fp16) or 4 (int32); K % 16 == 0; N % 8 == 0.
 * M is arbitrary (tail rows are handled inside the kernels).
 *
 * The reference project exposes each kernel through a generated per-kernel
 * header (module struct + tensor descriptors + `cute_dsl_<prefix>_wrapper`, or
 * HIP `fp8_*_wrapper`); those drop-in headers live next to this file and are thin
 * inline shims over the functions declared here.  Each declaration cites the
 * reference interface it stands in for (paths relative to the reference root).
 */
#ifndef GIGASLOP_B200_H_
#define GIGASLOP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GSB200_OK 0
#define GSB200_ERR_BAD_ARG (-1)      /* null / misaligned pointer, bad size (reference wrappers return -1 for a bad M) */
#define GSB200_ERR_UNSUPPORTED (-2)  /* shape outside what the kernels were built for */
#define GSB200_ERR_DEVICE (-3)       /* current device is not an sm_100 part */

#define GSB200_F16 0
#define GSB200_F32 1

/* bit flags for the `flags` argument of the GEMM entry points; any other bit is rejected with GSB200_ERR_BAD_ARG */
#define GSB200_FLAG_SCALAR_SCALE_B 4  /* plain dequant GEMMs: scale_b points to ONE fp32 used for every output column */
/* Rotary GEMMs share the row blocks of the last, incomplete round among the CTAs that would idle (3.7 % faster alone
 * at M = 65536).  A caller that fills those SMs itself, with another kernel on a second stream, switches that off. */
#define GSB200_FLAG_OWN_ROW_BLOCKS 8

typedef struct CUstream_st* gsb200_stream_t; /* == cudaStream_t */

/* Library / device management.  No reference counterpart: the generated
 * `<prefix>_Kernel_Module_Load` (cute/main.cpp:95-96) maps onto gsb200_init. */
const char* gsb200_version(void);
int32_t gsb200_init(void);

/* Module hooks behind `<prefix>_Kernel_Module_Load` of the exported-kernel headers (cute/main.cpp:14-15 declares them
 * per prefix as `_mlir_<prefix>_cuda_init` / `_mlir_<prefix>_cuda_load_to_device`; a generated header aliases those
 * names to this pair).  Arguments as the reference's: init(&lib_handle_ptr, &cudaError_t);
 * load_to_device(&lib_handle_ptr, &device, &cudaError_t).  They validate the device and set kernel attributes. */
void gsb200_module_cuda_init(void** args);
void gsb200_module_cuda_load_to_device(void** args);                       /* validate the current device, set kernel attributes */
int32_t gsb200_device_status(uint32_t out[4]);   /* read-and-clear the device status word (0 = healthy) */
int32_t gsb200_set_spin_budget(uint32_t clocks); /* bound (SM clocks) for device-side waits; 0 restores the default */
/* The persistent GEMM kernels launch at most `sms` CTAs (one per SM) from now on; 0 restores "all SMs".  A caller that
 * runs another kernel beside a GEMM on a second stream (the quantiser of the next batch, say) leaves it a few SMs
 * this way: a GEMM CTA fills an SM's register file, so nothing else runs on the SMs it occupies.  The cap is one value
 * for the whole process: it applies to every device and every host thread, and not to the LSTM kernels (whose CTAs
 * wait on one another and are always launched in full). */
int32_t gsb200_set_sm_limit(int32_t sms);
/* Tuning override for the dequant / rotary / SwiGLU GEMMs on 8-bit operands, which exist with eight or twelve epilogue
 * warps and with one CTA or a CTA pair (tcgen05 cta_group::2) per tile; every form gives the same bytes.
 * epilogue_warps: 8 or 12; cta_pairs: 0 or 1; -1 = chosen by shape (the default).  A shape a form cannot run (fewer
 * than two K blocks for pairs) falls back to the eight-warp single-CTA kernel.  One setting for the whole process;
 * the environment variables GSB200_GEMM_EW / GSB200_GEMM_PAIR give its initial value.  No reference counterpart. */
int32_t gsb200_set_gemm_variant(int32_t epilogue_warps, int32_t cta_pairs);
/* Launches one warp that waits on a barrier nothing signals; with a small spin budget the wait gives up and
 * sets bit 2 of the status word.  Exercises the give-up path without hanging the device. */
int32_t gsb200_selftest_wait_timeout(gsb200_stream_t stream);

/* Measurement utilities (no reference counterpart).
 * gsb200_tensor_peak_probe: one CTA per SM issues `mmas` tcgen05.mma (M = 128, N = n in {128, 256}, K = 32 bytes;
 * kind 0 = kind::i8, 1 = kind::f8f6f4 on E4M3) back to back on operands that never leave shared memory.  Time the
 * launch with events: 2 * 128 * n * 32 * mmas * CTAs operations.  clocks: device int64 [2 * SMs]; per CTA the SM clocks of
 * the issue loop and of the whole window up to the last MMA's completion (-1 if the bounded wait gave up).  ctas_out
 * (host, may be null) receives the number of CTAs launched.  This is how the tensor-side roofline denominator of the
 * benchmark is measured on the box instead of taken from a datasheet.
 * gsb200_tensor_map_encodes: TMA tensor maps encoded by this process so far (they are cached per host thread; a
 * steady-state launch on buffers seen before encodes none). */
int32_t gsb200_tensor_peak_probe(int32_t kind, int32_t n, int32_t mmas, int64_t* clocks, int32_t* ctas_out,
                                 gsb200_stream_t stream);
int64_t gsb200_tensor_map_encodes(void);

/* Per-token symmetric absmax INT8 quantiser: qs = (1/amax)*127 (as PyTorch evaluates 127/amax), q = rne(x*qs), scale = 1/qs.
 * Stands in for quantize_tensor (cute/bench_quant_i8.py:15-31); the reference has no
 * GPU kernel for it.  Bit-exact with that function on fp32(x). */
int32_t gsb200_ptq_int8(const void* x, int32_t x_dtype, int64_t ldx, int8_t* q, int64_t ldq, float* scale,
                        int64_t M, int32_t K, gsb200_stream_t stream);

/* Per-token E4M3 quantiser, scale = amax/448.  torch_formulation = 0: elements = x * (448/amax)
 * (the device kernel, fly/rdna_fp8_per_token_quantize.py:127-148, exported as fp8_ptq_wrapper
 * at fly/export_fp8_dual_gemm_silu.py:311-329); 1: elements = clamp(x / scale)
 * (fp8_quantize_per_token, fly/rdna_fp8_preshuffle_gemm.py:57-70). */
int32_t gsb200_ptq_fp8(const void* x, int32_t x_dtype, int64_t ldx, uint8_t* q, int64_t ldq, float* scale,
                       int64_t M, int32_t K, int32_t torch_formulation, gsb200_stream_t stream);

/* C_i32 = A_i8 . B_i8^T.  TensorOpGemmI8 int32-out (cute/ampere_gemm_i8.py:181-702).  N % 4 == 0. */
int32_t gsb200_gemm_i8_i32(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, int32_t* C, int64_t ldc,
                           int64_t M, int32_t N, int32_t K, gsb200_stream_t stream);

/* C_f16 = f16( f32(acc) * (sA[m]*sB[n]) ).  TensorOpGemmI8 with the dequant epilogue
 * (cute/ampere_gemm_i8_quant_rmem.py:181-786; exported as cute_dsl_gemm_i8_std_wrapper,
 * cute/export_gemm_i8.py:16-28, called at cute/main.cpp:125).  Also the SwiGLU down-projection. */
int32_t gsb200_gemm_i8_f16(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, void* C, int64_t ldc,
                           const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K,
                           int32_t flags, gsb200_stream_t stream);

/* QKV projection with rotary embedding fused into the epilogue.  TensorOpGemmI8Rotary
 * (cute/ampere_gemm_i8_rotary.py:44-397; wrapper called at cute/main_rotary.cpp:158).
 * In every head of the columns [0, 2*nhead*head_dim) the first rotary_dim columns are rotated (x0 = columns
 * [0, rotary_dim/2), x1 = [rotary_dim/2, rotary_dim) of the head; out0 = x0*cos - x1*sin, out1 = x0*sin + x1*cos); the
 * rest of the head and the V columns pass through (cute/ampere_gemm_i8_rotary.py:362-393).
 * sin/cos are fp32 [>= seqlen, rotary_dim/2] row-major; the angle row of output row m is
 * (m + row_offset) % seqlen (row_offset lets a shard of M keep global positions).
 * head_dim 64 or 128, rotary_dim 32, 64, 96 or 128 (<= head_dim), N % head_dim == 0; other values return
 * GSB200_ERR_UNSUPPORTED.  head_dim = rotary_dim = 64, the shape the reference exports and benchmarks, has a
 * kernel of its own; the others share a general (slower) epilogue.  The FP8 twin and its limits are the same. */
int32_t gsb200_gemm_i8_rotary_f16(const int8_t* A, int64_t lda, const int8_t* B, int64_t ldb, void* C,
                                  int64_t ldc, const float* scale_a, const float* scale_b, const float* sin_tab,
                                  const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                  int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                  int32_t flags, gsb200_stream_t stream);

/* Per-token int8 quantisation of fp16 activations FUSED into the QKV + rotary GEMM: x_f16 [M, K] goes in, the int8
 * operand is made on chip (two warps of each CTA write it into the shared-memory block the MMAs read, with the
 * arithmetic of gsb200_ptq_int8), and never travels to memory.  The result is bit-identical to gsb200_ptq_int8
 * followed by gsb200_gemm_i8_rotary_f16 (quantize_tensor, cute/ampere_gemm_i8_quant_rmem.py:1029-1033, then
 * `cute_dsl_gemm_i8_rotary_*_wrapper`, cute/export_gemm_i8_rotary.py:69-82).  scale_a_out: optional [M] fp32, receives
 * the token scales.  K must be a multiple of 128 and at most 512, ldx a multiple of 8.  A new entry point beside
 * the drop-in ones: the reference has no fused form.  It saves the int8 round trip through memory but, as built, not
 * time: the two quantiser warps share their schedulers with the epilogue warps that bound the GEMM, and the MMAs of a
 * row block wait for them (config 2: 184 us against 97 us for the two calls, 92 us for the two calls on two streams).
 * Use it where the int8 copy of the activations must not exist; otherwise the two calls. */
int32_t gsb200_ptq_gemm_i8_rotary_f16(const void* x_f16, int64_t ldx, const int8_t* B, int64_t ldb, void* C, int64_t ldc,
                                      float* scale_a_out, const float* scale_b, const float* sin_tab,
                                      const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                      int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                      int32_t flags, gsb200_stream_t stream);

/* C_f16 = silu(A.Bg^T * sA*sBg) * (A.Bu^T * sA*sBu).  TensorOpDualGemmI8Silu
 * (cute/ampere_dual_gemm_i8_silu.py:36-438; export at cute/export_dual_gemm_i8_silu.py:53-63). */
int32_t gsb200_dual_gemm_i8_silu_f16(const int8_t* A, int64_t lda, const int8_t* B_gate, const int8_t* B_up,
                                     int64_t ldb, void* C, int64_t ldc, const float* scale_a,
                                     const float* scale_b_gate, const float* scale_b_up, int64_t M, int32_t N,
                                     int32_t K, int32_t flags, gsb200_stream_t stream);

/* FP8-E4M3 twins (fp32 accumulate, C = (acc*sA[m])*sB[n]).  Weights are taken K-major [N,K]
 * (not the RDNA WMMA pre-shuffle of fly/rdna_fp8_preshuffle_gemm.py:40-54).
 * compile_fp8_gemm (fly/rdna_fp8_preshuffle_gemm.py:94-421), compile_fp8_gemm_rotary
 * (fly/rdna_fp8_gemm_rotary.py:64-421), compile_fp8_dual_gemm_silu (fly/rdna_fp8_dual_gemm_silu.py:70-395). */
int32_t gsb200_gemm_fp8_f16(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb, void* C, int64_t ldc,
                            const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K,
                            int32_t flags, gsb200_stream_t stream);
int32_t gsb200_gemm_fp8_rotary_f16(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb, void* C,
                                   int64_t ldc, const float* scale_a, const float* scale_b, const float* sin_tab,
                                   const float* cos_tab, int64_t M, int32_t N, int32_t K, int32_t nhead,
                                   int32_t head_dim, int32_t rotary_dim, int32_t seqlen, int64_t row_offset,
                                   int32_t flags, gsb200_stream_t stream);
int32_t gsb200_dual_gemm_fp8_silu_f16(const uint8_t* A, int64_t lda, const uint8_t* B_gate, const uint8_t* B_up,
                                      int64_t ldb, void* C, int64_t ldc, const float* scale_a,
                                      const float* scale_b_gate, const float* scale_b_up, int64_t M, int32_t N,
                                      int32_t K, int32_t flags, gsb200_stream_t stream);

/* Low-rank ("factored") projections of the reference's LSTM.  Weights K-major [N,K] (see gigaslop_b200.layout for
 * the conversion from the RDNA pre-shuffle).
 *   fp8_down_proj_wrapper (fly/export_fp8_down_proj.py:144-155, kernel fly/rdna_fp8_factored_gemm.py:442-651):
 *       x_down_f16[M,R] = (x_fp8 . dn_fp8^T) * sx[m] * s_dn   ==  gsb200_gemm_fp8_f16(..., scale_b = &s_dn,
 *       flags = GSB200_FLAG_SCALAR_SCALE_B)
 *   f16_down_proj_wrapper (fly/export_f16_down_proj.py:128-137, kernel fly/rdna_fp8_factored_gemm.py:660-843):
 *       x_down_f16[M,R] = x_f16 . dn_f16^T                      ==  gsb200_gemm_f16_f16 with null scales
 * gsb200_gemm_f16_f16: C_f16 = (A_f16 . B_f16^T)_f32 * sA[m] * sB[n], either scale pointer may be null (= 1).
 * K % 8 == 0, lda / ldb (elements) % 8 == 0. */
int32_t gsb200_gemm_f16_f16(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc,
                            const float* scale_a, const float* scale_b, int64_t M, int32_t N, int32_t K,
                            int32_t flags, gsb200_stream_t stream);

/* Hoisted low-rank input projection of the reference's LSTM in one call and without scratch
 * (fp8_fac_gemm_wrapper, fly/export_fp8_factored_gemm.py:178-203; kernel fly/rdna_fp8_factored_gemm.py:86-435):
 *     ih_f16[M,N] = f16( f16((x_fp8 . dn_fp8^T) * sx[m] * s_dn) . up_f16^T + bias[n] )
 * x [M,C] E4M3 with per-token scales sx[M]; dn [R,C] E4M3 K-major with ONE scale s_dn; up [N,R] fp16 K-major;
 * bias [N] fp32; any M.  The fp16 intermediate x_down[M,R] lives in the first R columns of each output row between
 * the two launches the call makes (N >= R), so the caller provides no workspace.  C % 16 == 0, R % 8 == 0,
 * R <= 256, N % 8 == 0, ldih % 8 == 0, ldup % 8 == 0. */
int32_t gsb200_fac_gemm_fp8_f16(const uint8_t* x, int64_t ldx, const float* scale_x, const uint8_t* dn_rc, int64_t lddn,
                                const float* scale_dn, const void* up_nr, int64_t ldup, const float* bias, void* ih,
                                int64_t ldih, int64_t M, int32_t C, int32_t R, int32_t N, gsb200_stream_t stream);

/* One step of the reference's low-rank LSTM cell (compile_fp8_factored_lstm, fly/rdna_fp8_factored_lstm.py:88-351;
 * fp8_factored_lstm_wrapper, fly/export_fp8_factored_lstm.py:158-182 -- same argument order):
 *   gates[B,4H] = hh_down[B,K_hh] . up_hh[4H,K_hh]^T + x_down[B,R] . up_ih[4H,R]^T + bias_hh + bias_ih   (f16 operands)
 *   i,f,o = clamp(0.2 x + 0.5, 0, 1), g = clamp(x, -1, 1) (gate blocks i|f|g|o of H columns);
 *   c = f c + i g (fp32, in place);  h = o tanh(c) -> E4M3 at the fixed scale 1/448.
 * H % 32 == 0; K_hh, R multiples of 64 with K_hh + R <= 384; any B (the reference wants B % 32 == 0). */
int32_t gsb200_factored_lstm_step(uint8_t* h_fp8_out, float* c_inout, const void* hh_down, const void* up_hh,
                                  const float* bias_hh, const void* x_down, const void* up_ih, const float* bias_ih,
                                  int64_t B, int32_t H, int32_t K_hh, int32_t R, gsb200_stream_t stream);

/* MXFP8 (OCP microscaling): E4M3 elements with one E8M0 scale (value 2^(byte-127)) per 32 consecutive
 * elements; byte = clamp(biased fp32 exponent of the block maximum - 8, 0, 254), elements are
 * e4m3_rn_satfinite(v * 2^(127-byte)).  The reference ships only the interface of its MXFP8 kernel
 * (fly/export_fp8_dual_gemm_silu_mxfp8.py:145-236; the kernel module is absent), so this rule is this
 * library's own choice (the OCP default) -- parity unpinned.
 *
 * gsb200_ptq_mxfp8: activations fp16/fp32 [M,K] -> E4M3 [M,K] + scales uint8 [M,K/32].  K % 32 == 0.
 * gsb200_dual_gemm_fp8_silu_mxfp8: the SwiGLU dual GEMM (per-token x per-channel scaled FP8 inputs) emitting
 * MXFP8 directly: out_fp8 [M,N] + out_scale uint8 [M,N/32] row-major -- fp8_dual_silu_mxfp8_wrapper
 * (fly/export_fp8_dual_gemm_silu_mxfp8.py:206-236).  N % 32 == 0, ld_out % 16 == 0. */
int32_t gsb200_ptq_mxfp8(const void* x, int32_t x_dtype, int64_t ldx, uint8_t* q, int64_t ldq, uint8_t* scales,
                         int64_t ld_scales, int64_t M, int32_t K, gsb200_stream_t stream);
int32_t gsb200_dual_gemm_fp8_silu_mxfp8(const uint8_t* A, int64_t lda, const uint8_t* B_gate, const uint8_t* B_up,
                                        int64_t ldb, uint8_t* out_fp8, int64_t ld_out, uint8_t* out_scale,
                                        int64_t ld_scale, const float* scale_a, const float* scale_b_gate,
                                        const float* scale_b_up, int64_t M, int32_t N, int32_t K, int32_t flags,
                                        gsb200_stream_t stream);

/* Block-scaled MXFP8 GEMMs (tcgen05 kind::mxf8f6f4): BOTH operands carry one E8M0 scale per 32 K elements, fp32
 * accumulate, fp16 out.  This is the "MXFP8 dual-GEMM variant with E8M0 scales per 32-element K-block on both
 * operands" of the benchmark configuration; the reference has no kernel source for it (see the note above), so
 * parity is unpinned.  Scale factors are passed in the 128 x 4 tile order of the tensor core: the byte of
 * (row r, 32-block b) sits at ((r/128)*(K/128) + b/4)*512 + (r%32)*16 + ((r%128)/32)*4 + b%4, rows padded to 128;
 * gsb200_mx_scales_to_tiled converts row-major [rows, K/32] scales (as written by gsb200_ptq_mxfp8 and
 * gsb200_dual_gemm_fp8_silu_mxfp8) into gsb200_mx_tiled_scale_bytes(rows, K) bytes of that order.
 * K % 128 == 0, N % 32 == 0 (dual: gate and up each [N,K]). */
int64_t gsb200_mx_tiled_scale_bytes(int64_t rows, int32_t K);
int32_t gsb200_mx_scales_to_tiled(const uint8_t* scales, int64_t ld, int64_t rows, int32_t K, uint8_t* tiled,
                                  gsb200_stream_t stream);
int32_t gsb200_gemm_mxfp8_f16(const uint8_t* A, int64_t lda, const uint8_t* sfa_tiled, const uint8_t* B, int64_t ldb,
                              const uint8_t* sfb_tiled, void* C, int64_t ldc, int64_t M, int32_t N, int32_t K,
                              gsb200_stream_t stream);
int32_t gsb200_dual_gemm_mxfp8_silu_f16(const uint8_t* A, int64_t lda, const uint8_t* sfa_tiled, const uint8_t* B_gate,
                                        const uint8_t* B_up, int64_t ldb, const uint8_t* sfb_gate_tiled,
                                        const uint8_t* sfb_up_tiled, void* C, int64_t ldc, int64_t M, int32_t N,
                                        int32_t K, gsb200_stream_t stream);

/* LSTM layer, recurrent half: T sequential steps in one persistent kernel (thread-block clusters exchanging h through
 * distributed shared memory for H <= 384; a cooperative kernel with global scratch otherwise).
 *   gates[b,4H] = ih[t,b,:] + (h_{t-1} . W_hh^T) * (s_hh[n]/448) + bias[n]   (gate blocks i|f|g|o, each H wide)
 *   c_t = sigmoid(f) c_{t-1} + sigmoid(i) tanh(g),  h_t = sigmoid(o) tanh(c_t)
 * ih is the hoisted input projection of all timesteps ([T*B, 4H] fp16, row = t*B + b; produce it with
 * gsb200_gemm_fp8_f16 over M = T*B rows).  h enters the recurrent GEMM as E4M3 at the fixed scale 1/448 (the
 * convention of fly/rdna_fp8_factored_lstm.py:321-326); c and the emitted h are fp16.  reverse != 0 walks
 * t = T-1..0.  Outputs (each may be null): h_out fp16 [T*B,H], h8_out E4M3 [T*B,H] (next layer's input, row
 * scale 1/448), c_last fp16 [B,H].  The reference drives its (low-rank, hard-gate) cell as two launches per step
 * from a graph (fly/bench_factored_lstm.py:82-85,106-121, fp8_factored_lstm_wrapper
 * fly/export_fp8_factored_lstm.py:158-182); the full-rank sigmoid/tanh cell here is the benchmark's (config 5).
 * Needs H % 32 == 0, H <= 512, ceil(B/128) * H/32 <= number of SMs, and caller-provided scratch of
 * gsb200_lstm_scratch_bytes(B, H) bytes (256-byte aligned; h exchange buffer + step counters). */
int64_t gsb200_lstm_scratch_bytes(int64_t B, int32_t H);
int32_t gsb200_lstm_layer_fp8(const void* ih, int64_t ld_ih, const uint8_t* w_hh, int64_t ld_w, const float* s_hh,
                              const float* bias, const uint8_t* h0, const void* c0, void* h_out, uint8_t* h8_out,
                              void* c_last, int64_t T, int64_t B, int32_t H, int32_t reverse, void* scratch,
                              int64_t scratch_bytes, gsb200_stream_t stream);

/* The whole LSTM stack in one call: per layer the hoisted input projection (gsb200_gemm_fp8_f16 over the T*B rows)
 * and the recurrence (gsb200_lstm_layer_fp8); layer l > 0 consumes the E4M3 h of layer l - 1 at the row scale 1/448;
 * directions alternate (reverse_first != 0: layers 0, 2, ... walk t = T-1..0).  The reference keeps this loop in
 * its caller and replays two launches per timestep and layer from a graph (fly/bench_factored_lstm.py:82-85,104-121).
 * x [T*B, C] E4M3 with per-row scales sx[T*B]; layer 0 has w_ih [4H, C], the others [4H, H]; h_out fp16 [T*B, H] is
 * the last layer's output.  aux_stream (may be null): a second stream of the caller.  With it, each recurrence is cut
 * into time_blocks launches (0 = 8) and the next layer's projection of a block's timesteps runs on aux_stream beside
 * the following block, on the SMs the recurrence leaves idle; the result is the same, bit for bit.  The call returns
 * with work queued on both streams; `stream` ends up ordered after all of it.
 * workspace: gsb200_lstm_stack_workspace_bytes(T, B, H, overlap = aux_stream given) bytes, 256-byte aligned. */
typedef struct {
  const uint8_t* w_ih; int64_t ld_w_ih; const float* s_ih;   /* input weights E4M3 K-major, per-channel scales [4H] */
  const uint8_t* w_hh; int64_t ld_w_hh; const float* s_hh;   /* recurrent weights [4H, H], per-channel scales [4H] */
  const float* bias;                                          /* b_ih + b_hh [4H], or null */
} gsb200_lstm_layer_t;
int64_t gsb200_lstm_stack_workspace_bytes(int64_t T, int64_t B, int32_t H, int32_t overlap);
int32_t gsb200_lstm_stack_fp8(const uint8_t* x, int64_t ldx, const float* sx, int32_t C,
                              const gsb200_lstm_layer_t* layers, int32_t n_layers, int32_t reverse_first, void* h_out,
                              int64_t T, int64_t B, int32_t H, int32_t time_blocks, void* workspace,
                              int64_t workspace_bytes, gsb200_stream_t stream, gsb200_stream_t aux_stream);

/* The same LSTM layer for hosts that may not allocate device memory.  It has no counterpart in the reference.
 * Who needs it: an inference server that hands this library a fixed arena and forbids cudaMalloc after start-up,
 * a plugin running inside another framework's memory pool, a real-time basecalling loop where an allocation (and
 * the implicit device synchronisation it can bring) in the middle of a run is not acceptable.  Such a caller still
 * passes its inputs and outputs, but the kernel's scratch (the h exchange buffer and the per-CTA step counters)
 * comes from a device array built into the library, so this call performs no cudaMalloc / cudaFree and calls no
 * allocating library routine.
 * Limits: B <= 512 and H <= 512; anything larger returns GSB200_ERR_UNSUPPORTED with a message on stderr (use
 * gsb200_lstm_layer_fp8 with your own scratch instead).  Cost: about 513 KiB of device memory on every GPU that
 * loads the library, held until the process exits.
 * The first call on each device looks up the array's device address (with that device current); make that first
 * call before starting any stream capture.  All calls on a device share the one array: the step counters are
 * cleared at the start of every call, the h buffer keeps the previous call's contents (it is fully rewritten
 * before it is read), and two calls that overlap on the GPU -- different streams, or different host threads --
 * would race on it, so keep calls on one device in order. */
int32_t gsb200_lstm_layer_fp8_static(const void* ih, int64_t ld_ih, const uint8_t* w_hh, int64_t ld_w,
                                     const float* s_hh, const float* bias, const uint8_t* h0, const void* c0,
                                     void* h_out, uint8_t* h8_out, void* c_last, int64_t T, int64_t B, int32_t H,
                                     int32_t reverse, gsb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GIGASLOP_B200_H_ */
