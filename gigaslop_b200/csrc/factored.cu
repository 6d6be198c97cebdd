// One step of the reference's low-rank ("factored") LSTM cell on the tensor core:
//     gates[B,4H] = hh_down[B,K_hh] . up_hh[4H,K_hh]^T + x_down[B,R] . up_ih[4H,R]^T + b_hh + b_ih    (fp16 operands)
// followed by the hard-sigmoid / hard-tanh gate math of fly/rdna_fp8_factored_lstm.py:275-326.  The two
// up-projections are one K = K_hh + R contraction whose A and W k-blocks come from two tensors each.
// CTA = 128 batch rows x 32 hidden units (gate columns i|f|g|o x 32 -> UMMA N = 128), one tile per CTA.
#include <cuda_fp8.h>

#include <atomic>

#include "capi_internal.h"
#include "ptx.cuh"

namespace gsb {

constexpr int FS_THREADS = 256;
constexpr int FS_ROWS = 128, FS_HS = 32, FS_NCOL = 128;
constexpr int FS_MAX_KB = 6;                                   // (K_hh + R) * 2 bytes <= 768
constexpr int FS_KB_BYTES = FS_ROWS * 128;
constexpr int FS_SMEM_A = 0;
constexpr int FS_SMEM_W = FS_MAX_KB * FS_KB_BYTES;
constexpr int FS_SMEM_BIAS = 2 * FS_MAX_KB * FS_KB_BYTES;
constexpr int FS_SMEM_BAR = FS_SMEM_BIAS + 512;
constexpr int FS_SMEM_BYTES = FS_SMEM_BAR + 64 + 1024;

struct FacStepParams {
  int B, H, kb_hh, kb_ih;            // k-blocks (64 fp16 each) of the hidden / input part
  const float* bias_hh; const float* bias_ih;
  float* c; uint8_t* h_out;
};

__global__ void __launch_bounds__(FS_THREADS, 1)
factored_lstm_step_kernel(const __grid_constant__ CUtensorMap tm_hh, const __grid_constant__ CUtensorMap tm_xd,
                          const __grid_constant__ CUtensorMap tm_uhh, const __grid_constant__ CUtensorMap tm_uih,
                          const FacStepParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_s = smem + FS_SMEM_A;
  uint8_t* w_s = smem + FS_SMEM_W;
  float* bias_s = reinterpret_cast<float*>(smem + FS_SMEM_BIAS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FS_SMEM_BAR);
  uint64_t* full = bars; uint64_t* mma_done = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slices = p.H / FS_HS;
  const int row0 = (blockIdx.x / slices) * FS_ROWS, hid0 = (blockIdx.x % slices) * FS_HS;
  const int kbs = p.kb_hh + p.kb_ih;

  if (tid == 0) {
    mbar_init(full, 1); mbar_init(mma_done, 1); abort_flag.set(0); fence_mbar_init();
    prefetch_tmap(&tm_hh); prefetch_tmap(&tm_xd); prefetch_tmap(&tm_uhh); prefetch_tmap(&tm_uih);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, FS_NCOL); tmem_relinquish(); }
  if (tid < FS_NCOL) {
    const int n = (tid >> 5) * p.H + hid0 + (tid & 31);
    bias_s[tid] = (p.bias_hh ? __ldg(p.bias_hh + n) : 0.f) + (p.bias_ih ? __ldg(p.bias_ih + n) : 0.f);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();          // bound of every wait below, fetched once

  if (tid == 0) {
    mbar_arrive_expect_tx(full, kbs * 2 * FS_KB_BYTES);
    for (int kb = 0; kb < kbs; ++kb) {
      const bool hh = kb < p.kb_hh;
      const int k0 = (hh ? kb : kb - p.kb_hh) * 64;                       // fp16 element offset inside its tensor
      tma_load_2d(a_s + kb * FS_KB_BYTES, hh ? &tm_hh : &tm_xd, full, k0, row0);
#pragma unroll
      for (int g = 0; g < 4; ++g)
        tma_load_2d(w_s + kb * FS_KB_BYTES + g * (FS_HS * 128), hh ? &tm_uhh : &tm_uih, full, k0, g * p.H + hid0);
    }
    if (mbar_wait(full, 0, abort_flag, ST_TIMEOUT_LSTM, 0x40, budget)) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(1, 0, 0, FS_ROWS, FS_NCOL);   // f16 x f16 -> f32
      for (int kb = 0; kb < kbs; ++kb) {
        const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(a_s + kb * FS_KB_BYTES));
        const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(w_s + kb * FS_KB_BYTES));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
      }
      umma_commit(mma_done);
    }
  }
  const int q = warp & 3, half = warp >> 2;
  const int row = row0 + q * 32 + lane;
  const bool row_ok = row < p.B;
  const size_t off = (size_t)row * p.H + hid0 + half * 16;
  float c[16];
  if (row_ok) {
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p.c + off + j);
      c[j] = v.x; c[j + 1] = v.y; c[j + 2] = v.z; c[j + 3] = v.w;
    }
  }
  const bool ok = __all_sync(0xffffffffu, mbar_wait(mma_done, 0, abort_flag, ST_TIMEOUT_LSTM, 0x50, budget));
  if (ok) {
    tc_fence_after();
    uint32_t acc[4][16];
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
    for (int g = 0; g < 4; ++g) tmem_ld_32x32b_x16(t_row + g * FS_HS + half * 16, acc[g]);
    tmem_ld_wait(acc[0], acc[1], acc[2], acc[3]);
    if (row_ok) {
      float hv[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int col = half * 16 + j;
        const float gi = __uint_as_float(acc[0][j]) + bias_s[col];
        const float gf = __uint_as_float(acc[1][j]) + bias_s[FS_HS + col];
        const float gg = __uint_as_float(acc[2][j]) + bias_s[2 * FS_HS + col];
        const float go = __uint_as_float(acc[3][j]) + bias_s[3 * FS_HS + col];
        const float ia = fminf(fmaxf(fmaf(gi, 0.2f, 0.5f), 0.f), 1.f);
        const float fa = fminf(fmaxf(fmaf(gf, 0.2f, 0.5f), 0.f), 1.f);
        const float ga = fminf(fmaxf(gg, -1.f), 1.f);
        const float oa = fminf(fmaxf(fmaf(go, 0.2f, 0.5f), 0.f), 1.f);
        const float cn = fa * c[j] + ia * ga;
        c[j] = cn;
        hv[j] = oa * tanhf(cn);
      }
#pragma unroll
      for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(p.c + off + j) = make_float4(c[j], c[j + 1], c[j + 2], c[j + 3]);
      uint32_t w8[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i] * 448.f, hv[4 * i + 1] * 448.f), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i + 2] * 448.f, hv[4 * i + 3] * 448.f), __NV_SATFINITE, __NV_E4M3);
        w8[i] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(p.h_out + off) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, FS_NCOL); }
}

static bool fs_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return tmap_2d(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, rows, cols, cols, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

int32_t launch_factored_lstm_step(uint8_t* h_out, float* c, const __half* hh_down, const __half* up_hh,
                                  const float* bias_hh, const __half* x_down, const __half* up_ih, const float* bias_ih,
                                  long long B, int H, int K_hh, int R, cudaStream_t st) {
  if (B == 0) return GSB200_OK;
  if (B < 0 || !h_out || !c || !hh_down || !up_hh || !x_down || !up_ih) return GSB200_ERR_BAD_ARG;
  if (H <= 0 || H % FS_HS != 0 || K_hh <= 0 || R <= 0 || K_hh % 64 != 0 || R % 64 != 0 || (K_hh + R) / 64 > FS_MAX_KB)
    return GSB200_ERR_UNSUPPORTED;
  const uintptr_t al = reinterpret_cast<uintptr_t>(h_out) | reinterpret_cast<uintptr_t>(c) |
                       reinterpret_cast<uintptr_t>(hh_down) | reinterpret_cast<uintptr_t>(up_hh) |
                       reinterpret_cast<uintptr_t>(x_down) | reinterpret_cast<uintptr_t>(up_ih);
  if (al & 15) return GSB200_ERR_BAD_ARG;
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;
  const long long grid = ((B + FS_ROWS - 1) / FS_ROWS) * (H / FS_HS);
  if (grid > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  static std::atomic<int> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return GSB200_ERR_DEVICE;
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(factored_lstm_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FS_SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(factored step)");
    attr_done[dev].store(1, std::memory_order_release);
  }
  // the four maps depend only on pointers and shapes: a caller stepping through time with the same buffers gets
  // them from the per-thread table after the first step
  CUtensorMap t_hh, t_xd, t_uhh, t_uih;
  if (!fs_map(&t_hh, hh_down, (uint64_t)B, (uint64_t)K_hh, FS_ROWS) || !fs_map(&t_xd, x_down, (uint64_t)B, (uint64_t)R, FS_ROWS) ||
      !fs_map(&t_uhh, up_hh, (uint64_t)4 * H, (uint64_t)K_hh, FS_HS) || !fs_map(&t_uih, up_ih, (uint64_t)4 * H, (uint64_t)R, FS_HS))
    return GSB200_ERR_BAD_ARG;
  FacStepParams p{};
  p.B = (int)B; p.H = H; p.kb_hh = K_hh / 64; p.kb_ih = R / 64;
  p.bias_hh = bias_hh; p.bias_ih = bias_ih; p.c = c; p.h_out = h_out;
  factored_lstm_step_kernel<<<(unsigned)grid, FS_THREADS, FS_SMEM_BYTES, st>>>(t_hh, t_xd, t_uhh, t_uih, p);
  return cuda_status(cudaGetLastError(), "factored lstm step launch");
}

}  // namespace gsb
