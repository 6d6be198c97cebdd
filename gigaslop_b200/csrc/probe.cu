// Measurement utility: how fast does this GPU's tensor core retire tcgen05.mma of the kinds the GEMM family uses?
// One CTA per SM; one thread issues `mmas` instructions (M = 128, N = 128 or 256, K = 32 bytes, kind::i8 or
// kind::f8f6f4) back to back into two alternating TMEM accumulators, walking shared-memory operand tiles the way a
// weight-stationary main loop does (A over 4 tiles x 4 K slices, B over 4 K blocks x 4 K slices), commits and waits
// (bounded).  Nothing is loaded from global memory: the operands are a fixed finite pattern written once, so the time
// is the tensor pipe's alone.  The caller times the launch with CUDA events (ops = 2 * 128 * N * 32 * mmas * CTAs)
// and gets each CTA's SM-clock count for the issue window back, from which MACs per clock and SM follow.
#include <atomic>

#include "capi_internal.h"
#include "ptx.cuh"

namespace gsb {

#ifndef PROBE_M
#define PROBE_M 128   // rows of the probe's MMAs (an experiment build may set 64)
#endif
constexpr int PROBE_THREADS = 128;
constexpr int PROBE_A_BYTES = 4 * 128 * 128;        // 4 A tiles of 128 rows x 128 K-bytes
constexpr int PROBE_B_BYTES = 4 * 256 * 128;        // 4 K blocks of up to 256 rows x 128 K-bytes
constexpr int PROBE_SMEM = PROBE_A_BYTES + PROBE_B_BYTES + 2048;   // 194 KiB
static_assert(PROBE_SMEM <= 227 * 1024, "shared memory budget");

template <int N, int KIND>   // KIND 0: kind::i8 (s8 x s8 -> s32), 1: kind::f8f6f4 (e4m3 x e4m3 -> f32)
__global__ void __launch_bounds__(PROBE_THREADS, 1) tensor_peak_probe_kernel(long long* clocks, int mmas) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abort_word;
  const AbortFlag abort_flag{smem_u32(&abort_word)};
  const int warp = threadIdx.x >> 5;
  // finite, non-trivial operand bytes (small int8 values; as E4M3 they are small normal / subnormal numbers)
  for (int i = threadIdx.x; i < (PROBE_A_BYTES + PROBE_B_BYTES) / 4; i += PROBE_THREADS)
    reinterpret_cast<uint32_t*>(smem)[i] = 0x01010101u * (uint32_t)((i * 7 + (i >> 5)) & 31);
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag.set(0); fence_mbar_init(); }
  if (warp == 1) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    const uint32_t a0 = smem_u32(smem), b0 = smem_u32(smem + PROBE_A_BYTES);
    constexpr uint32_t idesc = KIND == 0 ? umma_idesc(2, 1, 1, PROBE_M, N) : umma_idesc(1, 0, 0, PROBE_M, N);
    const long long t0 = clock64();
    for (int r = 0; r < mmas; ++r) {
      const int kk = r & 3, kb = (r >> 2) & 3, tile = (r >> 4) & 3;
      const uint64_t ad = umma_smem_desc_sw128(a0 + tile * (128 * 128)) + 2 * kk;
      const uint64_t bd = umma_smem_desc_sw128(b0 + kb * (N * 128)) + 2 * kk;
      const uint32_t d = tm + ((r >> 4) & 1) * N;          // a new accumulator every 16 MMAs (K = 512), two in turn
      if constexpr (KIND == 0) umma_i8(d, ad, bd, idesc, (r & 15) != 0);
      else umma_f8(d, ad, bd, idesc, (r & 15) != 0);
    }
    umma_commit(&bar);
    const long long t1 = clock64();
    const bool ok = mbar_wait(&bar, 0, abort_flag, ST_TIMEOUT_MMA, 0xB00, spin_budget());
    const long long t2 = clock64();
    clocks[blockIdx.x * 2 + 0] = t1 - t0;                  // the issuing thread's loop
    clocks[blockIdx.x * 2 + 1] = ok ? t2 - t0 : -1;        // until the last MMA has retired
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

int32_t launch_tensor_peak_probe(int kind, int n, int mmas, long long* clocks, int* ctas_out, cudaStream_t st) {
  if (!clocks || mmas <= 0 || mmas > (1 << 24) || (kind != 0 && kind != 1) || (n != 128 && n != 256)) return GSB200_ERR_BAD_ARG;
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;
  static std::atomic<int> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return GSB200_ERR_DEVICE;
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(tensor_peak_probe_kernel<128, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tensor_peak_probe_kernel<256, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tensor_peak_probe_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(tensor_peak_probe_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(probe)");
    attr_done[dev].store(1, std::memory_order_release);
  }
  const int ctas = sm_count_physical();
  if (ctas_out) *ctas_out = ctas;
  if (kind == 0 && n == 128) tensor_peak_probe_kernel<128, 0><<<ctas, PROBE_THREADS, PROBE_SMEM, st>>>(clocks, mmas);
  else if (kind == 0) tensor_peak_probe_kernel<256, 0><<<ctas, PROBE_THREADS, PROBE_SMEM, st>>>(clocks, mmas);
  else if (n == 128) tensor_peak_probe_kernel<128, 1><<<ctas, PROBE_THREADS, PROBE_SMEM, st>>>(clocks, mmas);
  else tensor_peak_probe_kernel<256, 1><<<ctas, PROBE_THREADS, PROBE_SMEM, st>>>(clocks, mmas);
  return cuda_status(cudaGetLastError(), "tensor peak probe launch");
}

}  // namespace gsb
