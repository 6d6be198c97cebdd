// Recurrent half of the LSTM layer: T sequential steps
//     gates[b, 4H] = ih[t, b, 4H] + (h_{t-1} . W_hh^T) * (s_hh[n] / 448) + bias[n]      (gate blocks i | f | g | o)
//     c_t = sigmoid(f) * c_{t-1} + sigmoid(i) * tanh(g);   h_t = sigmoid(o) * tanh(c_t)
// in ONE persistent cooperative kernel (the reference replays two launches per step from a graph,
// fly/bench_factored_lstm.py:106-121).  `ih` is the hoisted input projection for all timesteps (an FP8 GEMM of
// this library); h feeds the recurrent GEMM as E4M3 at the fixed scale 1/448 (the reference's convention for a
// value bounded by 1, fly/rdna_fp8_factored_lstm.py:321-326); c and the emitted h are fp16.
//
// Decomposition: CTA (g, s) owns 128 batch rows (row group g) x 32 hidden units (slice s) = 128 gate columns.
// Its W_hh slice (128 rows x H bytes) stays in shared memory for the whole layer, c_t stays in registers.
// Batch rows are independent, so only the H/32 CTAs of a row group exchange data: each step every CTA
// writes its 128 x 32 piece of h_t (E4M3) to a double-buffered global scratch and bumps its step counter;
// the others poll the counters (bounded), pull the full 128 x H tile into 128B-swizzled shared memory and
// run 128 x 128 x H on the tensor core (tcgen05 kind::f8f6f4, fp32 accumulators in TMEM).  The next step's ih tile
// is prefetched by TMA while the current step computes.  The step is latency-bound (0.3 us of tensor time).
#include <cooperative_groups.h>
#include <cuda_fp8.h>

#include <atomic>

#include "capi_internal.h"
#include "ptx.cuh"

namespace gsb {

#ifdef GSB200_LSTM_PROF
// Tuning aid (never in the shipped library): SM clock stamps of one step of CTA 0, threads 0 and 128.
__device__ long long g_lstm_prof[2][16];
#define LPROF(slot) do { if (blockIdx.x == 0 && s == 100 && (tid == 0 || tid == 128)) g_lstm_prof[tid == 128][slot] = clock64(); } while (0)
#define LPROF2(who, slot) do { if (blockIdx.x == 0 && (s == 100 || s == 101)) g_lstm_prof[who][(slot) + 8 * (s - 100)] = clock64(); } while (0)
#else
#define LPROF(slot) do { } while (0)
#define LPROF2(who, slot) do { } while (0)
#endif

constexpr int LSTM_THREADS = 256;            // 8 warps: all load / do gate math; warp 0 lane 0 also issues TMA + MMA
constexpr int LSTMC_MMA_TID = 128;           // cluster kernel: the thread (lane 0 of warp 4) that issues the MMAs
constexpr int LSTMC_IH_TID = 0;              // cluster kernel: the thread that issues the TMA loads of the ih tiles (on a thread of warp 7 the step is 12 % slower)
constexpr int LSTM_ROWS = 128;               // batch rows per CTA (UMMA M)
constexpr int LSTM_HS = 32;                  // hidden units per CTA
constexpr int LSTM_NCOL = 4 * LSTM_HS;       // gate columns per CTA (UMMA N)
constexpr int LSTM_MAX_KB = 4;               // H <= 512
constexpr int LSTM_PULLS = LSTM_ROWS * LSTM_MAX_KB * 8 / LSTM_THREADS;   // 16-byte pieces of h per thread and step (at most)
constexpr int LSTM_KB_BYTES = LSTM_ROWS * 128;                 // one 128-byte K block of a 128-row operand tile
constexpr int LSTM_IH_BYTES = LSTM_ROWS * LSTM_NCOL * 2;       // 32 KiB: four 128 x 32 fp16 boxes
constexpr int LSTM_SMEM_W = 0;
constexpr int LSTM_SMEM_H = LSTM_SMEM_W + LSTM_MAX_KB * LSTM_KB_BYTES;
constexpr int LSTM_SMEM_IH = LSTM_SMEM_H + LSTM_MAX_KB * LSTM_KB_BYTES;
constexpr int LSTM_SMEM_SC = LSTM_SMEM_IH + 2 * LSTM_IH_BYTES;   // 128 scales + 128 biases (fp32)
constexpr int LSTM_SMEM_BAR = LSTM_SMEM_SC + 1024;
constexpr int LSTM_SMEM_USED = LSTM_SMEM_BAR + 128;
constexpr int LSTM_SMEM_BYTES = LSTM_SMEM_USED + 1024;           // + alignment slack
static_assert(LSTM_SMEM_BYTES > 116 * 1024, "one CTA per SM");

struct LstmParams {
  int T, B, H;
  int reverse;                 // 1: iterate t = T-1 .. 0
  int k_blocks;                // ceil(H / 128)
  int slices;                  // H / 32
  const float* s_hh;           // [4H] per-channel scales of W_hh
  const float* bias;           // [4H] or null (b_ih + b_hh)
  const uint8_t* h0;           // [B, H] E4M3 at scale 1/448, or null (zeros)
  const __half* c0;            // [B, H] or null (zeros)
  __half* h_out;               // [T*B, H] fp16, row = t*B + b, or null
  uint8_t* h8_out;             // [T*B, H] E4M3 at scale 1/448 (input of the next layer's projection), or null
  __half* c_last;              // [B, H] final cell state, or null
  uint8_t* hbuf;               // scratch: [2][B][H] E4M3, h of the previous / current step
  unsigned int* flags;         // scratch: [row groups][slices] step counters, zero at launch
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Gate functions on the hardware tanh (one special-function instruction each, relative error about 2^-11):
// sigmoid(x) = 0.5 + 0.5 * tanh(x / 2).
__device__ __forceinline__ float tanh_f(float x) { return tanh_approx(x); }
__device__ __forceinline__ float sigmoid_f(float x) { return fmaf(0.5f, tanh_approx(0.5f * x), 0.5f); }

__global__ void __launch_bounds__(LSTM_THREADS, 1)
lstm_recurrent_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_ih,
                      const LstmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_s = smem + LSTM_SMEM_W;
  uint8_t* h_s = smem + LSTM_SMEM_H;
  uint8_t* ih_s = smem + LSTM_SMEM_IH;
  float* sc_s = reinterpret_cast<float*>(smem + LSTM_SMEM_SC);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LSTM_SMEM_BAR);
  uint64_t* w_full = bars;               // W slice landed
  uint64_t* ih_full = bars + 1;          // [2] ih tile of a step landed
  uint64_t* mma_done = bars + 3;         // accumulator of this step complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x / p.slices;        // row group
  const int slc = blockIdx.x % p.slices;        // hidden slice
  const int row0 = grp * LSTM_ROWS;
  const int hid0 = slc * LSTM_HS;
  const int H = p.H, B = p.B;

  if (tid == 0) {
    mbar_init(w_full, 1); mbar_init(&ih_full[0], 1); mbar_init(&ih_full[1], 1); mbar_init(mma_done, 1);
    abort_flag.set(0);
    fence_mbar_init();
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_ih);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, LSTM_NCOL); tmem_relinquish(); }
  // per-channel scale (with the 1/448 of h folded in) and bias of this CTA's 128 gate columns
  if (tid < LSTM_NCOL) {
    const int n = (tid >> 5) * H + hid0 + (tid & 31);
    sc_s[tid] = __ldg(p.s_hh + n) * (1.0f / 448.0f);
    sc_s[LSTM_NCOL + tid] = p.bias ? __ldg(p.bias + n) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();          // bound of every wait below, fetched once

  auto step_t = [&](int s) { return p.reverse ? p.T - 1 - s : s; };
  auto issue_ih = [&](int s) {   // one thread: TMA the four gate boxes of step s into buffer s & 1
    uint8_t* dst = ih_s + (s & 1) * LSTM_IH_BYTES;
    mbar_arrive_expect_tx(&ih_full[s & 1], LSTM_IH_BYTES);
    const int r = step_t(s) * B + row0;
#pragma unroll
    for (int g = 0; g < 4; ++g) tma_load_2d(dst + g * (LSTM_ROWS * LSTM_HS * 2), &tm_ih, &ih_full[s & 1], g * H + hid0, r);
  };
  if (tid == 0) {
    mbar_arrive_expect_tx(w_full, p.k_blocks * LSTM_KB_BYTES);
    for (int kb = 0; kb < p.k_blocks; ++kb)
#pragma unroll
      for (int g = 0; g < 4; ++g)
        tma_load_2d(w_s + kb * LSTM_KB_BYTES + g * (LSTM_HS * 128), &tm_w, w_full, kb * 128, g * H + hid0);
    issue_ih(0);
    if (p.T > 1) issue_ih(1);
  }

  // this thread's part of the tile: row (TMEM lane) q*32 + lane, hidden units half*16 .. +15 of the slice
  const int q = warp & 3, half = warp >> 2;
  const int r_loc = q * 32 + lane;
  const int row = row0 + r_loc;
  const bool row_ok = row < B;
  float c[16];
#pragma unroll
  for (int j = 0; j < 16; ++j)
    c[j] = (p.c0 && row_ok) ? __half2float(p.c0[(long long)row * H + hid0 + half * 16 + j]) : 0.f;

  bool ok = mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_LSTM, 0x10, budget);
  unsigned int* my_flags = p.flags + grp * p.slices;
  // The 16-byte pieces of the 128 x H tile of h this thread moves every step.  Piece i of a thread is row
  // (tid / 8) + 32 * (i % 4), 16-byte chunk tid % 8 of K block i / 4: eight neighbouring threads read one 128-byte
  // line, and both offsets are one per-thread base plus constants known at compile time (no per-piece state).
  const int pull_r = tid >> 3, pull_ck = tid & 7;
  const int pull_dst0 = pull_r * 128 + ((pull_ck ^ (pull_r & 7)) << 4);         // + kb * LSTM_KB_BYTES + j * 32 * 128
  const long long pull_src0 = (long long)(row0 + pull_r) * H + pull_ck * 16;     // + kb * 128 + j * 32 * H

  for (int s = 0; s < p.T; ++s) {
    // ---- 1. wait until every slice of this row group has published h_{s-1} -----------------------------
    const uint8_t* h_prev = (s == 0) ? p.h0 : p.hbuf + (size_t)((s + 1) & 1) * B * H;
    if (s > 0 && tid < p.slices) {
      long long t0 = clock64();
      while (ld_acquire_gpu(my_flags + tid) < (unsigned int)s) {
        if (abort_flag.get()) break;
        if (clock64() - t0 > budget) {
          abort_flag.set(1);
          atomicOr(&g_status[0], ST_TIMEOUT_LSTM);
          g_status[1] = (unsigned int)s;
          break;
        }
      }
    }
    __syncthreads();
    if (abort_flag.get() || !ok) break;
    // ---- 2. pull the 128 x H tile of h_{s-1} into the swizzled K-major operand layout ------------------
    // All of a thread's loads are issued before the first store, so their L2 latencies overlap (one after the
    // other they were the longest part of the step).
    {
      uint4 v[LSTM_PULLS];
#pragma unroll
      for (int i = 0; i < LSTM_PULLS; ++i) {
        const int kb = i >> 2, j = i & 3;
        v[i] = make_uint4(0, 0, 0, 0);
        if (h_prev && kb < p.k_blocks && row0 + pull_r + 32 * j < B && kb * 128 + pull_ck * 16 < H)
          v[i] = __ldcg(reinterpret_cast<const uint4*>(h_prev + pull_src0 + (long long)j * 32 * H + kb * 128));
      }
#pragma unroll
      for (int i = 0; i < LSTM_PULLS; ++i) {
        const int kb = i >> 2, j = i & 3;
        if (kb < p.k_blocks) *reinterpret_cast<uint4*>(h_s + pull_dst0 + kb * LSTM_KB_BYTES + j * (32 * 128)) = v[i];
      }
    }
    fence_proxy_async_smem();
    __syncthreads();
    // ---- 3. gates += h . W^T on the tensor core ----------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(1, 0, 0, LSTM_ROWS, LSTM_NCOL);
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        const uint64_t a_desc = umma_smem_desc_sw128(smem_u32(h_s + kb * LSTM_KB_BYTES));
        const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(w_s + kb * LSTM_KB_BYTES));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
      }
      umma_commit(mma_done);
    }
    // ---- 4. gate math on this thread's row ---------------------------------------------------------------
    ok = mbar_wait(&ih_full[s & 1], (s >> 1) & 1, abort_flag, ST_TIMEOUT_LSTM, 0x20, budget) &&
         mbar_wait(mma_done, s & 1, abort_flag, ST_TIMEOUT_LSTM, 0x30, budget);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      tc_fence_after();
      uint32_t acc[4][16];
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld_32x32b_x16(t_row + g * LSTM_HS + half * 16, acc[g]);
      tmem_ld_wait(acc[0], acc[1], acc[2], acc[3]);
      const uint8_t* ihb = ih_s + (s & 1) * LSTM_IH_BYTES;
      float hv[16];
#pragma unroll
      for (int j0 = 0; j0 < 16; j0 += 8) {
        float pre[4][8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          // 8 fp16 of gate g: one 16-byte piece of this row in the 64-byte-swizzled box
          const int piece = half * 2 + (j0 >> 3);
          const uint4 raw = *reinterpret_cast<const uint4*>(ihb + g * (LSTM_ROWS * LSTM_HS * 2) + r_loc * 64 +
                                                            ((piece ^ ((r_loc >> 1) & 3)) << 4));
          const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h2[i]);
            const int col = g * LSTM_HS + half * 16 + j0 + 2 * i;
            pre[g][2 * i] = fmaf(__uint_as_float(acc[g][j0 + 2 * i]), sc_s[col], f.x + sc_s[LSTM_NCOL + col]);
            pre[g][2 * i + 1] = fmaf(__uint_as_float(acc[g][j0 + 2 * i + 1]), sc_s[col + 1], f.y + sc_s[LSTM_NCOL + col + 1]);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float ig = sigmoid_f(pre[0][i]), fg = sigmoid_f(pre[1][i]), gg = tanh_f(pre[2][i]), og = sigmoid_f(pre[3][i]);
          const float cn = fmaf(fg, c[j0 + i], ig * gg);
          hv[j0 + i] = og * tanh_f(cn);
          c[j0 + i] = __half2float(__float2half_rn(cn));        // the cell state is carried in fp16
        }
      }
      uint32_t w8[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i] * 448.f, hv[4 * i + 1] * 448.f), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i + 2] * 448.f, hv[4 * i + 3] * 448.f), __NV_SATFINITE, __NV_E4M3);
        w8[i] = lo | (hi << 16);
      }
      const size_t off = (size_t)row * H + hid0 + half * 16;
      // the piece the other slices wait for goes out first
      if (row_ok) *reinterpret_cast<uint4*>(p.hbuf + (size_t)(s & 1) * B * H + off) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
      tc_fence_before();
      __syncthreads();
      // ---- 5. publish: one release store after the CTA barrier covers every thread's piece (the release is
      //         cumulative over what the barrier ordered before it); then prefetch the ih tile two steps ahead
      if (tid == 0) {
        st_release_gpu(my_flags + slc, (unsigned int)(s + 1));
        if (s + 2 < p.T) issue_ih(s + 2);
      }
      // ---- 6. the layer's outputs, off the other slices' critical path -------------------------------------
      if (row_ok) {
        const size_t toff = (size_t)step_t(s) * B * H + off;
        if (p.h8_out) *reinterpret_cast<uint4*>(p.h8_out + toff) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
        if (p.h_out) {
          uint32_t w16[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w16[i] = pack_half2(hv[2 * i], hv[2 * i + 1]);
          *reinterpret_cast<uint4*>(p.h_out + toff) = make_uint4(w16[0], w16[1], w16[2], w16[3]);
          *reinterpret_cast<uint4*>(p.h_out + toff + 8) = make_uint4(w16[4], w16[5], w16[6], w16[7]);
        }
      }
    } else {
      tc_fence_before();
      __syncthreads();
    }
    if (!ok || abort_flag.get()) break;
  }

  if (p.c_last && row_ok) {
#pragma unroll
    for (int j = 0; j < 16; ++j) p.c_last[(long long)row * H + hid0 + half * 16 + j] = __float2half_rn(c[j]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, LSTM_NCOL); }
}

// ---- cluster form: the slices of a row group exchange h through distributed shared memory ---------------------
// Same decomposition and arithmetic as lstm_recurrent_kernel, but the H/32 CTAs of a row group form ONE thread-block
// cluster.  The h operand tile is kept unswizzled as [16-byte K chunk][row][16 bytes], in which the 128 x 32 piece a
// CTA produces is one contiguous 4 KiB block: the CTA stages it in its own shared memory and sends it to every CTA of
// the cluster with one bulk copy each (cp.async.bulk shared::cta -> shared::cluster), whose bytes complete the
// destination's mbarrier.  No global scratch, no flag polling, no L2 round trips on the step's critical path, and no
// cooperative launch (row groups do not depend on one another).
// Operand tile and staging block are double-buffered: h_t goes to buffer t & 1 while the MMAs of step t read buffer
// (t + 1) & 1; a CTA can only reach the copies of step t + 2 after every CTA has finished the MMAs of step t + 1.
// Built for H <= 384 (W 48 KiB + 2 x 48 KiB h + 2 x 32 KiB ih); larger H uses the kernel above.
constexpr int LSTMC_MAX_KB = 3;
constexpr int LSTMC_SMEM_W = 0;
constexpr int LSTMC_SMEM_H = LSTMC_SMEM_W + LSTMC_MAX_KB * LSTM_KB_BYTES;
constexpr int LSTMC_HBUF = LSTMC_MAX_KB * LSTM_KB_BYTES;
constexpr int LSTMC_SMEM_IH = LSTMC_SMEM_H + 2 * LSTMC_HBUF;
constexpr int LSTMC_PIECE = LSTM_ROWS * LSTM_HS;                    // 4 KiB: one CTA's piece of h (two 16-byte K chunks x 128 rows)
constexpr int LSTMC_CHUNK = LSTM_ROWS * 16;                         // 2 KiB: one 16-byte K chunk of all 128 rows
constexpr int LSTMC_SMEM_STG = LSTMC_SMEM_IH + 2 * LSTM_IH_BYTES;   // [2] staging of this CTA's piece
constexpr int LSTMC_SMEM_SC = LSTMC_SMEM_STG + 2 * LSTMC_PIECE;
constexpr int LSTMC_SMEM_BAR = LSTMC_SMEM_SC + 1024;
constexpr int LSTMC_SMEM_USED = LSTMC_SMEM_BAR + 128;
constexpr int LSTMC_SMEM_BYTES = LSTMC_SMEM_USED + 1024;
static_assert(LSTMC_SMEM_BYTES <= 227 * 1024 && LSTMC_SMEM_BYTES > 116 * 1024, "one CTA per SM");

__global__ void __launch_bounds__(LSTM_THREADS, 1)
lstm_cluster_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_ih,
                    const LstmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // every CTA of the cluster must place its tiles at the same shared-memory offsets: the window offset of the
  // dynamic allocation is the same for all CTAs of a kernel, so the aligned base is too
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_s = smem + LSTMC_SMEM_W;
  uint8_t* h_s = smem + LSTMC_SMEM_H;
  uint8_t* ih_s = smem + LSTMC_SMEM_IH;
  float* sc_s = reinterpret_cast<float*>(smem + LSTMC_SMEM_SC);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + LSTMC_SMEM_BAR);
  uint64_t* w_full = bars;               // W slice landed
  uint64_t* ih_full = bars + 1;          // [2] ih tile of a step landed
  uint64_t* mma_done = bars + 3;         // accumulator of this step complete
  uint64_t* h_ready = bars + 4;          // [2] every slice's piece of h has landed in this CTA's buffer (bytes counted)
  uint8_t* stg_s = smem + LSTMC_SMEM_STG;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x / p.slices;        // row group = cluster
  const int slc = blockIdx.x % p.slices;        // hidden slice = rank inside the cluster
  const int row0 = grp * LSTM_ROWS;
  const int hid0 = slc * LSTM_HS;
  const int H = p.H, B = p.B;

  if (tid == 0) {
    mbar_init(w_full, 1); mbar_init(&ih_full[0], 1); mbar_init(&ih_full[1], 1); mbar_init(mma_done, 1);
    mbar_init(&h_ready[0], 1); mbar_init(&h_ready[1], 1);
    // arm the first use of each buffer: h_0 arrives in buffer 0 (if there is a step 1), h_1 in buffer 1
    if (p.T > 1) mbar_arrive_expect_tx(&h_ready[0], p.slices * LSTMC_PIECE);
    if (p.T > 2) mbar_arrive_expect_tx(&h_ready[1], p.slices * LSTMC_PIECE);
    abort_flag.set(0);
    fence_mbar_init();
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_ih);
  }
  if (warp == 0) { tmem_alloc(tmem_slot, LSTM_NCOL); tmem_relinquish(); }
  if (tid < LSTM_NCOL) {
    const int n = (tid >> 5) * H + hid0 + (tid & 31);
    sc_s[tid] = __ldg(p.s_hh + n) * (1.0f / 448.0f);
    sc_s[LSTM_NCOL + tid] = p.bias ? __ldg(p.bias + n) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();                    // every CTA's barriers exist before anyone sends to them
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();
  const bool rank_ok = cluster_ctarank() == (uint32_t)slc;

  auto step_t = [&](int s) { return p.reverse ? p.T - 1 - s : s; };
  auto issue_ih = [&](int s) {
    uint8_t* dst = ih_s + (s & 1) * LSTM_IH_BYTES;
    mbar_arrive_expect_tx(&ih_full[s & 1], LSTM_IH_BYTES);
    const int r = step_t(s) * B + row0;
#pragma unroll
    for (int g = 0; g < 4; ++g) tma_load_2d(dst + g * (LSTM_ROWS * LSTM_HS * 2), &tm_ih, &ih_full[s & 1], g * H + hid0, r);
  };
  if (tid == 0) {
    mbar_arrive_expect_tx(w_full, p.k_blocks * LSTM_KB_BYTES);
    for (int kb = 0; kb < p.k_blocks; ++kb)
#pragma unroll
      for (int g = 0; g < 4; ++g)
        tma_load_2d(w_s + kb * LSTM_KB_BYTES + g * (LSTM_HS * 128), &tm_w, w_full, kb * 128, g * H + hid0);
    issue_ih(0);
    if (p.T > 1) issue_ih(1);
  }

  const int q = warp & 3, half = warp >> 2;
  const int r_loc = q * 32 + lane;
  const int row = row0 + r_loc;
  const bool row_ok = row < B;
  float c[16];
#pragma unroll
  for (int j = 0; j < 16; ++j)
    c[j] = (p.c0 && row_ok) ? __half2float(p.c0[(long long)row * H + hid0 + half * 16 + j]) : 0.f;
  const int my_col = hid0 + half * 16;   // this thread's 16 hidden units = K chunk `half` of the CTA's piece

  bool ok = mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_LSTM, 0x10, budget) && rank_ok;
  if (!rank_ok && tid == 0) { abort_flag.set(1); atomicOr(&g_status[0], ST_TIMEOUT_LSTM); g_status[1] = 0x50; }

  // ---- step 0 reads h_0 (or zeros) from buffer 1, staged by this CTA's own threads -------------------------
  {
    const int chunks_per_row = H >> 4;
    for (int id = tid; id < LSTM_ROWS * chunks_per_row; id += LSTM_THREADS) {
      const int r = id / chunks_per_row, cc = id % chunks_per_row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (p.h0 && row0 + r < B) v = __ldcg(reinterpret_cast<const uint4*>(p.h0 + (size_t)(row0 + r) * H + cc * 16));
      *reinterpret_cast<uint4*>(h_s + LSTMC_HBUF + cc * LSTMC_CHUNK + r * 16) = v;
    }
  }
  fence_proxy_async_smem();
  __syncthreads();

  // The MMAs of step s + 1 are issued inside step s by one thread of warp 4, as soon as that warp has put out its
  // output stores (they take ~1700 clocks to get into the store queue: 768 partial-line writes per CTA and step; the
  // tile of h_s is complete ~1300 clocks after the CTA barrier, so the wait for it hides behind them).  Warp 0 has
  // the bulk copies and the next TMA loads to issue; everything of the next step waits for these MMAs.
  // Descriptors are built once; a K step adds a constant to the start-address field.
  const uint64_t a_base[2] = {umma_smem_desc_kchunks(smem_u32(h_s), LSTMC_CHUNK),
                              umma_smem_desc_kchunks(smem_u32(h_s + LSTMC_HBUF), LSTMC_CHUNK)};
  const uint64_t b_base = umma_smem_desc_sw128(smem_u32(w_s));
  auto issue_mmas = [&](int buf) {                    // one thread: gates += (tile of h in buffer `buf`) . W^T
    constexpr uint32_t idesc = umma_idesc(1, 0, 0, LSTM_ROWS, LSTM_NCOL);
    const uint64_t a_desc = buf ? a_base[1] : a_base[0];
    const int ksteps = H >> 5;                        // 32 bytes of K per MMA
    tc_fence_after();
    for (int ks = 0; ks < ksteps; ++ks)
      umma_f8(tmem_base, a_desc + (uint64_t)(ks * (2 * LSTMC_CHUNK >> 4)),
              b_base + (uint64_t)((ks >> 2) * (LSTM_KB_BYTES >> 4) + 2 * (ks & 3)), idesc, ks != 0);
    umma_commit(mma_done);
  };
  if (tid == LSTMC_MMA_TID && ok && p.T > 0) issue_mmas(1);       // step 0 reads buffer 1

  for (int s = 0; s < p.T; ++s) {
    if (abort_flag.get() || !ok) break;
    LPROF(0);
    // ---- 2. gate math on this thread's row ---------------------------------------------------------------------
    ok = mbar_wait(&ih_full[s & 1], (s >> 1) & 1, abort_flag, ST_TIMEOUT_LSTM, 0x20, budget) &&
         mbar_wait(mma_done, s & 1, abort_flag, ST_TIMEOUT_LSTM, 0x30, budget);
    ok = __all_sync(0xffffffffu, ok);
    LPROF(1);
    if (ok) {
      tc_fence_after();
      uint32_t acc[4][16];
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
      for (int g = 0; g < 4; ++g) tmem_ld_32x32b_x16(t_row + g * LSTM_HS + half * 16, acc[g]);
      tmem_ld_wait(acc[0], acc[1], acc[2], acc[3]);
      LPROF(2);
      const uint8_t* ihb = ih_s + (s & 1) * LSTM_IH_BYTES;
      float hv[16];
#pragma unroll
      for (int j0 = 0; j0 < 16; j0 += 8) {
        float pre[4][8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int piece = half * 2 + (j0 >> 3);
          const uint4 raw = *reinterpret_cast<const uint4*>(ihb + g * (LSTM_ROWS * LSTM_HS * 2) + r_loc * 64 +
                                                            ((piece ^ ((r_loc >> 1) & 3)) << 4));
          const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h2[i]);
            const int col = g * LSTM_HS + half * 16 + j0 + 2 * i;
            pre[g][2 * i] = fmaf(__uint_as_float(acc[g][j0 + 2 * i]), sc_s[col], f.x + sc_s[LSTM_NCOL + col]);
            pre[g][2 * i + 1] = fmaf(__uint_as_float(acc[g][j0 + 2 * i + 1]), sc_s[col + 1], f.y + sc_s[LSTM_NCOL + col + 1]);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float ig = sigmoid_f(pre[0][i]), fg = sigmoid_f(pre[1][i]), gg = tanh_f(pre[2][i]), og = sigmoid_f(pre[3][i]);
          const float cn = fmaf(fg, c[j0 + i], ig * gg);
          hv[j0 + i] = og * tanh_f(cn);
          c[j0 + i] = __half2float(__float2half_rn(cn));
        }
      }
      uint32_t w8[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i] * 448.f, hv[4 * i + 1] * 448.f), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(hv[4 * i + 2] * 448.f, hv[4 * i + 3] * 448.f), __NV_SATFINITE, __NV_E4M3);
        w8[i] = lo | (hi << 16);
      }
      LPROF(3);
      // ---- 3. stage this CTA's piece of h_s (K chunk `half`, 16 bytes per row) ...
      uint8_t* stg = stg_s + (s & 1) * LSTMC_PIECE;
      *reinterpret_cast<uint4*>(stg + half * LSTMC_CHUNK + r_loc * 16) =
          row_ok ? make_uint4(w8[0], w8[1], w8[2], w8[3]) : make_uint4(0, 0, 0, 0);
      LPROF(4);
      fence_proxy_async_smem();                       // generic-proxy staging stores before the bulk copies read them
      tc_fence_before();
      __syncthreads();
      LPROF(5);
      // ---- 4. ... and send it into buffer s & 1 of every CTA of the row group, one bulk copy each --------------
      if (s + 1 < p.T && tid < p.slices) {
        const uint32_t dst = mapa_shared(smem_u32(h_s + (s & 1) * LSTMC_HBUF + slc * LSTMC_PIECE), (uint32_t)tid);
        bulk_copy_to_cluster(dst, stg, LSTMC_PIECE, mapa_shared(smem_u32(&h_ready[s & 1]), (uint32_t)tid));
      }
      LPROF(6);
      if (tid == LSTMC_IH_TID && s + 2 < p.T) issue_ih(s + 2);
      LPROF(7);
      // ---- 5. the layer's outputs ------------------------------------------------------------------------------------
      if (row_ok) {
        const size_t toff = (size_t)step_t(s) * B * H + (size_t)row * H + my_col;
        if (p.h8_out) *reinterpret_cast<uint4*>(p.h8_out + toff) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
        if (p.h_out) {
          uint32_t w16[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) w16[i] = pack_half2(hv[2 * i], hv[2 * i + 1]);
          *reinterpret_cast<uint4*>(p.h_out + toff) = make_uint4(w16[0], w16[1], w16[2], w16[3]);
          *reinterpret_cast<uint4*>(p.h_out + toff + 8) = make_uint4(w16[4], w16[5], w16[6], w16[7]);
        }
      }
      LPROF(8);
      // ---- 6. the next step's MMAs: the tile of h_s (buffer s & 1) is complete once every slice has arrived ---------
      if (tid == LSTMC_MMA_TID && s + 1 < p.T) {
        const bool got = mbar_wait_cluster(&h_ready[s & 1], (s >> 1) & 1, abort_flag, ST_TIMEOUT_LSTM, 0x40, budget);
        LPROF(9);
        if (got) {
          // arm this buffer's next use: h_{s+2} arrives in it if there is a step s + 3
          if (s + 3 < p.T) mbar_arrive_expect_tx(&h_ready[s & 1], p.slices * LSTMC_PIECE);
          issue_mmas(s & 1);
          LPROF(10);
        } else {
          abort_flag.set(1);
        }
      }
    } else {
      tc_fence_before();
      __syncthreads();
    }
  }

  if (p.c_last && row_ok) {
#pragma unroll
    for (int j = 0; j < 16; ++j) p.c_last[(long long)row * H + my_col + j] = __float2half_rn(c[j]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, LSTM_NCOL); }
  cluster_sync_all();                    // nobody leaves while another CTA of the cluster may still store into it
}

// ---- cluster form, two interleaved 64-row halves per CTA -----------------------------------------------------------
// The step of the kernel above is one serial chain per CTA: gather h (about 1700 clocks from the CTA barrier until the
// last slice's piece has crossed the cluster), issue the MMAs (about 100 clocks each), wait for the accumulator, gate
// math, stage, barrier, send.  Nothing in it is busy for long; it is latency end to end.  Here a CTA still owns 128
// batch rows x 32 hidden units, but as TWO independent halves of 64 rows that take turns: while the pieces of one half
// are in flight and its MMAs run, the eight compute warps do the gate math of the other half.  What makes that work:
//  * M = 64 MMAs.  Their accumulator sits in the lower 16 lanes of each TMEM lane quarter, and tcgen05.ld.16x256b hands
//    a warp 16 rows x 16 columns as 2 rows x (2 + 2) column pairs per thread, so all 256 compute threads share a half's
//    64 x 128 gate values evenly: 8 cells each (2 rows x 4 hidden units, all four gates of a cell in one thread).
//  * a ninth warp that only issues MMAs (and the TMA loads of the ih tiles), so no compute thread ever waits for a gather;
//  * one mbarrier per (half, buffer, source slice): the K step that reads slice k's 32 bytes of h is issued as soon as
//    that slice's piece has landed, so the MMA issue overlaps the gather instead of following it.
// The outputs leave through the staged images of the piece (whole 32-byte / 64-byte runs per row, written by
// cooperating threads) instead of 16-byte slivers per row.  Arithmetic per cell is that of the other two kernels (a test
// holds all three to the same bytes).
constexpr int L64_ROWS = 64;
constexpr int L2_THREADS = 320;                                // 8 compute warps + the MMA warp + the send warp
constexpr int L2_COMPUTE = 256;
constexpr int L64_CHUNK = L64_ROWS * 16;                       // one 16-byte K chunk of all 64 rows
constexpr int L64_PIECE = L64_ROWS * LSTM_HS;                  // 2 KiB: this CTA's piece of a half's h (two chunks = one K step)
constexpr int L64_HBUF = LSTMC_MAX_KB * 8 * L64_CHUNK;         // 24 KiB: a half's 64 x 384 tile of h as 24 chunks
constexpr int L64_IH_GATE = L64_ROWS * LSTM_HS * 2;            // 4 KiB: one gate's 64 x 32 fp16 box
constexpr int L64_IH_BYTES = 4 * L64_IH_GATE;                  // 16 KiB
constexpr int L64_H16_BYTES = L64_ROWS * LSTM_HS * 2;          // 4 KiB: fp16 image of the piece (layer output)
constexpr int L2_MAX_SLICES = 12;
constexpr int L2_SMEM_W = 0;
constexpr int L2_SMEM_H = L2_SMEM_W + LSTMC_MAX_KB * LSTM_KB_BYTES;          // [half][buffer]
constexpr int L2_SMEM_IH = L2_SMEM_H + 4 * L64_HBUF;                         // [half][buffer]
constexpr int L2_SMEM_STG = L2_SMEM_IH + 4 * L64_IH_BYTES;                   // [half][buffer]
constexpr int L2_SMEM_H16 = L2_SMEM_STG + 4 * L64_PIECE;                     // [half]
constexpr int L2_SMEM_SC = L2_SMEM_H16 + 2 * L64_H16_BYTES;
constexpr int L2_SMEM_BAR = L2_SMEM_SC + 1024;
constexpr int L2_SMEM_USED = L2_SMEM_BAR + 512;
constexpr int L2_SMEM_BYTES = L2_SMEM_USED + 1024;
static_assert(L2_SMEM_BYTES <= 227 * 1024 && L2_SMEM_BYTES > 116 * 1024, "one CTA per SM");

__global__ void __launch_bounds__(L2_THREADS, 1)
lstm_cluster2_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_ih,
                     const LstmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_s = smem + L2_SMEM_W;
  uint8_t* h_s = smem + L2_SMEM_H;                 // + (2 * half + buffer) * L64_HBUF
  uint8_t* ih_s = smem + L2_SMEM_IH;               // + (2 * half + buffer) * L64_IH_BYTES
  uint8_t* stg_s = smem + L2_SMEM_STG;             // + (2 * half + buffer) * L64_PIECE
  uint8_t* h16_base = smem + L2_SMEM_H16;          // + half * L64_H16_BYTES
  float* sc_s = reinterpret_cast<float*>(smem + L2_SMEM_SC);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L2_SMEM_BAR);
  uint64_t* w_full = bars;
  uint64_t* ih_full = bars + 1;                    // [half][buffer]
  uint64_t* mma_done = bars + 5;                   // [half]
  uint64_t* staged = bars + 7;                     // [half]: this CTA's piece of the step's h is staged, the send warp may copy it
  uint64_t* h_ready = bars + 9;                    // [half][buffer]: every slice's piece of h has landed (bytes counted)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x / p.slices;        // 128-row group = cluster
  const int slc = blockIdx.x % p.slices;        // hidden slice = rank inside the cluster
  const int row0 = grp * LSTM_ROWS;
  const int hid0 = slc * LSTM_HS;
  const int H = p.H, B = p.B;
  const int halves = (B - row0 > L64_ROWS) ? 2 : 1;     // the last group may have rows for one half only

  if (tid == 0) {
    mbar_init(w_full, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&ih_full[i], 1);
    mbar_init(&mma_done[0], 1); mbar_init(&mma_done[1], 1);
    mbar_init(&staged[0], 1); mbar_init(&staged[1], 1);
    for (int i = 0; i < 4; ++i) mbar_init(&h_ready[i], 1);
    // arm the first use of each tile barrier: h_0 arrives in buffer 0 (if there is a step 1), h_1 in buffer 1
    for (int hf = 0; hf < halves; ++hf) {
      if (p.T > 1) mbar_arrive_expect_tx(&h_ready[2 * hf + 0], p.slices * L64_PIECE);
      if (p.T > 2) mbar_arrive_expect_tx(&h_ready[2 * hf + 1], p.slices * L64_PIECE);
    }
    abort_flag.set(0);
    fence_mbar_init();
    prefetch_tmap(&tm_w); prefetch_tmap(&tm_ih);
  }
  if (warp == 8) { tmem_alloc(tmem_slot, 2 * LSTM_NCOL); tmem_relinquish(); }
  if (tid < LSTM_NCOL) {
    const int n = (tid >> 5) * H + hid0 + (tid & 31);
    sc_s[tid] = __ldg(p.s_hh + n) * (1.0f / 448.0f);
    sc_s[LSTM_NCOL + tid] = p.bias ? __ldg(p.bias + n) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();                    // every CTA's barriers exist (and are armed) before anyone sends to them
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();
  const bool rank_ok = cluster_ctarank() == (uint32_t)slc;
  if (!rank_ok && tid == 0) { abort_flag.set(1); atomicOr(&g_status[0], ST_TIMEOUT_LSTM); g_status[1] = 0x50; }

  auto step_t = [&](int s) { return p.reverse ? p.T - 1 - s : s; };
  auto issue_ih = [&](int hf, int s) {     // one thread: TMA the four gate boxes of step s, half hf
    const int ib = 2 * hf + (s & 1);
    uint8_t* dst = ih_s + ib * L64_IH_BYTES;
    mbar_arrive_expect_tx(&ih_full[ib], L64_IH_BYTES);
    const int r = step_t(s) * B + row0 + hf * L64_ROWS;
#pragma unroll
    for (int g = 0; g < 4; ++g) tma_load_2d(dst + g * L64_IH_GATE, &tm_ih, &ih_full[ib], g * H + hid0, r);
  };

  // this thread's cells of a half (compute warps): rows ra and ra + 8, hidden units u0 + {0, 1} and u0 + 8 + {0, 1} of
  // the slice; cell index = 4 * k + 2 * rowsel + j, the order in which tcgen05.ld.16x256b.x2 delivers them
  const int q = warp & 3, hh = (warp >> 2) & 1;
  const int ra = 16 * q + (lane >> 2);
  const int u0 = 16 * hh + 2 * (lane & 3);
  auto cell_row = [&](int i) { return ra + ((i >> 1) & 1) * 8; };
  auto cell_u = [&](int i) { return u0 + (i >> 2) * 8 + (i & 1); };
  float c[2][8];
  float2 sc2[4][2], bi2[4][2];
  int ih_off[4];
  if (warp >= 8) {
    if (warp == 8 && lane == 0) {         // W slice and the first two ih tiles of each half
      mbar_arrive_expect_tx(w_full, p.k_blocks * LSTM_KB_BYTES);
      for (int kb = 0; kb < p.k_blocks; ++kb)
#pragma unroll
        for (int g = 0; g < 4; ++g)
          tma_load_2d(w_s + kb * LSTM_KB_BYTES + g * (LSTM_HS * 128), &tm_w, w_full, kb * 128, g * H + hid0);
      for (int hf = 0; hf < halves; ++hf) { issue_ih(hf, 0); if (p.T > 1) issue_ih(hf, 1); }
    }
  } else {
#pragma unroll
    for (int hf = 0; hf < 2; ++hf)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int row = row0 + hf * L64_ROWS + cell_row(i);
        c[hf][i] = (p.c0 && row < B) ? __half2float(p.c0[(long long)row * H + hid0 + cell_u(i)]) : 0.f;
      }
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int col = g * LSTM_HS + u0 + 8 * k;
        sc2[g][k] = make_float2(sc_s[col], sc_s[col + 1]);
        bi2[g][k] = make_float2(sc_s[LSTM_NCOL + col], sc_s[LSTM_NCOL + col + 1]);
      }
    // byte offsets of this thread's ih values inside a gate box (64-byte swizzle): one half2 per (k, rowsel)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = i >> 1, row = ra + (i & 1) * 8;
      ih_off[i] = row * 64 + (((2 * hh + k) ^ ((row >> 1) & 3)) << 4) + 4 * (lane & 3);
    }
    // step 0 reads h_0 (or zeros) from buffer 1 of each half, staged by this CTA's own compute threads
    const int chunks_per_row = H >> 4;
    for (int hf = 0; hf < halves; ++hf)
      for (int id = tid; id < L64_ROWS * chunks_per_row; id += L2_COMPUTE) {
        const int r = id / chunks_per_row, cc = id % chunks_per_row;
        const int row = row0 + hf * L64_ROWS + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p.h0 && row < B) v = __ldcg(reinterpret_cast<const uint4*>(p.h0 + (size_t)row * H + cc * 16));
        *reinterpret_cast<uint4*>(h_s + (2 * hf + 1) * L64_HBUF + cc * L64_CHUNK + r * 16) = v;
      }
    fence_proxy_async_smem();
  }
  __syncthreads();                       // h_0 is staged before the first MMAs read it

  if (warp == 8) {
    // ------------------------------ MMA warp: one thread issues the MMAs and the ih loads ------------------------------
    if (lane == 0) {
      bool ok = rank_ok && mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_LSTM, 0x10, budget);
      constexpr uint32_t idesc = umma_idesc(1, 0, 0, L64_ROWS, LSTM_NCOL);
      const uint64_t b_base = umma_smem_desc_sw128(smem_u32(w_s));
      const int ksteps = H >> 5;                        // one K step (32 bytes of h) per hidden slice
      for (int s = 0; ok && s < p.T; ++s) {
        for (int hf = 0; ok && hf < halves; ++hf) {
          // gates of step s, half hf: h_{s-1} sits in buffer (s + 1) & 1 (step 0: h_0 or zeros, staged locally)
          LPROF2(1, 4 * hf + 0);
          const int hb = 2 * hf + ((s + 1) & 1);
          const uint64_t a_desc = umma_smem_desc_kchunks(smem_u32(h_s + hb * L64_HBUF), L64_CHUNK);
          if (s > 0) {
            if (!mbar_wait_cluster(&h_ready[hb], (uint32_t)((s - 1) >> 1) & 1u, abort_flag, ST_TIMEOUT_LSTM, 0x40, budget)) { ok = false; break; }
            if (s + 2 < p.T) mbar_arrive_expect_tx(&h_ready[hb], p.slices * L64_PIECE);   // its next use: h_{s+1}, read by step s + 2
          }
          for (int ks = 0; ks < ksteps; ++ks) {
            if (ks == 0) { tc_fence_after(); LPROF2(1, 4 * hf + 1); }
            umma_f8(tmem_base + hf * LSTM_NCOL, a_desc + (uint64_t)(ks * (2 * L64_CHUNK >> 4)),
                    b_base + (uint64_t)((ks >> 2) * (LSTM_KB_BYTES >> 4) + 2 * (ks & 3)), idesc, ks != 0);
          }
          if (!ok) break;
          LPROF2(1, 4 * hf + 2);
          umma_commit(&mma_done[hf]);
          // every slice's piece of h_{s-1} is here, our own included, and that one was sent after the compute warps'
          // barrier of step s - 1: the ih tile of step s - 1 has been consumed and its buffer can take step s + 1
          if (s > 0 && s + 1 < p.T) issue_ih(hf, s + 1);
          LPROF2(1, 4 * hf + 3);
        }
      }
      if (!ok) abort_flag.set(1);
    }
  } else if (warp == 9) {
    // ------------------------------ send warp: the all-gather of h through distributed shared memory ------------------------------
    // One bulk copy per destination CTA (lane = destination rank), issued when the compute warps have staged the piece;
    // its bytes are counted by the destination's barrier of that half and buffer.  A copy costs the SM about 220 clocks,
    // one after the other whichever threads issue them: twelve are ~2700 clocks, which no compute warp pays here and
    // which pass while the other half is computed.
    for (int s = 0; s + 1 < p.T; ++s) {
      bool ok = true;
      for (int hf = 0; hf < halves; ++hf) {
        const int ib = 2 * hf + (s & 1);
        ok = mbar_wait(&staged[hf], s & 1, abort_flag, ST_TIMEOUT_LSTM, 0x60, budget);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane < p.slices) {
          const uint32_t dst = mapa_shared(smem_u32(h_s + ib * L64_HBUF + slc * L64_PIECE), (uint32_t)lane);
          bulk_copy_to_cluster(dst, stg_s + ib * L64_PIECE, L64_PIECE, mapa_shared(smem_u32(&h_ready[ib]), (uint32_t)lane));
        }
      }
      if (!ok) break;
    }
  } else {
    // ------------------------------ compute warps: the halves take turns ------------------------------
    bool ok = true;
    for (int s = 0; ok && s < p.T; ++s) {
      for (int hf = 0; hf < halves; ++hf) {
        if (tid == 0) LPROF2(0, 4 * hf + 0);
        const int ib = 2 * hf + (s & 1);
        bool mine = mbar_wait(&ih_full[ib], (s >> 1) & 1, abort_flag, ST_TIMEOUT_LSTM, 0x20, budget) &&
                    mbar_wait(&mma_done[hf], s & 1, abort_flag, ST_TIMEOUT_LSTM, 0x30, budget);
        mine = __all_sync(0xffffffffu, mine);
        uint8_t* stg = stg_s + ib * L64_PIECE;
        uint8_t* h16_s = h16_base + (halves == 2 ? hf : (s & 1)) * L64_H16_BYTES;
        if (tid == 0) LPROF2(0, 4 * hf + 1);
        if (mine) {
          tc_fence_after();
          uint32_t acc[4][8];
          const uint32_t t_row = tmem_base + hf * LSTM_NCOL + ((uint32_t)(q * 32) << 16);
#pragma unroll
          for (int g = 0; g < 4; ++g) tmem_ld_16x256b_x2(t_row + g * LSTM_HS + hh * 16, acc[g]);
          tmem_ld_wait(acc[0], acc[1], acc[2], acc[3]);
          const uint8_t* ihb = ih_s + ib * L64_IH_BYTES;
          float hv[8];
#pragma unroll
          for (int kr = 0; kr < 4; ++kr) {              // (k, rowsel): two adjacent hidden units of one row
            const int k = kr >> 1, rs = kr & 1;
            float pre[4][2];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(ihb + g * L64_IH_GATE + ih_off[kr]));
              pre[g][0] = fmaf(__uint_as_float(acc[g][4 * k + 2 * rs + 0]), sc2[g][k].x, f.x + bi2[g][k].x);
              pre[g][1] = fmaf(__uint_as_float(acc[g][4 * k + 2 * rs + 1]), sc2[g][k].y, f.y + bi2[g][k].y);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int i = 4 * k + 2 * rs + j;
              const float ig = sigmoid_f(pre[0][j]), fg = sigmoid_f(pre[1][j]), gg = tanh_f(pre[2][j]), og = sigmoid_f(pre[3][j]);
              const float cprev = hf ? c[1][i] : c[0][i];
              const float cn = fmaf(fg, cprev, ig * gg);
              hv[i] = og * tanh_f(cn);
              const float cr = __half2float(__float2half_rn(cn));       // the cell state is carried in fp16
              if (hf) c[1][i] = cr; else c[0][i] = cr;
            }
          }
          // stage this thread's bytes of the CTA's piece: chunk hh, 2 bytes per (k, rowsel); rows past the batch as zeros
#pragma unroll
          for (int kr = 0; kr < 4; ++kr) {
            const int k = kr >> 1, rs = kr & 1, i = 4 * k + 2 * rs;
            const int r = ra + rs * 8;
            const bool live = row0 + hf * L64_ROWS + r < B;
            const uint32_t b2 = live ? (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(hv[i] * 448.f, hv[i + 1] * 448.f), __NV_SATFINITE, __NV_E4M3) : 0u;
            *reinterpret_cast<uint16_t*>(stg + hh * L64_CHUNK + r * 16 + 8 * k + 2 * (lane & 3)) = (uint16_t)b2;
            if (p.h_out)    // fp16 image: rows of 64 bytes, 16-byte pieces XOR-swizzled by the row pair like the ih boxes
              *reinterpret_cast<uint32_t*>(h16_s + r * 64 + (((2 * hh + k) ^ ((r >> 1) & 3)) << 4) + 4 * (lane & 3)) = pack_half2(hv[i], hv[i + 1]);
          }
          fence_proxy_async_smem();                     // the staging stores before the bulk copies read them
        }
        tc_fence_before();
        if (tid == 0) LPROF2(0, 4 * hf + 2);
        ok = named_barrier_and(1, L2_COMPUTE, mine) != 0;    // all compute warps go on, or all leave, together
        if (tid == 0) LPROF2(0, 4 * hf + 3);
        if (!ok) break;
        if (tid == 0 && s + 1 < p.T) mbar_arrive(&staged[hf]);   // the send warp takes it from here
        // the layer's outputs, from the staged images: whole 32-byte (E4M3) / 64-byte (fp16) runs per row
        const size_t trow = (size_t)step_t(s) * B + row0 + hf * L64_ROWS;
        const int rows_live = B - (row0 + hf * L64_ROWS);
        if (p.h8_out && tid >= 128) {                   // (the upper compute warps: the lower ones issue the sends)
          const int r = (tid - 128) >> 1, cch = tid & 1;
          if (r < rows_live)
            *reinterpret_cast<uint4*>(p.h8_out + (trow + r) * H + hid0 + 16 * cch) = *reinterpret_cast<const uint4*>(stg + cch * L64_CHUNK + r * 16);
        }
        if (p.h_out) {
          const int r = tid >> 2, pc = tid & 3;
          if (r < rows_live)
            *reinterpret_cast<uint4*>(p.h_out + (trow + r) * H + hid0 + 8 * pc) =
                *reinterpret_cast<const uint4*>(h16_s + r * 64 + ((pc ^ ((r >> 1) & 3)) << 4));
        }
      }
    }
    if (p.c_last) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = row0 + hf * L64_ROWS + cell_row(i);
          if (hf < halves && row < B) p.c_last[(long long)row * H + hid0 + cell_u(i)] = __float2half_rn(c[hf][i]);
        }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * LSTM_NCOL); }
  cluster_sync_all();                    // nobody leaves while another CTA of the cluster may still store into it
}

// ---- host -------------------------------------------------------------------------------------------------
size_t lstm_scratch_bytes(long long B, int H) {
  const size_t hbuf = ((size_t)2 * B * H + 255) & ~(size_t)255;
  const size_t flags = (size_t)((B + LSTM_ROWS - 1) / LSTM_ROWS) * (H / LSTM_HS) * sizeof(unsigned int);
  return hbuf + ((flags + 255) & ~(size_t)255);
}

int32_t launch_lstm_layer(const LstmLayerArgs& a, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (a.T == 0 || a.B == 0) return GSB200_OK;
  if (a.T < 0 || a.B < 0 || a.H <= 0 || a.H % LSTM_HS != 0 || a.H > LSTM_MAX_KB * 128) return GSB200_ERR_UNSUPPORTED;
  if (!a.ih || !a.w_hh || !a.s_hh || !scratch) return GSB200_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a.ih) & 15) || (reinterpret_cast<uintptr_t>(a.w_hh) & 15) ||
      (reinterpret_cast<uintptr_t>(scratch) & 255))
    return GSB200_ERR_BAD_ARG;
  if (a.ld_ih < 4 * a.H || a.ld_ih % 8 != 0 || a.H % 16 != 0) return GSB200_ERR_BAD_ARG;
  if ((a.h_out && (reinterpret_cast<uintptr_t>(a.h_out) & 15)) || (a.h8_out && (reinterpret_cast<uintptr_t>(a.h8_out) & 15)) ||
      (a.h0 && (reinterpret_cast<uintptr_t>(a.h0) & 15)))
    return GSB200_ERR_BAD_ARG;
  if ((long long)a.T * a.B > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  if (scratch_bytes < lstm_scratch_bytes(a.B, a.H)) return GSB200_ERR_BAD_ARG;
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;

  const int groups = (int)((a.B + LSTM_ROWS - 1) / LSTM_ROWS);
  const int slices = a.H / LSTM_HS;
  const int grid = groups * slices;
  // every CTA must be resident (they wait on one another); the grid is never capped, so the physical SM count
  // is what bounds it, not the cap a caller may have set for the GEMM grids
  if (grid > sm_count_physical()) return GSB200_ERR_UNSUPPORTED;

  static std::atomic<int> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return GSB200_ERR_DEVICE;
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(lstm_recurrent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LSTM_SMEM_BYTES);
    if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(lstm)");
    attr_done[dev].store(1, std::memory_order_release);
  }

  LstmParams p{};
  p.T = (int)a.T; p.B = (int)a.B; p.H = a.H; p.reverse = a.reverse ? 1 : 0;
  p.k_blocks = (a.H + 127) / 128; p.slices = slices;
  p.s_hh = a.s_hh; p.bias = a.bias; p.h0 = a.h0; p.c0 = a.c0;
  p.h_out = a.h_out; p.h8_out = a.h8_out; p.c_last = a.c_last;
  const size_t hbuf_bytes = ((size_t)2 * a.B * a.H + 255) & ~(size_t)255;
  p.hbuf = static_cast<uint8_t*>(scratch);
  p.flags = reinterpret_cast<unsigned int*>(static_cast<uint8_t*>(scratch) + hbuf_bytes);

  if (a.ld_w < a.H || a.ld_w % 16 != 0) return GSB200_ERR_BAD_ARG;
  CUtensorMap tw, tih;
  if (!tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w_hh, (uint64_t)4 * a.H, (uint64_t)a.H, (uint64_t)a.ld_w, 128,
               LSTM_HS, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !tmap_2d(&tih, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.ih, (uint64_t)a.T * a.B, (uint64_t)4 * a.H,
               (uint64_t)a.ld_ih, LSTM_HS, LSTM_ROWS, CU_TENSOR_MAP_SWIZZLE_64B))
    return GSB200_ERR_BAD_ARG;
  // Cluster forms first (h exchanged through distributed shared memory): H <= 384, the slices of a 128-row group in one
  // cluster of H / 32 CTAs (more than 8 needs the non-portable cluster size).  The default runs a CTA's rows as two
  // interleaved 64-row halves.  In the environment, GSB200_LSTM_ROWS128=1 selects the older cluster kernel (one
  // 128-row tile per CTA, a thread per row) and GSB200_LSTM_NO_CLUSTER=1 the cooperative kernel with global scratch; a
  // device that cannot host a cluster of that size falls back the same way.  What the device can host is asked once per
  // (device, kernel, cluster size); a refusal is reported on stderr once and only switches off that combination.
  static std::atomic<int> env_state{-1};
  int env = env_state.load(std::memory_order_relaxed);
  if (env < 0) {
    const char* e1 = getenv("GSB200_LSTM_NO_CLUSTER");
    const char* e2 = getenv("GSB200_LSTM_ROWS128");
    env = ((e1 && e1[0] == '1') ? 1 : 0) | ((e2 && e2[0] == '1') ? 2 : 0);
    env_state.store(env, std::memory_order_relaxed);
  }
  if (!(env & 1) && p.k_blocks <= LSTMC_MAX_KB && slices <= 16) {
    static std::atomic<int> cluster_state[2][64][17];       // [64-row form][device][cluster size]: 0 unknown, 1 usable, -1 not
    auto try_cluster = [&](bool rows64, int cgrid, const CUtensorMap& tih_k) -> bool {
      void (*kern)(const CUtensorMap, const CUtensorMap, const LstmParams) = rows64 ? lstm_cluster2_kernel : lstm_cluster_kernel;
      const int smem_bytes = rows64 ? L2_SMEM_BYTES : LSTMC_SMEM_BYTES;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(cgrid); cfg.blockDim = dim3(rows64 ? L2_THREADS : LSTM_THREADS);
      cfg.dynamicSmemBytes = smem_bytes; cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = slices; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      std::atomic<int>& slot = cluster_state[rows64 ? 1 : 0][dev][slices];
      int state = slot.load(std::memory_order_acquire);
      if (state == 0) {
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (ce == cudaSuccess && slices > 8) ce = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        int max_clusters = 0;
        if (ce == cudaSuccess) ce = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
        state = (ce == cudaSuccess && max_clusters >= 1) ? 1 : -1;
        if (getenv("GSB200_LSTM_VERBOSE"))
          fprintf(stderr, "gigaslop_b200: LSTM cluster form (%s), cluster of %d: %d clusters can be resident (%d CTAs asked)\n",
                  rows64 ? "two 64-row halves" : "128-row tile", slices, max_clusters, cgrid);
        if (state < 0) {
          cudaGetLastError();
          fprintf(stderr, "gigaslop_b200: device %d cannot host a cluster of %d LSTM CTAs (%s: %s)\n", dev, slices,
                  rows64 ? "two 64-row halves" : "128-row tile", ce == cudaSuccess ? "no active cluster fits" : cudaGetErrorName(ce));
        }
        slot.store(state, std::memory_order_release);
      }
      if (state != 1) return false;
      cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tw, tih_k, p);
      if (ce == cudaSuccess) return true;
      cudaGetLastError();
      fprintf(stderr, "gigaslop_b200: cluster launch of the LSTM layer failed (%s); trying the next form\n", cudaGetErrorName(ce));
      return false;
    };
    if (!(env & 2) && slices <= L2_MAX_SLICES) {          // two interleaved 64-row halves per CTA: ih boxes of 64 rows
      CUtensorMap tih64;
      if (tmap_2d(&tih64, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.ih, (uint64_t)a.T * a.B, (uint64_t)4 * a.H,
                  (uint64_t)a.ld_ih, LSTM_HS, L64_ROWS, CU_TENSOR_MAP_SWIZZLE_64B) &&
          try_cluster(true, grid, tih64))
        return GSB200_OK;
    }
    if (try_cluster(false, grid, tih)) return GSB200_OK;
  }
  // the cooperative kernel exchanges h through the scratch; its step counters start at zero
  cudaError_t e = cudaMemsetAsync(p.flags, 0, (size_t)grid * sizeof(unsigned int), st);
  if (e != cudaSuccess) return cuda_status(e, "lstm flags memset");
  void* args[3] = {&tw, &tih, &p};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(lstm_recurrent_kernel), dim3(grid), dim3(LSTM_THREADS), args,
                                  LSTM_SMEM_BYTES, st);
  return cuda_status(e, "lstm launch");
}

// ---- variant for callers that cannot allocate device memory ------------------------------------------------
// The h exchange buffer and the step counters live in a file-scope device array instead of caller scratch.
// Limits: B <= 512 and H <= 512 (the benchmark layer is B = 512, H = 384).  Every GPU that loads the library
// holds these ~513 KiB until the process exits.
constexpr long long LSTM_STATIC_MAX_B = 512;
constexpr int LSTM_STATIC_MAX_H = 512;
constexpr size_t LSTM_STATIC_BYTES = (size_t)2 * LSTM_STATIC_MAX_B * LSTM_STATIC_MAX_H + 1024;
static __device__ __align__(256) unsigned char g_lstm_static_scratch[LSTM_STATIC_BYTES];

// In host code the array's name is only a stand-in for the symbol, not a device address: the address a kernel
// can use comes from cudaGetSymbolAddress, looked up once per device with that device current.
static void* g_lstm_static_ptr[64];

int32_t launch_lstm_layer_static(const LstmLayerArgs& a, cudaStream_t st) {
  if (a.T == 0 || a.B == 0) return GSB200_OK;
  if (a.B > LSTM_STATIC_MAX_B || a.H > LSTM_STATIC_MAX_H || lstm_scratch_bytes(a.B, a.H) > LSTM_STATIC_BYTES) {
    fprintf(stderr, "gigaslop_b200: lstm_layer_fp8_static supports B <= %lld and H <= %d (got B = %lld, H = %d); "
                    "use gsb200_lstm_layer_fp8 with caller scratch for larger shapes\n",
            LSTM_STATIC_MAX_B, LSTM_STATIC_MAX_H, a.B, a.H);
    return GSB200_ERR_UNSUPPORTED;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return GSB200_ERR_DEVICE;
  if (!g_lstm_static_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_lstm_static_scratch);
    if (e != cudaSuccess || !ptr) return cuda_status(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "cudaGetSymbolAddress(lstm scratch)");
    g_lstm_static_ptr[dev] = ptr;
  }
  return launch_lstm_layer(a, g_lstm_static_ptr[dev], LSTM_STATIC_BYTES, st);
}

#ifdef GSB200_LSTM_PROF
}  // namespace gsb
extern "C" int gsb200_debug_lstm_prof(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, gsb::g_lstm_prof, sizeof(long long) * 32);
}
namespace gsb {
#endif

// ---- the whole stack behind one call ---------------------------------------------------------------------------
// Per layer: the hoisted input projection (FP8 GEMM over the T*B rows) and the persistent recurrence; layers
// alternate direction and hand each other h as E4M3 at the row scale 1/448.  With an auxiliary stream the
// recurrence of a layer is cut into `time_blocks` launches (the state crosses a cut exactly: h as the E4M3 bytes
// the kernel itself feeds back, c as the fp16 it carries), and as soon as a block of layer l is done the hoisted
// projection of layer l + 1 over the same timesteps runs on the auxiliary stream, on the SMs the recurrence
// leaves idle -- ordered by events only, no kernel waits for another kernel.
//
// Workspace: [ih 0][ih 1 (overlap only)][h8 0][h8 1][row scales = 1/448][c 0][c 1][layer scratch]
__global__ void fill_f32_kernel(float* dst, long long n, float v) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = v;
}

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t lstm_stack_workspace_bytes(long long T, long long B, int H, int overlap) {
  if (T <= 0 || B <= 0 || H <= 0) return 0;
  const size_t rows = (size_t)T * (size_t)B;
  return (overlap ? 2 : 1) * align256(rows * 4 * H * 2) + 2 * align256(rows * H) + align256(rows * 4) +
         2 * align256((size_t)B * H * 2) + align256(lstm_scratch_bytes(B, H));
}

int32_t launch_lstm_stack(const uint8_t* x, long long ldx, const float* sx, int C, const gsb200_lstm_layer_t* layers,
                          int n_layers, int reverse_first, __half* h_out, long long T, long long B, int H,
                          int time_blocks, void* ws, size_t ws_bytes, cudaStream_t st, cudaStream_t aux) {
  if (T == 0 || B == 0 || n_layers == 0) return GSB200_OK;
  if (!x || !sx || !layers || !h_out || !ws || T < 0 || B < 0 || n_layers < 0 || C <= 0) return GSB200_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return GSB200_ERR_BAD_ARG;
  if (H <= 0 || H % LSTM_HS != 0 || H > LSTM_MAX_KB * 128) return GSB200_ERR_UNSUPPORTED;
  if ((long long)T * B > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  for (int l = 0; l < n_layers; ++l)
    if (!layers[l].w_ih || !layers[l].s_ih || !layers[l].w_hh || !layers[l].s_hh) return GSB200_ERR_BAD_ARG;
  const bool overlap = aux != nullptr && aux != st && n_layers > 1;
  int nb = overlap ? (time_blocks > 0 ? time_blocks : 8) : 1;
  if (nb > T) nb = (int)T;
  if (ws_bytes < lstm_stack_workspace_bytes(T, B, H, overlap ? 1 : 0)) return GSB200_ERR_BAD_ARG;
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;

  const size_t rows = (size_t)T * (size_t)B;
  uint8_t* w = static_cast<uint8_t*>(ws);
  __half* ih[2];
  ih[0] = reinterpret_cast<__half*>(w); w += align256(rows * 4 * H * 2);
  ih[1] = ih[0];
  if (overlap) { ih[1] = reinterpret_cast<__half*>(w); w += align256(rows * 4 * H * 2); }
  uint8_t* h8[2];
  h8[0] = w; w += align256(rows * H);
  h8[1] = w; w += align256(rows * H);
  float* row_scale = reinterpret_cast<float*>(w); w += align256(rows * 4);
  __half* cst[2];
  cst[0] = reinterpret_cast<__half*>(w); w += align256((size_t)B * H * 2);
  cst[1] = reinterpret_cast<__half*>(w); w += align256((size_t)B * H * 2);
  void* scratch = w;
  const size_t scratch_bytes = align256(lstm_scratch_bytes(B, H));

  if (n_layers > 1) {
    const long long blocks = ((long long)rows + 255) / 256;
    fill_f32_kernel<<<(unsigned)blocks, 256, 0, st>>>(row_scale, (long long)rows, 1.0f / 448.0f);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_status(e, "lstm stack: row scale fill");
  }
  // hoisted projection of layer l over timesteps [t0, t1) on stream s, at most sm_cap CTAs (0 = all)
  auto project = [&](int l, long long t0, long long t1, cudaStream_t s, int sm_cap) -> int32_t {
    GemmArgs g{};
    g.kind = KIND_F8; g.epi = EPI_DEQUANT;
    if (l == 0) { g.A = x + (size_t)t0 * B * ldx; g.lda = ldx; g.scale_a = sx + (size_t)t0 * B; g.K = C; }
    else { g.A = h8[(l - 1) & 1] + (size_t)t0 * B * H; g.lda = H; g.scale_a = row_scale; g.K = H; }
    g.B0 = layers[l].w_ih; g.ldb = layers[l].ld_w_ih;
    g.C = ih[l & 1] + (size_t)t0 * B * 4 * H; g.ldc = 4 * H;
    g.scale_b0 = layers[l].s_ih;
    g.M = (t1 - t0) * B; g.N = 4 * H;
    g.sm_cap = sm_cap;
    return launch_gemm(g, s);
  };
  rc = project(0, 0, T, st, 0);
  if (rc != GSB200_OK) return rc;

  const int groups = (int)((B + LSTM_ROWS - 1) / LSTM_ROWS);
  const int lstm_ctas = groups * (H / LSTM_HS);
  int gemm_cap = sm_count_physical() - lstm_ctas;
  if (gemm_cap < 8) gemm_cap = 8;
  cudaError_t ce = cudaSuccess;
  for (int l = 0; l < n_layers; ++l) {
    const bool last = l == n_layers - 1;
    const bool rev = ((l % 2) == 0) == (reverse_first != 0);
    uint8_t* h8_l = h8[l & 1];
    for (int k = 0; k < nb; ++k) {
      // block k in processing order covers steps [s0, s1); in time that is [t0, t1)
      const long long s0 = T * k / nb, s1 = T * (k + 1) / nb;
      const long long t0 = rev ? T - s1 : s0, t1 = rev ? T - s0 : s1;
      LstmLayerArgs a{};
      a.ih = ih[l & 1] + (size_t)t0 * B * 4 * H; a.ld_ih = 4 * H;
      a.w_hh = layers[l].w_hh; a.ld_w = layers[l].ld_w_hh; a.s_hh = layers[l].s_hh; a.bias = layers[l].bias;
      if (k > 0) {                       // state at the cut: h of the step processed just before, c of the previous block
        const long long t_prev = rev ? t1 : t0 - 1;
        a.h0 = h8_l + (size_t)t_prev * B * H;
        a.c0 = cst[(k - 1) & 1];
      }
      a.h_out = last ? h_out + (size_t)t0 * B * H : nullptr;
      a.h8_out = h8_l + (size_t)t0 * B * H;
      a.c_last = k + 1 < nb ? cst[k & 1] : nullptr;
      a.T = t1 - t0; a.B = B; a.H = H; a.reverse = rev ? 1 : 0;
      rc = launch_lstm_layer(a, scratch, scratch_bytes, st);
      if (rc != GSB200_OK) return rc;
      if (overlap && !last) {
        cudaEvent_t ev;
        ce = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (ce != cudaSuccess) return cuda_status(ce, "lstm stack: event");
        ce = cudaEventRecord(ev, st);
        if (ce == cudaSuccess) ce = cudaStreamWaitEvent(aux, ev, 0);
        cudaEventDestroy(ev);            // released by the runtime once the recorded work has completed
        if (ce != cudaSuccess) return cuda_status(ce, "lstm stack: event");
        rc = project(l + 1, t0, t1, aux, gemm_cap);
        if (rc != GSB200_OK) return rc;
      }
    }
    if (!last) {
      if (overlap) {                     // the next layer starts when its whole projection is there
        cudaEvent_t ev;
        ce = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
        if (ce != cudaSuccess) return cuda_status(ce, "lstm stack: event");
        ce = cudaEventRecord(ev, aux);
        if (ce == cudaSuccess) ce = cudaStreamWaitEvent(st, ev, 0);
        cudaEventDestroy(ev);
        if (ce != cudaSuccess) return cuda_status(ce, "lstm stack: event");
      } else {
        rc = project(l + 1, 0, T, st, 0);
        if (rc != GSB200_OK) return rc;
      }
    }
  }
  return GSB200_OK;
}


}  // namespace gsb
