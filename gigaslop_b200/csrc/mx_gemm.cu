// Block-scaled MXFP8 GEMMs on tcgen05 kind::mxf8f6f4: both operands are E4M3 with one E8M0 scale per 32
// consecutive K elements (per row of A, per row of W), fp32 accumulation in TMEM, fp16 output.
//
//   plain : C[M,N]      = A . W^T                      (e.g. the down-projection fed by an MXFP8 activation)
//   dual  : C[M,N]      = silu(A . Wg^T) * (A . Wu^T)  (SwiGLU)
//
// Scale factors travel in the 128 x 4 tile order the tensor core consumes: for a matrix with R rows and
// K columns the byte for (row r, 32-block b) lives at
//     ((r / 128) * (K / 128) + b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4)
// (rows padded to 128, K a multiple of 128).  One such 512-byte tile is exactly what one 128-byte K stage of
// 128 rows needs; it is bulk-copied into shared memory next to the operand tiles and moved to TMEM with
// tcgen05.cp.32x128b.warpx4 by the MMA thread, in order with the MMAs that read it.  The instruction
// descriptor's scale ids select the byte (the 32-block inside the stage) for each K = 32 MMA.
//
// Tiles are 128 rows x 128 accumulator columns; two accumulator stages (256 TMEM columns) overlap the
// epilogue with the next tile; the scale factors use 12 further columns.  The dual form issues two N = 64
// MMAs per K step (gate -> columns 0..63, up -> 64..127) so each keeps its own scale tile.
//
// Two kernels.  K <= 512 runs the weight-stationary one further down (its comment explains why); anything else the
// streaming kernel described above.
#include "capi_internal.h"
#include "ptx.cuh"

namespace gsb {

constexpr int MX_BM = 128, MX_BN = 128, MX_BK = 128;
constexpr int MX_STAGES = 5;
constexpr int MX_A_BYTES = MX_BM * MX_BK;            // 16 KiB
constexpr int MX_B_BYTES = MX_BN * MX_BK;            // 16 KiB
constexpr int MX_SF_BYTES = 512;
constexpr int MX_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 4 * MX_SF_BYTES;   // A | B | SFA | SFB0 | SFB1 | pad  = 34 KiB
constexpr int MX_EPI_WARPS = 8, MX_FRONT_WARPS = 4;
constexpr int MX_THREADS = 32 * (MX_EPI_WARPS + MX_FRONT_WARPS);
constexpr int MX_OUT_BUF = 2048, MX_OUT_BUFS = 2;
constexpr int MX_SMEM_OUT = MX_STAGES * MX_STAGE_BYTES;
constexpr int MX_SMEM_BAR = MX_SMEM_OUT + MX_EPI_WARPS * MX_OUT_BUFS * MX_OUT_BUF;
constexpr int MX_SMEM_BYTES = MX_SMEM_BAR + 256 + 1024;
constexpr int MX_TMEM_COLS = 512;                    // power of two >= 256 + 12
constexpr int MX_SF_COL = 256;                       // SFA at +0, SFB0 at +4, SFB1 at +8
static_assert(MX_SMEM_BYTES > 116 * 1024 && MX_SMEM_BYTES <= 227 * 1024, "one CTA per SM");

struct MxParams {
  int M, N, K;
  int m_blocks, n_blocks, k_blocks;
  int n_groups;                      // weight-stationary kernel: row-block groups (grid = n_groups * n_blocks)
  const uint8_t* sfa; const uint8_t* sfb0; const uint8_t* sfb1;    // tiled scale factors
};

// Shared-memory descriptor of one scale tile for tcgen05.cp: 32 rows of 16 bytes, unswizzled K-major, 8-row
// groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;       // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                // descriptor version
  return d;                              // layout type 0: no swizzle
}

template <bool DUAL>
__global__ void __launch_bounds__(MX_THREADS, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
               const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_c, const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_base = smem + MX_SMEM_OUT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + MX_SMEM_BAR);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + MX_STAGES;
  uint64_t* acc_full = bars + 2 * MX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int OUT_COLS = DUAL ? MX_BN / 2 : MX_BN;          // output columns per tile
  const long long num_tiles = (long long)p.m_blocks * p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MX_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], MX_EPI_WARPS); }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_b0); prefetch_tmap(&tm_b1); prefetch_tmap(&tm_c);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, MX_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const long long budget = spin_budget();          // bound of every wait below, fetched once

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = (int)(t / p.n_blocks), n_blk = (int)(t % p.n_blocks);
        const int m0 = m_blk * MX_BM, n0 = n_blk * OUT_COLS;
        const int nb128 = n0 / 128;                              // scale tile row block of W
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, 0x600 | s, budget)) { ok = false; break; }
          uint8_t* st = smem + s * MX_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], MX_A_BYTES + MX_B_BYTES + (DUAL ? 3 : 2) * MX_SF_BYTES);
          tma_load_2d(st, &tm_a, &full_bar[s], kb * MX_BK, m0);
          if constexpr (DUAL) {
            tma_load_2d(st + MX_A_BYTES, &tm_b0, &full_bar[s], kb * MX_BK, n0);                    // 64 gate rows
            tma_load_2d(st + MX_A_BYTES + MX_B_BYTES / 2, &tm_b1, &full_bar[s], kb * MX_BK, n0);   // 64 up rows
          } else {
            tma_load_2d(st + MX_A_BYTES, &tm_b0, &full_bar[s], kb * MX_BK, n0);
          }
          uint8_t* sf = st + MX_A_BYTES + MX_B_BYTES;
          bulk_load(sf, p.sfa + ((size_t)m_blk * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[s]);
          bulk_load(sf + MX_SF_BYTES, p.sfb0 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[s]);
          if constexpr (DUAL)
            bulk_load(sf + 2 * MX_SF_BYTES, p.sfb1 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[s]);
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) { long long t0 = clock64(); while (clock64() - t0 < 2000000) { } }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true; int it = 0;
      const uint32_t sf_tmem = tmem_base + MX_SF_COL;
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
        const int n0 = (int)(t % p.n_blocks) * OUT_COLS;
        const uint32_t sfb_sub = (uint32_t)((n0 % 128) / 32);      // dual: which 64-row half of the scale tile
        if (!mbar_wait(&acc_empty[as], aph ^ 1, abort_flag, ST_TIMEOUT_MMA, 0x700 | as, budget)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * MX_BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abort_flag, ST_TIMEOUT_MMA, 0x800 | s, budget)) { ok = false; break; }
          tc_fence_after();
          const uint32_t st = smem_u32(smem + s * MX_STAGE_BYTES);
          const uint32_t sf = st + MX_A_BYTES + MX_B_BYTES;
          tmem_cp_32x128b_warpx4(sf_tmem, sf_smem_desc(sf));
          tmem_cp_32x128b_warpx4(sf_tmem + 4, sf_smem_desc(sf + MX_SF_BYTES));
          if constexpr (DUAL) tmem_cp_32x128b_warpx4(sf_tmem + 8, sf_smem_desc(sf + 2 * MX_SF_BYTES));
          const uint64_t a_desc = umma_smem_desc_sw128(st);
          const uint64_t b_desc = umma_smem_desc_sw128(st + MX_A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t acc = (kb | k) != 0;
            if constexpr (DUAL) {
              const uint64_t bu_desc = umma_smem_desc_sw128(st + MX_A_BYTES + MX_B_BYTES / 2);
              const uint32_t idesc = umma_idesc_mx(0, 0, MX_BM, 64, k, k);
              umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sf_tmem, sf_tmem + 4 + sfb_sub, acc);
              umma_mxf8(d_tmem + 64, a_desc + 2 * k, bu_desc + 2 * k, idesc, sf_tmem, sf_tmem + 8 + sfb_sub, acc);
            } else {
              const uint32_t idesc = umma_idesc_mx(0, 0, MX_BM, MX_BN, k, k);
              umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sf_tmem, sf_tmem + 4, acc);
            }
          }
          umma_commit(&empty_bar[s]);
          if (++s == MX_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&acc_full[as]);
      }
    }
  } else if (warp >= MX_FRONT_WARPS) {
    const int e = warp - MX_FRONT_WARPS, q = warp & 3, half = e >> 2;
    uint8_t* out_buf = out_base + e * MX_OUT_BUFS * MX_OUT_BUF;
    uint32_t stg_off[4];
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) stg_off[pc] = lane * 64 + ((pc ^ ((lane >> 1) & 3)) << 4);
    int it = 0, obuf = 0; bool ok = true;
    for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
      const int m0 = (int)(t / p.n_blocks) * MX_BM, n0 = (int)(t % p.n_blocks) * OUT_COLS;
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[as], aph, abort_flag, ST_TIMEOUT_EPILOGUE, 0x900 | as, budget))) { ok = false; break; }
      tc_fence_after();
      const int row_base = m0 + q * 32;
      const uint32_t t_row = tmem_base + as * MX_BN + ((uint32_t)(q * 32) << 16);
      if (row_base < p.M) {
        auto emit_box = [&](int n, const uint32_t (&w)[16]) {      // 32 fp16 of this thread's row -> one staged box -> TMA store
          if (lane == 0) tma_store_wait_read<MX_OUT_BUFS - 1>();
          __syncwarp();
          uint8_t* buf = out_buf + obuf * MX_OUT_BUF;
#pragma unroll
          for (int pc = 0; pc < 4; ++pc)
            *reinterpret_cast<uint4*>(buf + stg_off[pc]) = make_uint4(w[4 * pc], w[4 * pc + 1], w[4 * pc + 2], w[4 * pc + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) { tma_store_2d(&tm_c, buf, n, row_base); tma_store_commit(); }
          obuf ^= 1;
        };
        if constexpr (DUAL) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(t_row + half * 32, g);
          tmem_ld_32x32b_x32(t_row + 64 + half * 32, u);
          tmem_ld_wait();
          const int n = n0 + half * 32;
          if (n < p.N) {
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              // silu(gate) * up with silu(g) = h + h * tanh(h), h = g / 2
              const float2 hv = __fmul2_rn(make_float2(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1])), make_float2(0.5f, 0.5f));
              const float2 uv = make_float2(__uint_as_float(u[2 * j]), __uint_as_float(u[2 * j + 1]));
              w[j] = pack_half2_from(__fmul2_rn(silu_from_half2(hv), uv));
            }
            emit_box(n, w);
          }
        } else {
          uint32_t v[2][32];
          tmem_ld_32x32b_x32(t_row + half * 64, v[0]);
          tmem_ld_32x32b_x32(t_row + half * 64 + 32, v[1]);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int n = n0 + half * 64 + h * 32;
            if (n < p.N) {
              uint32_t w[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) w[j] = pack_half2(__uint_as_float(v[h][2 * j]), __uint_as_float(v[h][2 * j + 1]));
              emit_box(n, w);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, MX_TMEM_COLS); }
}

// ---- weight-stationary kernel (K <= 512) ----------------------------------------------------------------------
// What bounds these GEMMs at K = 512 is neither HBM nor the tensor core but what one SM can take in from L2: about
// 36 bytes per clock, measured with plain bulk copies (10 TB/s over the 148 SMs).  A 128-byte K block of A (16 KiB)
// takes ~460 clocks to arrive and feeds 256 clocks of N = 128 MMAs, so a 128 x 128 tile that streams both operands
// spends most of its time waiting for data.  This kernel cuts the bytes taken in per output:
//   * the CTA owns a fixed slice of 256 rows of W (dual: 128 gate + 128 up) for the whole launch - all K blocks of
//     it stay in shared memory (128 KiB), their scale tiles in TMEM; only A and its scale tiles stream;
//   * one accumulator of 256 columns: every A byte taken in feeds 256 output columns (dual: 128), twice the reuse of
//     the streaming kernel.  TMEM (512 columns) cannot hold two such accumulators next to the scale factors, so
//     the epilogue pulls the whole accumulator into registers at once (128 per thread) and hands it back before
//     it converts and stores; the A ring keeps filling meanwhile;
//   * N = 256 MMAs run 128 clocks each, more than the ~55 clocks the issuing thread spends per tcgen05.mma and
//     enough to hide its barrier wait, scale copy and commit behind the tensor core's queue (N = 128 MMAs are not).
// CTA (group g, slice n) walks row blocks g, g + groups, ...; grid = groups * slices <= SM count.
constexpr int MXW_BN = 256;
constexpr int MXW_MAX_KB = 4;
constexpr int MXW_WKB_BYTES = MXW_BN * MX_BK;                        // 32 KiB of W per K block
constexpr int MXW_W_BYTES = MXW_MAX_KB * MXW_WKB_BYTES;              // 128 KiB
constexpr int MXW_SFB_BYTES = MXW_MAX_KB * 2 * MX_SF_BYTES;          // per K block two scale tiles (256 rows)
constexpr int MXW_STAGE_BYTES = MX_A_BYTES + 2 * MX_SF_BYTES;        // A | SFA | pad = 17 KiB (keeps 1 KiB alignment)
constexpr int MXW_STAGES = 3;
constexpr int MXW_OUT_BUF = 4096;                                    // per epilogue warp: one 32 x 64 fp16 box
constexpr int MXW_SMEM_SFB = MXW_W_BYTES;
constexpr int MXW_SMEM_RING = MXW_SMEM_SFB + MXW_SFB_BYTES;
constexpr int MXW_SMEM_OUT = MXW_SMEM_RING + MXW_STAGES * MXW_STAGE_BYTES;
constexpr int MXW_SMEM_BAR = MXW_SMEM_OUT + MX_EPI_WARPS * MXW_OUT_BUF;
constexpr int MXW_SMEM_BYTES = MXW_SMEM_BAR + 256 + 1024;
constexpr int MXW_SFA_COL = MXW_BN;                                  // + (kb % 4) * 4: a slot per K block
constexpr int MXW_SFB_COL = MXW_BN + 16;                             // + kb * 8: rows 0..127 | rows 128..255
constexpr int MXW_FRONT_REGS = 56, MXW_EPI_REGS = 224;               // setmaxnreg budgets: 4 x 32 x 56 + 8 x 32 x 224 <= 64 Ki
static_assert(MXW_SMEM_BYTES > 116 * 1024 && MXW_SMEM_BYTES <= 227 * 1024, "one CTA per SM");
static_assert(MXW_SFB_COL + MXW_MAX_KB * 8 <= MX_TMEM_COLS, "TMEM budget");

template <bool DUAL>
__global__ void __launch_bounds__(MX_THREADS, 1)
mx_gemm_wres_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_c, const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_res = smem;
  uint8_t* sfb_res = smem + MXW_SMEM_SFB;
  uint8_t* ring = smem + MXW_SMEM_RING;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + MXW_SMEM_BAR);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + MXW_STAGES;
  uint64_t* acc_full = bars + 2 * MXW_STAGES;
  uint64_t* acc_empty = acc_full + 1;
  uint64_t* w_full = acc_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int OUT_COLS = DUAL ? MXW_BN / 2 : MXW_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MXW_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(acc_full, 1); mbar_init(acc_empty, MX_EPI_WARPS); mbar_init(w_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_b0); prefetch_tmap(&tm_b1); prefetch_tmap(&tm_c);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, MX_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const long long budget = spin_budget();
  const int slice = (int)(blockIdx.x % p.n_blocks), grp = (int)(blockIdx.x / p.n_blocks);
  const int n0 = slice * OUT_COLS;
  const int sf_rows128 = (p.N + 127) / 128;                // row blocks the W scale tensors hold

  if (warp < MX_FRONT_WARPS) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(MXW_FRONT_REGS));
  if (warp == 0) {
    if (lane == 0) {
      // resident slice: per K block 256 rows of W and their two scale tiles
      const int nb128 = n0 / 128;                          // plain: first of two row blocks; dual: the one of gate and up
      const bool second = DUAL || nb128 + 1 < sf_rows128;  // plain, N % 256 == 128: the last slice has one scale tile
      mbar_arrive_expect_tx(w_full, p.k_blocks * (MXW_WKB_BYTES + (second ? 2 : 1) * MX_SF_BYTES));
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        uint8_t* wb = w_res + kb * MXW_WKB_BYTES;
        uint8_t* sf = sfb_res + kb * 2 * MX_SF_BYTES;
        if constexpr (DUAL) {
          tma_load_2d(wb, &tm_b0, w_full, kb * MX_BK, n0);
          tma_load_2d(wb + MXW_WKB_BYTES / 2, &tm_b1, w_full, kb * MX_BK, n0);
          bulk_load(sf, p.sfb0 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
          bulk_load(sf + MX_SF_BYTES, p.sfb1 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
        } else {
          tma_load_2d(wb, &tm_b0, w_full, kb * MX_BK, n0);                       // rows past N arrive as zeros
          tma_load_2d(wb + MXW_WKB_BYTES / 2, &tm_b0, w_full, kb * MX_BK, n0 + 128);
          bulk_load(sf, p.sfb0 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
          if (second) bulk_load(sf + MX_SF_BYTES, p.sfb0 + ((size_t)(nb128 + 1) * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
        }
      }
      int s = 0; uint32_t ph = 0; bool ok = true;
      for (int m_blk = grp; ok && m_blk < p.m_blocks; m_blk += p.n_groups) {
        // the row block two tiles ahead goes to L2 now (one CTA of those that will read it asks for it)
        const int m_pf = m_blk + 2 * p.n_groups;
        if (m_pf < p.m_blocks && slice == m_pf % p.n_blocks)
          for (int kb = 0; kb < p.k_blocks; ++kb) tma_prefetch_l2_2d(&tm_a, kb * MX_BK, m_pf * MX_BM);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, 0x600 | s, budget)) { ok = false; break; }
          uint8_t* st = ring + s * MXW_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], MX_A_BYTES + MX_SF_BYTES);
          tma_load_2d(st, &tm_a, &full_bar[s], kb * MX_BK, m_blk * MX_BM);
          bulk_load(st + MX_A_BYTES, p.sfa + ((size_t)m_blk * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full_bar[s]);
          if (++s == MXW_STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (!ok) { long long t0 = clock64(); while (clock64() - t0 < 2000000) { } }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t sfa_tmem = tmem_base + MXW_SFA_COL, sfb_tmem = tmem_base + MXW_SFB_COL;
      bool ok = mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_MMA, 0xA00, budget);
      if (ok) {
        tc_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb) {          // the slice's scale tiles go to TMEM once
          tmem_cp_32x128b_warpx4(sfb_tmem + kb * 8, sf_smem_desc(smem_u32(sfb_res + kb * 2 * MX_SF_BYTES)));
          tmem_cp_32x128b_warpx4(sfb_tmem + kb * 8 + 4, sf_smem_desc(smem_u32(sfb_res + kb * 2 * MX_SF_BYTES + MX_SF_BYTES)));
        }
      }
      int s = 0; uint32_t ph = 0, aph = 0;
      for (int m_blk = grp; ok && m_blk < p.m_blocks; m_blk += p.n_groups, aph ^= 1) {
        if (!mbar_wait(acc_empty, aph ^ 1, abort_flag, ST_TIMEOUT_MMA, 0x700, budget)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          // the wait orders the TMA writes before the reads below; no tcgen05 fence is needed for that
          if (!mbar_wait(&full_bar[s], ph, abort_flag, ST_TIMEOUT_MMA, 0x800 | s, budget)) { ok = false; break; }
          const uint32_t st = smem_u32(ring + s * MXW_STAGE_BYTES);
          const uint32_t sfa_t = sfa_tmem + (kb & 3) * 4;  // a slot per K block: this copy does not wait for the MMAs before it
          tmem_cp_32x128b_warpx4(sfa_t, sf_smem_desc(st + MX_A_BYTES));
          const uint64_t a_desc = umma_smem_desc_sw128(st);
          const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(w_res + kb * MXW_WKB_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_mxf8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, umma_idesc_mx(0, 0, MX_BM, MXW_BN, k, k), sfa_t,
                      sfb_tmem + kb * 8, (kb | k) != 0);
          umma_commit(&empty_bar[s]);
          if (++s == MXW_STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(acc_full);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(MXW_EPI_REGS));
    // warp e: TMEM lane quarter e % 4 (32 rows), column half e / 4 (plain: 128 output columns; dual: 64)
    const int e = warp - MX_FRONT_WARPS, q = warp & 3, half = e >> 2;
    uint8_t* out_buf = smem + MXW_SMEM_OUT + e * MXW_OUT_BUF;
    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t aph = 0;
    for (int m_blk = grp; m_blk < p.m_blocks; m_blk += p.n_groups, aph ^= 1) {
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full, aph, abort_flag, ST_TIMEOUT_EPILOGUE, 0x900, budget))) break;
      tc_fence_after();
      const int row_base = m_blk * MX_BM + q * 32;
      uint32_t v[4][32];                                   // plain: 128 columns; dual: gate 2 x 32 | up 2 x 32
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = DUAL ? (c >> 1) * (MXW_BN / 2) + half * 64 + (c & 1) * 32 : half * 128 + c * 32;
        tmem_ld_32x32b_x32(t_row + col, v[c]);
      }
      tmem_ld_wait();
      tc_fence_before();                                   // the accumulator goes back before anything is converted
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      // one 32 x 64 fp16 box (rows of 128 bytes, 128-byte swizzle) per 64 output columns
      auto emit = [&](int n, const uint32_t (&w)[32]) {
        if (row_base >= p.M || n >= p.N) return;
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int pc = 0; pc < 8; ++pc)
          *reinterpret_cast<uint4*>(out_buf + lane * 128 + ((pc ^ (lane & 7)) << 4)) = make_uint4(w[4 * pc], w[4 * pc + 1], w[4 * pc + 2], w[4 * pc + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) { tma_store_2d(&tm_c, out_buf, n, row_base); tma_store_commit(); }
      };
      if constexpr (DUAL) {
        uint32_t w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          // silu(gate) * up with silu(g) = h + h * tanh(h), h = g / 2
          const uint32_t* g = v[j >> 4]; const uint32_t* u = v[2 + (j >> 4)];
          const int i = (2 * j) & 31;
          const float2 hv = __fmul2_rn(make_float2(__uint_as_float(g[i]), __uint_as_float(g[i + 1])), make_float2(0.5f, 0.5f));
          const float2 uv = make_float2(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
          w[j] = pack_half2_from(__fmul2_rn(silu_from_half2(hv), uv));
        }
        emit(n0 + half * 64, w);
      } else {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          uint32_t w[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const uint32_t* x = v[2 * b + (j >> 4)];
            const int i = (2 * j) & 31;
            w[j] = pack_half2(__uint_as_float(x[i]), __uint_as_float(x[i + 1]));
          }
          emit(n0 + half * 128 + b * 64, w);
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, MX_TMEM_COLS); }
}

// ---- row-major [rows, K/32] scales -> the 128 x 4 tile order (one thread per output byte) -------------------
__global__ void mx_scales_to_tiled_kernel(const uint8_t* __restrict__ src, long long ld, long long rows, int k32,
                                          uint8_t* __restrict__ dst, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int kt = k32 / 4;                                  // 128-wide K tiles
  const long long tile = i / 512; const int in = (int)(i % 512);
  const long long rb = tile / kt; const int kb = (int)(tile % kt);
  const int r = (in / 16) + 32 * ((in % 16) / 4);          // row inside the 128-row block
  const int b = kb * 4 + (in % 4);
  const long long row = rb * 128 + r;
  dst[i] = (row < rows) ? src[row * ld + b] : (uint8_t)127;   // padding rows: scale 1.0 on zero data
}

typedef CUresult (*EncodeTiledFnM)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

size_t mx_tiled_scale_bytes(long long rows, int K) {
  return (size_t)((rows + 127) / 128) * (size_t)(K / 128) * 512;
}

int32_t launch_mx_scales_to_tiled(const uint8_t* src, long long ld, long long rows, int K, uint8_t* dst, cudaStream_t st) {
  if (rows == 0) return GSB200_OK;
  if (!src || !dst || rows < 0 || K <= 0 || K % 128 != 0 || ld < K / 32) return GSB200_ERR_BAD_ARG;
  const long long total = (long long)mx_tiled_scale_bytes(rows, K);
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  mx_scales_to_tiled_kernel<<<(unsigned)blocks, 256, 0, st>>>(src, ld, rows, K / 32, dst, total);
  return cuda_status(cudaGetLastError(), "mx scale re-tiling launch");
}

int32_t launch_mx_gemm(bool dual, const uint8_t* A, long long lda, const uint8_t* sfa, const uint8_t* B0,
                       const uint8_t* B1, long long ldb, const uint8_t* sfb0, const uint8_t* sfb1, void* C,
                       long long ldc, long long M, int N, int K, cudaStream_t st) {
  if (M == 0) return GSB200_OK;
  if (M < 0 || M > 0x7fffff00ll || N <= 0 || K <= 0) return GSB200_ERR_BAD_ARG;
  if (!A || !sfa || !B0 || !sfb0 || !C || (dual && (!B1 || !sfb1))) return GSB200_ERR_BAD_ARG;
  const uintptr_t al = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(B0) |
                       reinterpret_cast<uintptr_t>(sfb0) | reinterpret_cast<uintptr_t>(C) |
                       (dual ? (reinterpret_cast<uintptr_t>(B1) | reinterpret_cast<uintptr_t>(sfb1)) : 0);
  if (al & 15) return GSB200_ERR_BAD_ARG;
  if (K % 128 != 0 || lda < K || ldb < K || lda % 16 != 0 || ldb % 16 != 0) return GSB200_ERR_BAD_ARG;
  if (N % 32 != 0 || ldc < N || ldc % 8 != 0) return GSB200_ERR_BAD_ARG;
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;
  static bool attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e1 = cudaFuncSetAttribute(mx_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM_BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(mx_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MX_SMEM_BYTES);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return cuda_status(e1 != cudaSuccess ? e1 : e2, "cudaFuncSetAttribute(mx gemm)");
    e1 = cudaFuncSetAttribute(mx_gemm_wres_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MXW_SMEM_BYTES);
    e2 = cudaFuncSetAttribute(mx_gemm_wres_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MXW_SMEM_BYTES);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return cuda_status(e1 != cudaSuccess ? e1 : e2, "cudaFuncSetAttribute(mx gemm)");
    attr_done[dev] = true;
  }
  void* fnp = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fnp, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return GSB200_ERR_DEVICE;
  EncodeTiledFnM enc = reinterpret_cast<EncodeTiledFnM>(fnp);
  auto map2d = [&](CUtensorMap* m, CUtensorMapDataType dt, int esz, const void* base, uint64_t rows, uint64_t cols,
                   uint64_t ld, uint32_t bc, uint32_t br, CUtensorMapSwizzle sw) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * (uint64_t)esz};
    cuuint32_t box[2] = {bc, br};
    cuuint32_t es[2] = {1, 1};
    return enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  };
  CUtensorMap ta, tb0, tb1, tc;
  MxParams p{};
  p.M = (int)M; p.N = N; p.K = K;
  p.m_blocks = (int)((M + MX_BM - 1) / MX_BM);
  p.k_blocks = K / MX_BK;
  p.sfa = sfa; p.sfb0 = sfb0; p.sfb1 = sfb1;
  const int wres_cols = dual ? MXW_BN / 2 : MXW_BN;
  const int wres_slices = (N + wres_cols - 1) / wres_cols;
  if (p.k_blocks <= MXW_MAX_KB && wres_slices <= sm_count()) {       // weight-stationary kernel
    bool ok = map2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    ok = ok && map2d(&tb0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    ok = ok && map2d(&tb1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, dual ? B1 : B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    ok = ok && map2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return GSB200_ERR_BAD_ARG;
    p.n_blocks = wres_slices;
    int groups = sm_count() / wres_slices;
    if (groups > p.m_blocks) groups = p.m_blocks;
    p.n_groups = groups;
    const int grid = groups * wres_slices;
    if (dual) mx_gemm_wres_kernel<true><<<grid, MX_THREADS, MXW_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
    else mx_gemm_wres_kernel<false><<<grid, MX_THREADS, MXW_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
    return cuda_status(cudaGetLastError(), "mx gemm launch");
  }
  const uint32_t brows = dual ? 64 : 128;
  bool ok = map2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && map2d(&tb0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, brows, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && map2d(&tb1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, dual ? B1 : B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, brows, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && map2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
  if (!ok) return GSB200_ERR_BAD_ARG;
  const int out_cols = dual ? 64 : 128;
  p.n_blocks = (N + out_cols - 1) / out_cols;
  const long long tiles = (long long)p.m_blocks * p.n_blocks;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  if (dual) mx_gemm_kernel<true><<<grid, MX_THREADS, MX_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
  else mx_gemm_kernel<false><<<grid, MX_THREADS, MX_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
  return cuda_status(cudaGetLastError(), "mx gemm launch");
}

}  // namespace gsb
