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
// Tiles are 128 rows x 128 accumulator columns (dual: gate -> columns 0..63, up -> 64..127), two accumulator
// stages.  The CTA runs TWO independent pipelines, one per accumulator stage: pipeline 0 takes the even tiles of
// the CTA, pipeline 1 the odd ones, each with its own producer thread (warps 0 / 3), its own MMA-issuing thread
// (warps 1 / 2), its own ring of operand stages and its own barriers; they share the tensor core and the eight
// epilogue warps.  The reasons, all measured on B200 with small probe kernels:
//   * an N = 128 MMA runs 64 clocks, but a tcgen05.mma costs the thread that issues it ~55 clocks, and a barrier
//     wait, a scale copy and a commit cost 60-90 each: one issuing thread leaves the tensor core idle more than half
//     the time.  Two threads can issue concurrently; the tensor core takes their MMAs in turn without loss;
//   * a producer thread that waits for a free stage and then issues its loads completes one round per ~570 clocks
//     plus ~170 per 16 KiB box, however many stages are in flight: 22 bytes per clock with one box per round, 37 with
//     two.  A second producer thread doubles that;
//   * a parity wait is only valid for a thread that sees every phase of its barrier, so no ring stage is ever shared
//     between the two threads of a role: each pipeline has its own stages.
// Two forms:
//   streaming (any K)            a stage holds one K block of A and of W and their scale tiles, three stages per
//                                pipeline; tiles are dealt round-robin; the dual form issues two N = 64 MMAs per K step
//                                so that gate and up keep their own scale tiles.
//   weight-stationary (K <= 512) CTA (group g, slice n) keeps the 128 rows of W of column slice n (dual: 64 gate + 64
//                                up) in shared memory and their scale tiles in TMEM for the whole launch and walks row
//                                blocks g, g + groups, ...; a stage holds TWO K blocks of A (one wait and one commit
//                                per 8 MMAs), two stages per pipeline.  Gate and up rows are adjacent in shared memory
//                                and are multiplied as ONE N = 128 operand whose scale tile is assembled once per CTA
//                                from the row groups of the two tiles.
// M = 65536, N = 2048, K = 512: 104 us (plain) / 276 us (dual) with one pipeline and both operands streamed, 75 / 128 us
// in the weight-stationary form.
#include <atomic>

#include "capi_internal.h"
#include "ptx.cuh"

namespace gsb {

constexpr int MX_BM = 128, MX_BN = 128, MX_BK = 128;
constexpr int MX_A_BYTES = MX_BM * MX_BK;            // 16 KiB
constexpr int MX_B_BYTES = MX_BN * MX_BK;            // 16 KiB
constexpr int MX_SF_BYTES = 512;
constexpr int MX_EPI_WARPS = 8, MX_FRONT_WARPS = 4;
constexpr int MX_THREADS = 32 * (MX_EPI_WARPS + MX_FRONT_WARPS);
constexpr int MX_OUT_BUF = 2048;                     // per epilogue warp: one 32 x 32 fp16 box
constexpr int MX_TMEM_COLS = 512;
constexpr int MX_SF_COL = 256;                       // scale-factor columns: pipeline pl uses MX_SF_COL + pl * 16 ...
constexpr int MXW_SFB_COL = MX_SF_COL + 32;          // ... and the resident W scales sit at MXW_SFB_COL + kb * 4
// streaming form: stage = A | W | SFA | SFB0 | SFB1 | pad (keeps 1 KiB alignment), three stages per pipeline
constexpr int MXS_STAGE_BYTES = MX_A_BYTES + MX_B_BYTES + 4 * MX_SF_BYTES;     // 34 KiB
constexpr int MXS_STAGES = 3;
// weight-stationary form: resident W slice (up to 4 K blocks) and its scale tiles, then stages of
// A(kb) | A(kb+1) | SFA(kb) | SFA(kb+1), two per pipeline
constexpr int MXW_MAX_KB = 4;
constexpr int MXW_KPS = 2;                                           // K blocks per stage
constexpr int MXW_W_BYTES = MXW_MAX_KB * MX_B_BYTES;                 // 64 KiB
constexpr int MXW_SFB_BYTES = MXW_MAX_KB * 2 * MX_SF_BYTES;          // 4 KiB: per K block SFB0 | SFB1
constexpr int MXW_STAGE_BYTES = MXW_KPS * (MX_A_BYTES + MX_SF_BYTES);   // 33 KiB
constexpr int MXW_STAGES = 2;
static_assert(MXW_STAGE_BYTES % 1024 == 0 && MXS_STAGE_BYTES % 1024 == 0, "swizzled tiles need 1 KiB alignment");

template <bool WST>
struct MxSmem {
  static constexpr int STAGES = WST ? MXW_STAGES : MXS_STAGES;       // per pipeline
  static constexpr int STAGE_BYTES = WST ? MXW_STAGE_BYTES : MXS_STAGE_BYTES;
  static constexpr int RING = WST ? MXW_W_BYTES + MXW_SFB_BYTES : 0;
  static constexpr int OUT = RING + 2 * STAGES * STAGE_BYTES;
  static constexpr int BAR = OUT + MX_EPI_WARPS * MX_OUT_BUF;
  static constexpr int BYTES = BAR + 256 + 1024;
  static_assert(BYTES > 116 * 1024 && BYTES <= 227 * 1024, "one CTA per SM");
};

struct MxParams {
  int M, N, K;
  int m_blocks, n_blocks, k_blocks;
  int n_groups;                      // weight-stationary: row-block groups (grid = n_groups * n_blocks)
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

template <bool DUAL, bool WST>
__global__ void __launch_bounds__(MX_THREADS, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
               const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_c, const MxParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = MxSmem<WST>;
  constexpr int STAGES = L::STAGES, STAGE_BYTES = L::STAGE_BYTES;
  uint8_t* w_res = smem;                                   // WST: resident W slice, MX_B_BYTES per K block
  uint8_t* sfb_res = smem + MXW_W_BYTES;                   // WST: its scale tiles, 1 KiB per K block
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR);
  uint64_t* full_bar = bars;                               // [pipeline * STAGES + stage]
  uint64_t* empty_bar = bars + 2 * STAGES;
  uint64_t* acc_full = bars + 4 * STAGES;                  // [pipeline]
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* w_full = acc_empty + 2;                        // WST: resident slice landed
  uint64_t* sfb_ready = w_full + 1;                        // WST: its scale tiles are in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sfb_ready + 1);
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int OUT_COLS = DUAL ? MX_BN / 2 : MX_BN;          // output columns per tile
  const long long num_tiles = (long long)p.m_blocks * p.n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], MX_EPI_WARPS); }
    mbar_init(w_full, 1); mbar_init(sfb_ready, 1);
    abort_flag.set(0);
    fence_mbar_init();
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_b0); prefetch_tmap(&tm_b1); prefetch_tmap(&tm_c);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, MX_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();          // bound of every wait below, fetched once
  // this CTA's tiles: streaming form t = cta, cta + grid, ... (column block fastest); weight-stationary form: a fixed
  // column block and row blocks group, group + n_groups, ...  Tile number `it` of the CTA belongs to pipeline it % 2.
  const int ws_n = WST ? (int)(blockIdx.x % p.n_blocks) : 0;
  const int ws_g = WST ? (int)(blockIdx.x / p.n_blocks) : 0;
  auto tile_at = [&](int it, int& m_blk, int& n_blk) -> bool {
    if constexpr (WST) {
      m_blk = ws_g + it * p.n_groups; n_blk = ws_n;
      return m_blk < p.m_blocks;
    } else {
      const long long t = (long long)blockIdx.x + (long long)it * gridDim.x;
      if (t >= num_tiles) return false;
      m_blk = (int)(t / p.n_blocks); n_blk = (int)(t % p.n_blocks);
      return true;
    }
  };

  if (warp == 0 || warp == 3) {
    // ------------------------------ producers: warp 0 -> pipeline 0, warp 3 -> pipeline 1 ------------------------------
    const int pl = warp == 3 ? 1 : 0;
    if (lane == 0) {
      uint8_t* ring = smem + L::RING + pl * STAGES * STAGE_BYTES;
      uint64_t* full = full_bar + pl * STAGES; uint64_t* empty = empty_bar + pl * STAGES;
      int s = 0; uint32_t ph = 0; bool ok = true;
      if (WST && pl == 0) {                                // the resident slice and its scale tiles
        const int n0 = ws_n * OUT_COLS, nb128 = n0 / 128;
        mbar_arrive_expect_tx(w_full, p.k_blocks * (MX_B_BYTES + (DUAL ? 2 : 1) * MX_SF_BYTES));
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          uint8_t* wb = w_res + kb * MX_B_BYTES;
          if constexpr (DUAL) {
            tma_load_2d(wb, &tm_b0, w_full, kb * MX_BK, n0);                     // 64 gate rows
            tma_load_2d(wb + MX_B_BYTES / 2, &tm_b1, w_full, kb * MX_BK, n0);    // 64 up rows
          } else {
            tma_load_2d(wb, &tm_b0, w_full, kb * MX_BK, n0);
          }
          bulk_load(sfb_res + kb * 2 * MX_SF_BYTES, p.sfb0 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
          if constexpr (DUAL)
            bulk_load(sfb_res + kb * 2 * MX_SF_BYTES + MX_SF_BYTES, p.sfb1 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, w_full);
        }
      }
      int m_blk, n_blk;
      for (int it = pl; ok && tile_at(it, m_blk, n_blk); it += 2) {
        const int m0 = m_blk * MX_BM, n0 = n_blk * OUT_COLS;
        if constexpr (WST) {
          // this pipeline's next row block goes to L2 now (one CTA of the column slices asks for it)
          const int m_pf = m_blk + 2 * p.n_groups;
          if (m_pf < p.m_blocks && ws_n == m_pf % p.n_blocks)
            for (int kb = 0; kb < p.k_blocks; ++kb) tma_prefetch_l2_2d(&tm_a, kb * MX_BK, m_pf * MX_BM);
          for (int kb = 0; kb < p.k_blocks; kb += MXW_KPS) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, 0x600 | (pl << 4) | s, budget)) { ok = false; break; }
            uint8_t* st = ring + s * STAGE_BYTES;
            const int nk = p.k_blocks - kb < MXW_KPS ? p.k_blocks - kb : MXW_KPS;
            mbar_arrive_expect_tx(&full[s], nk * (MX_A_BYTES + MX_SF_BYTES));
            for (int j = 0; j < nk; ++j) tma_load_2d(st + j * MX_A_BYTES, &tm_a, &full[s], (kb + j) * MX_BK, m0);
            bulk_load(st + MXW_KPS * MX_A_BYTES, p.sfa + ((size_t)m_blk * p.k_blocks + kb) * MX_SF_BYTES, nk * MX_SF_BYTES, &full[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        } else {
          const int nb128 = n0 / 128;                      // scale tile row block of W
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, 0x600 | (pl << 4) | s, budget)) { ok = false; break; }
            uint8_t* st = ring + s * STAGE_BYTES;
            mbar_arrive_expect_tx(&full[s], MX_A_BYTES + MX_B_BYTES + (DUAL ? 3 : 2) * MX_SF_BYTES);
            tma_load_2d(st, &tm_a, &full[s], kb * MX_BK, m0);
            if constexpr (DUAL) {
              tma_load_2d(st + MX_A_BYTES, &tm_b0, &full[s], kb * MX_BK, n0);                    // 64 gate rows
              tma_load_2d(st + MX_A_BYTES + MX_B_BYTES / 2, &tm_b1, &full[s], kb * MX_BK, n0);   // 64 up rows
            } else {
              tma_load_2d(st + MX_A_BYTES, &tm_b0, &full[s], kb * MX_BK, n0);
            }
            uint8_t* sf = st + MX_A_BYTES + MX_B_BYTES;
            bulk_load(sf, p.sfa + ((size_t)m_blk * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
            bulk_load(sf + MX_SF_BYTES, p.sfb0 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
            if constexpr (DUAL)
              bulk_load(sf + 2 * MX_SF_BYTES, p.sfb1 + ((size_t)nb128 * p.k_blocks + kb) * MX_SF_BYTES, MX_SF_BYTES, &full[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
      if (!ok) { long long t0 = clock64(); while (clock64() - t0 < 2000000) { } }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------ MMA issuers: warp 1 -> pipeline 0, warp 2 -> pipeline 1 ------------------------------
    const int pl = warp - 1;
    bool ok = true;
    if constexpr (WST) {
      // warp 1 waits for the resident slice; the dual form then builds, per K block, the scale tile of its N = 128
      // operand [64 gate rows | 64 up rows] in place: row groups sub, sub+1 of the gate tile, then of the up tile
      if (pl == 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_MMA, 0xA00, budget));
        if constexpr (DUAL) {
          if (ok) {
            const int sub = ((ws_n * OUT_COLS) % 128) / 32;
            for (int kb = 0; kb < p.k_blocks; ++kb) {
              uint32_t* tg = reinterpret_cast<uint32_t*>(sfb_res + kb * 2 * MX_SF_BYTES);
              const uint32_t* tu = tg + MX_SF_BYTES / 4;
              const uint4 v = make_uint4(tg[lane * 4 + sub], tg[lane * 4 + sub + 1], tu[lane * 4 + sub], tu[lane * 4 + sub + 1]);
              *reinterpret_cast<uint4*>(tg + lane * 4) = v;
            }
            fence_proxy_async_smem();
          }
        }
        __syncwarp();
      }
    }
    if (lane == 0 && ok) {
      const uint8_t* ring = smem + L::RING + pl * STAGES * STAGE_BYTES;
      uint64_t* full = full_bar + pl * STAGES; uint64_t* empty = empty_bar + pl * STAGES;
      int s = 0; uint32_t ph = 0;
      const uint32_t sf_tmem = tmem_base + MX_SF_COL + pl * 16;    // this pipeline's scale-factor columns
      const uint32_t sfb_tmem = tmem_base + MXW_SFB_COL;
      if constexpr (WST) {
        if (pl == 0) {                                     // the slice's scale tiles go to TMEM once
          tc_fence_after();
          for (int kb = 0; kb < p.k_blocks; ++kb)
            tmem_cp_32x128b_warpx4(sfb_tmem + kb * 4, sf_smem_desc(smem_u32(sfb_res + kb * 2 * MX_SF_BYTES)));
          umma_commit(sfb_ready);
        }
        ok = mbar_wait(w_full, 0, abort_flag, ST_TIMEOUT_MMA, 0xA01, budget) &&
             mbar_wait(sfb_ready, 0, abort_flag, ST_TIMEOUT_MMA, 0xA02, budget);
        tc_fence_after();
      }
      const uint32_t d_tmem = tmem_base + pl * MX_BN;
      int m_blk, n_blk;
      for (int it = pl; ok && tile_at(it, m_blk, n_blk); it += 2) {
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&acc_empty[pl], aph ^ 1, abort_flag, ST_TIMEOUT_MMA, 0x700 | pl, budget)) { ok = false; break; }
        tc_fence_after();
        if constexpr (WST) {
          for (int kb0 = 0; kb0 < p.k_blocks; kb0 += MXW_KPS) {
            // the wait orders the TMA writes before the reads below; no tcgen05 fence is needed for that
            if (!mbar_wait(&full[s], ph, abort_flag, ST_TIMEOUT_MMA, 0x800 | (pl << 4) | s, budget)) { ok = false; break; }
            const uint32_t st = smem_u32(ring + s * STAGE_BYTES);
            const int nk = p.k_blocks - kb0 < MXW_KPS ? p.k_blocks - kb0 : MXW_KPS;
            for (int j = 0; j < nk; ++j) {
              const int kb = kb0 + j;
              const uint32_t sfa_t = sf_tmem + (kb & 3) * 4;       // a slot per K block: no copy waits for earlier MMAs
              tmem_cp_32x128b_warpx4(sfa_t, sf_smem_desc(st + MXW_KPS * MX_A_BYTES + j * MX_SF_BYTES));
              const uint64_t a_desc = umma_smem_desc_sw128(st + j * MX_A_BYTES);
              const uint64_t b_desc = umma_smem_desc_sw128(smem_u32(w_res + kb * MX_B_BYTES));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, umma_idesc_mx(0, 0, MX_BM, MX_BN, k, k), sfa_t,
                          sfb_tmem + kb * 4, (kb | k) != 0);
            }
            umma_commit(&empty[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        } else {
          const uint32_t sfb_sub = (uint32_t)(((n_blk * OUT_COLS) % 128) / 32);   // dual: which 64-row half of the scale tile
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait(&full[s], ph, abort_flag, ST_TIMEOUT_MMA, 0x800 | (pl << 4) | s, budget)) { ok = false; break; }
            const uint32_t st = smem_u32(ring + s * STAGE_BYTES);
            const uint32_t sf = st + MX_A_BYTES + MX_B_BYTES;
            tmem_cp_32x128b_warpx4(sf_tmem, sf_smem_desc(sf));
            tmem_cp_32x128b_warpx4(sf_tmem + 4, sf_smem_desc(sf + MX_SF_BYTES));
            if constexpr (DUAL) tmem_cp_32x128b_warpx4(sf_tmem + 8, sf_smem_desc(sf + 2 * MX_SF_BYTES));
            const uint32_t b_addr = st + MX_A_BYTES;
            const uint64_t a_desc = umma_smem_desc_sw128(st);
            const uint64_t b_desc = umma_smem_desc_sw128(b_addr);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t acc = (kb | k) != 0;
              if constexpr (DUAL) {
                const uint64_t bu_desc = umma_smem_desc_sw128(b_addr + MX_B_BYTES / 2);
                const uint32_t idesc = umma_idesc_mx(0, 0, MX_BM, 64, k, k);
                umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, sf_tmem, sf_tmem + 4 + sfb_sub, acc);
                umma_mxf8(d_tmem + 64, a_desc + 2 * k, bu_desc + 2 * k, idesc, sf_tmem, sf_tmem + 8 + sfb_sub, acc);
              } else {
                umma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, umma_idesc_mx(0, 0, MX_BM, MX_BN, k, k), sf_tmem, sf_tmem + 4, acc);
              }
            }
            umma_commit(&empty[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
        if (ok) umma_commit(&acc_full[pl]);
      }
    }
  } else if (warp >= MX_FRONT_WARPS) {
    // ------------------------------ epilogue ------------------------------
    // Warp e: TMEM lane quarter e % 4 (32 rows) and column half e / 4 of every tile, in tile order.  The accumulator
    // stage goes back to its pipeline as soon as this warp's part is in registers; the values leave as 32 x 32
    // fp16 boxes (64-byte swizzle) through the warp's one staging buffer.
    const int e = warp - MX_FRONT_WARPS, q = warp & 3, half = e >> 2;
    uint8_t* out_buf = smem + L::OUT + e * MX_OUT_BUF;
    bool ok = true;
    int m_blk, n_blk;
    auto emit_box = [&](int n, int row_base, const uint32_t (&w)[16]) {
      if (lane == 0) tma_store_wait_read<0>();               // the previous box has left the buffer
      __syncwarp();
#pragma unroll
      for (int pc = 0; pc < 4; ++pc)
        *reinterpret_cast<uint4*>(out_buf + lane * 64 + ((pc ^ ((lane >> 1) & 3)) << 4)) = make_uint4(w[4 * pc], w[4 * pc + 1], w[4 * pc + 2], w[4 * pc + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) { tma_store_2d(&tm_c, out_buf, n, row_base); tma_store_commit(); }
    };
    for (int it = 0; ok && tile_at(it, m_blk, n_blk); ++it) {
      const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
      const int n0 = n_blk * OUT_COLS;
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[as], aph, abort_flag, ST_TIMEOUT_EPILOGUE, 0x900 | as, budget))) { ok = false; break; }
      tc_fence_after();
      const int row_base = m_blk * MX_BM + q * 32;
      const uint32_t t_row = tmem_base + as * MX_BN + ((uint32_t)(q * 32) << 16);
      uint32_t v[2][32];                                     // plain: 64 columns; dual: 32 gate | 32 up
      tmem_ld_32x32b_x32(t_row + (DUAL ? half * 32 : half * 64), v[0]);
      tmem_ld_32x32b_x32(t_row + (DUAL ? 64 + half * 32 : half * 64 + 32), v[1]);
      tmem_ld_wait(v[0], v[1]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
      if (row_base >= p.M) continue;
      if constexpr (DUAL) {
        const int n = n0 + half * 32;
        if (n < p.N) {
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            // silu(gate) * up with silu(g) = h + h * tanh(h), h = g / 2
            const float2 hv = __fmul2_rn(make_float2(__uint_as_float(v[0][2 * j]), __uint_as_float(v[0][2 * j + 1])), make_float2(0.5f, 0.5f));
            const float2 uv = make_float2(__uint_as_float(v[1][2 * j]), __uint_as_float(v[1][2 * j + 1]));
            w[j] = pack_half2_from(__fmul2_rn(silu_from_half2(hv), uv));
          }
          emit_box(n, row_base, w);
        }
      } else {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int n = n0 + half * 64 + b * 32;
          if (n < p.N) {
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = pack_half2(__uint_as_float(v[b][2 * j]), __uint_as_float(v[b][2 * j + 1]));
            emit_box(n, row_base, w);
          }
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
  static std::atomic<int> attr_done[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return GSB200_ERR_DEVICE;
  if (!attr_done[dev].load(std::memory_order_acquire)) {
    cudaError_t e1 = cudaFuncSetAttribute(mx_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<false>::BYTES);
    cudaError_t e2 = cudaFuncSetAttribute(mx_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<false>::BYTES);
    cudaError_t e3 = cudaFuncSetAttribute(mx_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<true>::BYTES);
    cudaError_t e4 = cudaFuncSetAttribute(mx_gemm_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<true>::BYTES);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return cuda_status(e1 != cudaSuccess ? e1 : e2, "cudaFuncSetAttribute(mx gemm)");
    if (e3 != cudaSuccess || e4 != cudaSuccess) return cuda_status(e3 != cudaSuccess ? e3 : e4, "cudaFuncSetAttribute(mx gemm)");
    attr_done[dev].store(1, std::memory_order_release);
  }
  auto map2d = [&](CUtensorMap* m, CUtensorMapDataType dt, int esz, const void* base, uint64_t rows, uint64_t cols,
                   uint64_t ld, uint32_t bc, uint32_t br, CUtensorMapSwizzle sw) {
    return tmap_2d(m, dt, esz, base, rows, cols, ld, bc, br, sw);
  };
  CUtensorMap ta, tb0, tb1, tc;
  const uint32_t brows = dual ? 64 : 128;
  bool ok = map2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && map2d(&tb0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, brows, CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && map2d(&tb1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, dual ? B1 : B0, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128, brows, CU_TENSOR_MAP_SWIZZLE_128B);
  const bool wst = K / MX_BK <= MXW_MAX_KB && (N + (dual ? 64 : 128) - 1) / (dual ? 64 : 128) <= sm_count();
  ok = ok && map2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
  if (!ok) return GSB200_ERR_BAD_ARG;
  MxParams p{};
  p.M = (int)M; p.N = N; p.K = K;
  const int out_cols = dual ? 64 : 128;
  p.m_blocks = (int)((M + MX_BM - 1) / MX_BM);
  p.n_blocks = (N + out_cols - 1) / out_cols;
  p.k_blocks = K / MX_BK;
  p.sfa = sfa; p.sfb0 = sfb0; p.sfb1 = sfb1;
  const long long tiles = (long long)p.m_blocks * p.n_blocks;
  if (wst) {                                                        // weight-stationary form
    int groups = sm_count() / p.n_blocks;
    if (groups > p.m_blocks) groups = p.m_blocks;
    p.n_groups = groups;
    const int grid = groups * p.n_blocks;
    if (dual) mx_gemm_kernel<true, true><<<grid, MX_THREADS, MxSmem<true>::BYTES, st>>>(ta, tb0, tb1, tc, p);
    else mx_gemm_kernel<false, true><<<grid, MX_THREADS, MxSmem<true>::BYTES, st>>>(ta, tb0, tb1, tc, p);
    return cuda_status(cudaGetLastError(), "mx gemm launch");
  }
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  if (dual) mx_gemm_kernel<true, false><<<grid, MX_THREADS, MxSmem<false>::BYTES, st>>>(ta, tb0, tb1, tc, p);
  else mx_gemm_kernel<false, false><<<grid, MX_THREADS, MxSmem<false>::BYTES, st>>>(ta, tb0, tb1, tc, p);
  return cuda_status(cudaGetLastError(), "mx gemm launch");
}

}  // namespace gsb
