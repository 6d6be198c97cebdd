// Persistent warp-specialised tcgen05 GEMM for 8-bit K-major operands
// (kind::i8 -> s32 accumulators, kind::f8f6f4 -> f32 accumulators) with the fused
// epilogues of the quantized-GEMM path:
//
//   EPI_I32      raw int32 accumulators                       (bit-exact tier)
//   EPI_DEQUANT  f16( acc * sA[m] * sB[n] )                   per-token x per-channel dequant
//   EPI_ROTARY   dequant, then rotate-half on the Q|K columns  (QKV projection; heads of 64, all of it rotated)
//   EPI_ROTARY_GEN  the same for heads of 64 or 128 columns of which the first 32, 64, 96 or 128 are rotated
//   EPI_SILU     f16( silu(gate) * up ), gate|up in one UMMA   (SwiGLU dual GEMM)
//   EPI_SILU_MX  the same product emitted as MXFP8: E4M3 elements + one E8M0 scale per 32 output columns
//   EPI_BIAS     f16( acc * sA[m] + b[n] )                    second GEMM of the low-rank input projection
//
// Three schedules share the epilogue (tiles are 128 rows x 256 accumulator columns):
//
//   SCHED_WRES   (K <= 512; dequant / SwiGLU): weight-stationary.  A CTA keeps its 256-row slice of W
//                (all of K, <= 128 KiB) in shared memory for the whole kernel and streams 128-row
//                blocks of A through a ring: L2 -> SM traffic per tile is the 64 KiB of A only.  CTAs
//                form (row-block group) x (W slice); the CTAs of a group walk the same row blocks, so
//                A comes from HBM once and from L2 for the other slices.
//   SCHED_ARES   (K <= 512; rotary): activation-stationary.  A CTA owns row blocks; the 64 KiB A block
//                stays in shared memory while every column block of W streams past it.  The per-row
//                epilogue state (token scale, the token's sin/cos row) is fetched once per row block.
//   SCHED_STREAM (any K, e.g. the K = 2048 down-projection): both operands stream through a ring.
//
//   warp 0      TMA producer   global -> 128B-swizzled smem (no multicast)
//   warp 1      TMEM owner + single-thread tcgen05.mma issue
//   warps 2,3   idle; they complete the first warpgroup, which gives its registers to the epilogue
//               (setmaxnreg: 56 per thread for warps 0-3, 224 for the two epilogue warpgroups)
//   warps 4..11 epilogue, free-running (no barrier between them): tcgen05.ld (thread = accumulator row,
//               next chunk in flight during the math of the current) -> math -> swizzled smem staging
//               -> TMA store (per-warp boxes of 16 rows x 64 fp16, issued in pairs)
//
// Two more template parameters give the dequant / rotary / SwiGLU kernels four forms (same bytes from each):
//   EW = 12    twelve epilogue warps (512 threads, 56 / 152 registers), three per SM sub-partition, each working on
//              64-column items of its lane quarter's stream of tiles
//   PAIR       two CTAs of a cluster on one tcgen05.mma.cta_group::2: 256 rows x 256 columns per MMA, half of the
//              tile's W rows in each CTA's shared memory, barriers of the first CTA collecting both CTAs' loads
//
// Two 256-column accumulator stages fill the 512 TMEM columns, so the epilogue of tile i overlaps the
// MMAs of tile i+1; a warp returns its part of a stage as soon as its last chunk is in registers.  The
// epilogue reads nothing from global memory inside its column loop: per-channel scales sit in shared
// memory, the per-token scale and the next tile's channel scales are fetched one tile ahead.
#pragma once
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace gsb {

enum : int { EPI_I32 = 0, EPI_DEQUANT = 1, EPI_ROTARY = 2, EPI_SILU = 3, EPI_SILU_MX = 4, EPI_BIAS = 5, EPI_ROTARY_GEN = 6 };
enum : int { KIND_I8 = 0, KIND_F8 = 1, KIND_F16 = 2 };   // F16: fp16 operands (K counted in bytes = 2 per element), f32 accumulate
enum : int { SCHED_STREAM = 0, SCHED_WRES = 1, SCHED_ARES = 2 };

constexpr int BM = 128;            // rows per tile (UMMA M)
constexpr int BN = 256;            // accumulator columns per tile (UMMA N)
constexpr int BK = 128;            // K bytes per smem stage (= one 128B swizzle row)
constexpr int UMMA_K = 32;         // K bytes per tcgen05.mma for 8-bit kinds
constexpr int ACC_STAGES = 2;
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 8;                            // warp e: TMEM lane quarter e % 4, column half e / 4
constexpr int FRONT_WARPS = 4;                          // warp 0 producer, warp 1 MMA, warps 2-3 idle (one warpgroup)
constexpr int GEMM_THREADS = 32 * (FRONT_WARPS + EPI_WARPS);
constexpr int FRONT_REGS = 56;                          // register budgets after setmaxnreg (per thread)
constexpr int EPI_REGS = 224;
constexpr int FRONT_REGS_FUSEQ = 80;                    // with the fused quantiser warps 2-3 hold four rows in flight
constexpr int EPI_REGS_FUSEQ = 208;
constexpr int A_STAGE_BYTES = BM * BK;                  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK;                  // 32 KiB
constexpr int RES_MAX_KBLOCKS = 4;                      // resident operand (W slice or A block): up to K = 512
constexpr int NSTAGE = 3;                               // ring depth of every schedule
constexpr int OUT_BOX_ROWS = 16;                        // output boxes of 16 rows x 64 fp16: full 128-byte lines,
constexpr int OUT_BOX_COLS = 64;                        // SWIZZLE_128B; a warp's 32 rows x 64 columns leave as two boxes
constexpr int OUT_BUF_BYTES = OUT_BOX_ROWS * OUT_BOX_COLS * 2;   // 2 KiB
constexpr int SCALE_BUF_BYTES = BN * 4;                 // channel scales of one tile, indexed by accumulator column (dual: gate | up)

// Shared-memory map (offsets from a 1 KiB-aligned base).
//   STREAM: [ring 3 x (A 16 KiB | B 32 KiB)]              [staging 8 warps x 4 x 2 KiB][scales 6 x 1 KiB][barriers]
//   WRES:   [W slice 4 x 32 KiB][A ring 3 x 16 KiB]       [staging 8 warps x 3 x 2 KiB][scales 1 KiB][barriers]
//   ARES:   [A block 4 x 16 KiB][B ring 3 x 32 KiB]       [staging 8 warps x 3 x 2 KiB][scales 6 x 1 KiB][barriers]
//   PAIR (two CTAs on one tcgen05.mma.cta_group::2): a CTA holds only HALF of the tile's W rows (16 KiB per K block), and
//   the memory that frees goes into deeper rings (5 stages streaming, 6 with a resident operand).
//   EW = 12 (twelve epilogue warps, each working on 64-column items): one box pair (4 KiB) of staging per warp.
template <int SCHED, bool PAIR = false, int EW = EPI_WARPS>
struct SmemMap {
  static constexpr int B_BYTES = PAIR ? B_STAGE_BYTES / 2 : B_STAGE_BYTES;      // W bytes per K block in one CTA
  static constexpr int NSTAGE = !PAIR ? gsb::NSTAGE : SCHED == SCHED_STREAM ? 5 : 6;
  static constexpr int RES_BYTES = SCHED == SCHED_WRES ? RES_MAX_KBLOCKS * B_BYTES
                                 : SCHED == SCHED_ARES ? RES_MAX_KBLOCKS * A_STAGE_BYTES : 0;
  static constexpr int STAGE_BYTES = SCHED == SCHED_WRES ? A_STAGE_BYTES
                                   : SCHED == SCHED_ARES ? B_BYTES : A_STAGE_BYTES + B_BYTES;
  static constexpr int RING_OFF = RES_BYTES;
  static constexpr int OUT_BUFS = EW == 12 ? 2 : (SCHED == SCHED_STREAM && !PAIR) ? 4 : 3;   // 2 KiB staging boxes per epilogue warp
  // Channel-scale buffers, filled by the producer beside each tile's first K block.  A weight-stationary
  // CTA keeps one column block, hence one buffer.  Otherwise tile j uses buffer j % 6: when the producer
  // fills it again (tile j + 6) it holds a ring slot the MMA warp freed at most ceil(NSTAGE / k_blocks) <= 3
  // tiles earlier (the deeper rings of a pair need k_blocks >= 2 for that; the host sends other shapes elsewhere), the MMA warp of tile t has been given the accumulator stage of tile t - 2 by every
  // epilogue warp, and a warp that has released tile t - 2 is done with tile t - 3: 3 + 3 = 6.
  static constexpr int SCALE_BUFS = SCHED == SCHED_WRES ? 1 : 6;
  static constexpr int OUT_OFF = RING_OFF + NSTAGE * STAGE_BYTES;
  static constexpr int SCALE_OFF = OUT_OFF + EW * OUT_BUFS * OUT_BUF_BYTES;
  // fused activation quantiser (activation-stationary only): the token scales of up to four row blocks in flight
  static constexpr int SA_OFF = SCALE_OFF + SCALE_BUFS * SCALE_BUF_BYTES;
  static constexpr int SA_BUFS = 4;
  static constexpr int SA_BYTES = SCHED == SCHED_ARES ? SA_BUFS * BM * 4 : 0;
  static constexpr int BAR_OFF = SA_OFF + SA_BYTES;
  static constexpr int USED = BAR_OFF + 512;
};
constexpr int GEMM_SMEM_BYTES = 227 * 1024;             // request the maximum; the base is aligned up to 1 KiB
static_assert(SmemMap<0>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<1>::USED + 1024 <= GEMM_SMEM_BYTES &&
              SmemMap<2>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<0, true>::USED + 1024 <= GEMM_SMEM_BYTES &&
              SmemMap<1, true>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<2, true>::USED + 1024 <= GEMM_SMEM_BYTES &&
              SmemMap<0, false, 12>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<1, false, 12>::USED + 1024 <= GEMM_SMEM_BYTES &&
              SmemMap<2, false, 12>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<0, true, 12>::USED + 1024 <= GEMM_SMEM_BYTES &&
              SmemMap<1, true, 12>::USED + 1024 <= GEMM_SMEM_BYTES && SmemMap<2, true, 12>::USED + 1024 <= GEMM_SMEM_BYTES,
              "shared memory budget");
static_assert(GEMM_SMEM_BYTES > 116 * 1024, "one CTA per SM is what makes the 512-column TMEM allocation safe");

constexpr unsigned int ST_BAD_SMEM_ALIGN = 1u << 8;

struct GemmParams {
  int M, N, K;                 // N = output columns (dual GEMM: columns of each of gate / up)
  int m_blocks, n_blocks, k_blocks;
  int n_groups;                // WRES: number of row-block groups (grid = n_groups * n_blocks)
  int m_major;                 // STREAM: a CTA walks all column blocks of a row block before the next (ARES always does)
  int ares_split;              // ARES: CTAs that share each row block of the last, incomplete round (1 = no sharing)
  void* C;                     // output base (direct-store path and int32 output)
  uint8_t* out_scale;          // EPI_SILU_MX: E8M0 scales [M, N/32]
  long long ld_scale;          //              row stride of out_scale in bytes
  long long ldc;               // output row stride in elements
  const float* scale_a;        // [M]
  const float* scale_b0;       // [N]   (dual: gate)
  const float* scale_b1;       // [N]   (dual: up)
  int scale_b_scalar;          // scale_b0 points to ONE value used for every column (scalar-quantised weights)
  const float* sin_tab;        // [seqlen_max, 32]
  const float* cos_tab;
  int seqlen;                  // runtime sequence length: angle row = (row + row_offset) % seqlen
  int rot_cols;                // 2 * nhead * head_dim: the Q and K columns
  int head_dim;                // EPI_ROTARY_GEN: 64 or 128 (EPI_ROTARY: 64)
  int rot_half;                // EPI_ROTARY_GEN: rotary_dim / 2, a multiple of 16 (EPI_ROTARY: 32); also the width of a sin / cos row
  int row_offset;              // global row index of this shard's row 0
  const __half* x_f16;         // fused activation quantiser: fp16 activations [M, K] (the int8 A operand is then made on chip)
  long long ldx;               //   row stride of x_f16 in elements
  float* scale_a_out;          //   optional: the token scales [M], as quantize_tensor would return them
  // Diagnostics, honoured only by a library built with -DGSB200_DIAG (never by the shipped one):
  int direct_store;            // 1: plain st.global from registers instead of smem + TMA store
  int ablate;                  // timing ablations (results are then wrong): 1 = skip the output stores, 2 = skip the epilogue body, 4 = skip the main loop, 8 = half of the epilogue warps skip their body
};
#ifdef GSB200_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif

// Role timers of a profiling build (-DGSB200_GEMM_PROF, never the shipped library): clocks spent in each role's
// waits, summed per CTA.
#ifdef GSB200_GEMM_PROF
__device__ long long g_gemm_prof[160][16];
#define GP_DECL(n) long long gp_##n = 0
#define GP_BEGIN(t) const long long t = clock64()
#define GP_END(n, t) gp_##n += clock64() - t
#define GP_STORE(slot, n) g_gemm_prof[blockIdx.x % 160][slot] = gp_##n
#else
#define GP_DECL(n) do { } while (0)
#define GP_BEGIN(t) do { } while (0)
#define GP_END(n, t) do { } while (0)
#define GP_STORE(slot, n) do { } while (0)
#endif

template <int KIND>
__device__ __forceinline__ float acc_to_float(uint32_t v) {
  if constexpr (KIND == KIND_I8) return static_cast<float>(static_cast<int32_t>(v));   // cvt.rn.f32.s32
  else return __uint_as_float(v);
}

// Dequantise two adjacent accumulator columns.  The per-token and per-channel scales are combined with
// the accumulator exactly as the reference kernels do: INT8 multiplies the two scales first and applies
// the product (cute/ampere_gemm_i8_quant_rmem.py:603,727); FP8 applies them left to right
// (fly/rdna_fp8_preshuffle_gemm.py:392-396).  sa2 = (sA, sA), sb2 = (sB[n], sB[n+1]).
template <int KIND>
__device__ __forceinline__ float2 dequant2(uint32_t a0, uint32_t a1, float2 sa2, float2 sb2) {
  const float2 acc = pk2(acc_to_float<KIND>(a0), acc_to_float<KIND>(a1));
  if constexpr (KIND == KIND_I8) return fmul2(acc, fmul2(sa2, sb2));
  else return fmul2(fmul2(acc, sa2), sb2);
}

// 8 consecutive columns -> 8 fp16 (one 16-byte piece).  s01/s23 hold the 8 per-channel scales as pairs.
template <int KIND>
__device__ __forceinline__ uint4 dequant_piece(const uint32_t* v, float2 sa2, float4 s_lo, float4 s_hi) {
  uint4 o;
  o.x = pack_half2_from(dequant2<KIND>(v[0], v[1], sa2, make_float2(s_lo.x, s_lo.y)));
  o.y = pack_half2_from(dequant2<KIND>(v[2], v[3], sa2, make_float2(s_lo.z, s_lo.w)));
  o.z = pack_half2_from(dequant2<KIND>(v[4], v[5], sa2, make_float2(s_hi.x, s_hi.y)));
  o.w = pack_half2_from(dequant2<KIND>(v[6], v[7], sa2, make_float2(s_hi.z, s_hi.w)));
  return o;
}

// 8 consecutive columns of the bias epilogue: f16( acc * sA + b[n] ), b in s_lo / s_hi.
template <int KIND>
__device__ __forceinline__ uint4 bias_piece(const uint32_t* v, float2 sa2, float4 s_lo, float4 s_hi) {
  auto one = [&](uint32_t a0, uint32_t a1, float2 b2) {
    return pack_half2_from(__ffma2_rn(pk2(acc_to_float<KIND>(a0), acc_to_float<KIND>(a1)), sa2, b2));
  };
  uint4 o;
  o.x = one(v[0], v[1], make_float2(s_lo.x, s_lo.y));
  o.y = one(v[2], v[3], make_float2(s_lo.z, s_lo.w));
  o.z = one(v[4], v[5], make_float2(s_hi.x, s_hi.y));
  o.w = one(v[6], v[7], make_float2(s_hi.z, s_hi.w));
  return o;
}

// Staging boxes are 32 rows x 32 fp16 in the 64-byte swizzle a SWIZZLE_64B TMA store expects: the 16-byte
// piece p (0..3) of row r lives at r*64 + ((p ^ ((r >> 1) & 3)) * 16), which is also conflict-free for
// 16-byte shared stores by a warp whose lane index is the row.
struct true_tag { static constexpr bool value = true; };
struct false_tag { static constexpr bool value = false; };

// A CTA's walk over its tiles (row block m, column block n), advanced without divisions:
//   WRES:               fixed column block, row blocks group, group + n_groups, ...
//   ARES, STREAM m_major: row blocks cta, cta + grid, ...; all column blocks of one before the next
//   STREAM:             tiles cta, cta + grid, ... with the column block fastest
//   PAIR: the walk's unit is the CTA pair (pair = blockIdx.x / 2) and a "row block" is 256 rows, 128 per CTA.
template <int SCHED, bool PAIR = false>
struct TileWalk {
  static __device__ __forceinline__ int cta() { return PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x; }
  static __device__ __forceinline__ int ncta() { return PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x; }
  int m, n;
  int dm, dn;      // STREAM with the column block fastest: what one step of `grid` tiles adds
  int n_lo, n_hi;  // row-block-major walks: this CTA's column blocks of row block m are [n_lo, n_hi)
  int visit;       // row-block-major walks: how many row blocks this CTA has left behind
  // Row blocks cta, cta + grid, ... while whole rounds last.  The row blocks left over (fewer than CTAs) would
  // keep some SMs busy for a whole row block while the others idle: with the activation-stationary schedule each of
  // them is shared by p.ares_split CTAs, which take consecutive column blocks of it (each loads the A block).
  __device__ __forceinline__ void set_visit(const GemmParams& p) {
    const int grid = ncta(), full = p.m_blocks / grid, rem = p.m_blocks - full * grid;
    m = p.m_blocks;                                   // nothing left unless one of the cases below applies
    n_lo = 0; n_hi = p.n_blocks;
    if (visit < full) {
      m = cta() + visit * grid;
    } else if (visit == full && rem > 0) {
      const int S = (SCHED == SCHED_ARES && p.ares_split > 1) ? p.ares_split : 1;
      const int per = (p.n_blocks + S - 1) / S;
      const int c = cta();
      if (c < rem * S && (c % S) * per < p.n_blocks) {
        m = full * grid + c / S;
        n_lo = (c % S) * per;
        n_hi = n_lo + per < p.n_blocks ? n_lo + per : p.n_blocks;
      }
    }
    n = n_lo;
  }
  __device__ __forceinline__ void start(const GemmParams& p) {
    dm = dn = 0; n_lo = 0; n_hi = p.n_blocks; visit = 0;
    if constexpr (SCHED == SCHED_WRES) {
      n = cta() % p.n_blocks; m = cta() / p.n_blocks;
    } else {
      if (SCHED == SCHED_ARES || p.m_major) set_visit(p);
      else {
        m = cta() / p.n_blocks; n = cta() % p.n_blocks;
        dm = ncta() / p.n_blocks; dn = ncta() % p.n_blocks;
      }
    }
  }
  __device__ __forceinline__ bool valid(const GemmParams& p) const { return m < p.m_blocks; }
  __device__ __forceinline__ bool first() const { return n == n_lo; }       // first / last tile of this CTA's stay on row block m
  __device__ __forceinline__ bool last() const { return n == n_hi - 1; }
  __device__ __forceinline__ void next(const GemmParams& p) {
    if constexpr (SCHED == SCHED_WRES) {
      m += p.n_groups;
    } else {
      if (SCHED == SCHED_ARES || p.m_major) { if (++n == n_hi) { ++visit; set_visit(p); } }
      else { m += dm; n += dn; if (n >= p.n_blocks) { n -= p.n_blocks; ++m; } }
    }
  }
  // row block of this CTA's next stay, or -1
  __device__ __forceinline__ int next_row_block(const GemmParams& p) const {
    TileWalk nx = *this;
    nx.n = nx.n_hi - 1;
    nx.next(p);
    return nx.valid(p) ? nx.m : -1;
  }
};

// Register budgets of the twelve-epilogue-warp form (512 threads compiled at 128 registers: 128 x 56 + 384 x 152 = 65536).
constexpr int EW12_THREADS = 32 * (FRONT_WARPS + 12);
constexpr int EW12_FRONT_REGS = 56;
constexpr int EW12_EPI_REGS = 152;
constexpr int EW12_REG_POOL_NEEDED = 32 * (FRONT_WARPS * EW12_FRONT_REGS + 12 * EW12_EPI_REGS);

template <int KIND, int EPI, int SCHED, bool FUSEQ = false, bool PAIR = false, int EW = EPI_WARPS>
__global__ void __launch_bounds__(32 * (FRONT_WARPS + EW), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b0,
                    const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_c,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using Map = SmemMap<SCHED, PAIR, EW>;
  static_assert(EW == EPI_WARPS || (EW == 12 && !FUSEQ && (EPI == EPI_DEQUANT || EPI == EPI_ROTARY || EPI == EPI_SILU)),
                "twelve epilogue warps: built for the dequant, rotary and SwiGLU epilogues");
  constexpr int NTHREADS = 32 * (FRONT_WARPS + EW);
  // EW = 12: the epilogue's unit of work is an ITEM, 32 rows x 64 output columns.  Every epilogue warp hands every
  // accumulator stage back once (also for a tile in which it has no item: the MMA warp may then never run more than
  // two tiles ahead of ANY epilogue warp, which is what keeps each warp's barrier phases in step).
  constexpr int ITEMS = (EPI == EPI_SILU || EPI == EPI_SILU_MX) ? 2 : 4;
  constexpr int ACC_RELEASES = EW * (PAIR ? 2 : 1);
  using Walk = TileWalk<SCHED, PAIR>;
  constexpr int NSTAGE = Map::NSTAGE;
  constexpr bool WRES = SCHED == SCHED_WRES;
  constexpr bool ARES = SCHED == SCHED_ARES;
  constexpr int OUT_BUFS = Map::OUT_BUFS;
  // (the offset of the dynamic window is the same in every CTA of a launch, so both CTAs of a pair take this exit or neither)
  if (smem + Map::USED > smem_raw + GEMM_SMEM_BYTES) {     // cannot happen with a 1 KiB-aligned window; never run off the end
    if (threadIdx.x == 0) atomicOr(&g_status[0], ST_BAD_SMEM_ALIGN);
    return;
  }
  uint8_t* res_base = smem;                                // WRES: W slice, ARES: A block (k_blocks pieces)
  uint8_t* ring = smem + Map::RING_OFF;
  uint8_t* out_base = smem + Map::OUT_OFF;
  float* scale_base = reinterpret_cast<float*>(smem + Map::SCALE_OFF);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Map::BAR_OFF);
  uint64_t* full_bar = bars;                               // [NSTAGE]  ring stage filled
  uint64_t* empty_bar = bars + NSTAGE;                     // [NSTAGE]  ring stage consumed
  uint64_t* acc_full = bars + 2 * NSTAGE;                  // [ACC_STAGES]
  uint64_t* acc_empty = acc_full + ACC_STAGES;             // [ACC_STAGES]
  uint64_t* res_full = acc_empty + ACC_STAGES;             // [RES_MAX_KBLOCKS] resident piece landed (WRES uses [0] only)
  uint64_t* res_empty = res_full + RES_MAX_KBLOCKS;        // [RES_MAX_KBLOCKS] ARES: A piece no longer needed
  uint64_t* sa_ready = res_empty + RES_MAX_KBLOCKS;        // [SA_BUFS] FUSEQ: token scales of a row block written
  uint64_t* sc_full = sa_ready + Map::SA_BUFS;             // [SCALE_BUFS] PAIR: channel scales of a tile landed (in this CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sc_full + Map::SCALE_BUFS);
  static_assert(!(PAIR && FUSEQ), "the fused quantiser is built for the single-CTA kernel");
  // PAIR: CTA rank 0 of the pair issues the MMAs; its barriers collect both CTAs' loads and releases
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  auto rowblk = [&](int m) { return PAIR ? 2 * m + (int)rank : m; };      // walk unit -> 128-row block of this CTA
  float* sa_s = reinterpret_cast<float*>(smem + Map::SA_OFF);
  static_assert(!FUSEQ || (SCHED == SCHED_ARES && KIND == KIND_I8), "the fused quantiser feeds the resident int8 A block");
  const AbortFlag abort_flag{smem_u32(tmem_slot + 1)};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr bool DUAL = (EPI == EPI_SILU || EPI == EPI_SILU_MX);
  constexpr int OUT_COLS_PER_TILE = DUAL ? BN / 2 : BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < ACC_STAGES; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], ACC_RELEASES); }
    for (int s = 0; s < Map::SCALE_BUFS; ++s) mbar_init(&sc_full[s], 1);
    // FUSEQ: the two quantiser warps both report a finished A block
    for (int s = 0; s < RES_MAX_KBLOCKS; ++s) { mbar_init(&res_full[s], FUSEQ ? 2 : 1); mbar_init(&res_empty[s], 1); }
    for (int s = 0; s < Map::SA_BUFS; ++s) mbar_init(&sa_ready[s], 2);
    abort_flag.set(0);
    fence_mbar_init();
    prefetch_tmap(&tm_a); prefetch_tmap(&tm_b0); prefetch_tmap(&tm_b1);
    if (EPI != EPI_I32) prefetch_tmap(&tm_c);
  }
  if (warp == 1) {
    if constexpr (PAIR) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  }
  // Channel scales normally arrive by bulk copy from the producer; without a per-channel vector (none given,
  // or one scalar for all columns) every buffer is filled with the constant once, here.
  const bool copy_scales = EPI != EPI_I32 && p.scale_b0 != nullptr && !p.scale_b_scalar;
  if (EPI != EPI_I32 && !copy_scales) {
    const float v = p.scale_b0 ? __ldg(p.scale_b0) : 1.f;
    for (int i = threadIdx.x; i < Map::SCALE_BUFS * BN; i += NTHREADS) scale_base[i] = v;
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();             // the other CTA's barriers are initialised before anything arrives at them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const unsigned int budget = spin_budget();          // bound of every wait below, fetched once

  // The register re-split sits inside each role's branch: code placed after the point where the two
  // branches meet would be compiled for the smaller budget.
  if (warp < FRONT_WARPS) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(EW == 12 ? EW12_FRONT_REGS : FUSEQ ? FRONT_REGS_FUSEQ : FRONT_REGS));
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; bool ok = true;
      GP_DECL(p_total); GP_DECL(p_empty); GP_BEGIN(gp_p0);
      // channel scales of the tile whose first output column is n0 -> buffer dst, bytes reported to bar
      auto scale_bytes = [&](int n0) -> uint32_t {
        return copy_scales ? (uint32_t)((DUAL ? 2 : 1) * min(OUT_COLS_PER_TILE, p.N - n0) * 4) : 0u;
      };
      auto load_scales = [&](float* dst, int n0, uint64_t* bar) {
        if (!copy_scales) return;
        const uint32_t bytes = (uint32_t)(min(OUT_COLS_PER_TILE, p.N - n0) * 4);
        bulk_load(dst, p.scale_b0 + n0, bytes, bar);
        if constexpr (DUAL) bulk_load(dst + BN / 2, p.scale_b1 + n0, bytes, bar);
      };
      // `bytes` = what ONE CTA loads onto the barrier; of a pair only the first CTA arrives, for both
      auto expect = [&](uint64_t* bar, uint32_t bytes) {
        if constexpr (!PAIR) mbar_arrive_expect_tx(bar, bytes);
        else if (rank == 0) mbar_arrive_expect_tx(bar, 2 * bytes);
      };
      auto load_a = [&](void* dst, uint64_t* bar, int x, int y) {
        if constexpr (PAIR) tma_load_2d_pair(dst, &tm_a, mapa_shared(smem_u32(bar), 0), x, y);
        else tma_load_2d(dst, &tm_a, bar, x, y);
      };
      // the tile's W rows: both halves, or of a pair the half of this CTA (first CTA: rows n0.., second: rows n1..)
      auto load_b = [&](uint8_t* dst, uint64_t* bar, int x, int n0, int n1) {
        if constexpr (PAIR) {
          tma_load_2d_pair(dst, rank ? &tm_b1 : &tm_b0, mapa_shared(smem_u32(bar), 0), x, rank ? n1 : n0);
        } else {
          tma_load_2d(dst, &tm_b0, bar, x, n0);
          tma_load_2d(dst + (BN / 2) * BK, &tm_b1, bar, x, n1);
        }
      };
      // PAIR: a tile's channel scales report to a barrier of this CTA (an untiled bulk copy cannot report to the other CTA)
      auto load_scales_own = [&](int sb, int n0) {
        const uint32_t bytes = scale_bytes(n0);
        if (bytes) { mbar_arrive_expect_tx(&sc_full[sb], bytes); load_scales(scale_base + sb * BN, n0, &sc_full[sb]); }
      };
      int sbuf = 0;                           // scale buffer of the current tile
      // WRES: every K block of the resident W slice has a barrier of its own, and a single CTA requests them one by one
      // beside the first tile's A blocks, so the first MMAs start after 48 KiB have landed instead of 144 (a pair asks
      // for its W halves up front: its producer has no registers left for the interleaved form)
      auto load_w_block = [&](int kb, int n0, int n1) {
        mbar_arrive_expect_tx(&res_full[kb], B_STAGE_BYTES + (kb == 0 ? scale_bytes(n0) : 0u));
        if (kb == 0) load_scales(scale_base, n0, &res_full[0]);
        load_b(res_base + kb * Map::B_BYTES, &res_full[kb], kb * BK, n0, n1);
      };
      if constexpr (WRES && PAIR) {
        const int n0 = (Walk::cta() % p.n_blocks) * OUT_COLS_PER_TILE;
        const int n1 = DUAL ? n0 : n0 + BN / 2;
        load_scales_own(0, n0);
        expect(&res_full[0], p.k_blocks * Map::B_BYTES);
        for (int kb = 0; kb < p.k_blocks; ++kb) load_b(res_base + kb * Map::B_BYTES, &res_full[0], kb * BK, n0, n1);
      }
      uint32_t rph = 0;                       // ARES: phase of the resident-A barriers, flips per row block
      int rot = 0;                            // WRES: it % n_blocks, which CTA of a group asks for the L2 prefetch
      Walk tw; tw.start(p);
      for (int it = 0; ok && !(kDiag && (p.ablate & 4)) && tw.valid(p); ++it, tw.next(p)) {
        const int n_blk = tw.n;
        const int m0 = rowblk(tw.m) * BM;
        const int n0 = n_blk * OUT_COLS_PER_TILE;
        const int n1 = DUAL ? n0 : n0 + BN / 2;
        const bool rb_first = tw.first();      // first tile of this CTA's stay on the row block
        if (ARES && rb_first && it != 0) rph ^= 1;
        // A comes from HBM with a latency the small ring cannot cover: ask for it in L2 well ahead.
        //   WRES: the row block two tiles on (one CTA of the group asks, the others find it in L2)
        //   ARES: this CTA's next row block, when the last tile of the current one is requested
        if constexpr (WRES) {
          const int pm = tw.m + 2 * p.n_groups;
          if (pm < p.m_blocks && rot == n_blk)
            for (int kb = 0; kb < p.k_blocks; ++kb) tma_prefetch_l2_2d(&tm_a, kb * BK, rowblk(pm) * BM);
          if (++rot == p.n_blocks) rot = 0;
        } else if constexpr (ARES) {
          // (asked for at the row block's first tile, six tiles ahead, the lines are gone from L2 again when the
          // block is loaded -- 201 MB of output pass through it meanwhile -- and the wait for the resident block doubles)
          if (!FUSEQ && tw.n == tw.n_hi - 1) {
            const int nm = tw.next_row_block(p);
            if (nm >= 0)
              for (int kb = 0; kb < p.k_blocks; ++kb) tma_prefetch_l2_2d(&tm_a, kb * BK, rowblk(nm) * BM);
          }
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if constexpr (ARES && !FUSEQ) {
            if (rb_first) {                   // new row block: refill this K piece of A once its last reader retired
              if (!mbar_wait(&res_empty[kb], rph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, (0u << 16) | 0x300 | kb, budget)) { ok = false; break; }
              expect(&res_full[kb], A_STAGE_BYTES);
              load_a(res_base + kb * A_STAGE_BYTES, &res_full[kb], kb * BK, m0);
            }
          }
          GP_BEGIN(gp_t);
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, ST_TIMEOUT_PRODUCER, (0u << 16) | s, budget)) { ok = false; break; }
          GP_END(p_empty, gp_t);
          uint8_t* st = ring + s * Map::STAGE_BYTES;
          // the scales ride on the first K block (of a pair: on a barrier of their own)
          const uint32_t sc_bytes = (!PAIR && !WRES && kb == 0) ? scale_bytes(n0) : 0u;
          if (PAIR && !WRES && kb == 0) load_scales_own(sbuf, n0);
          if constexpr (WRES) {
            if (!PAIR && it == 0) load_w_block(kb, n0, n1);
            expect(&full_bar[s], A_STAGE_BYTES);
            load_a(st, &full_bar[s], kb * BK, m0);
          } else if constexpr (ARES) {
            expect(&full_bar[s], Map::B_BYTES + sc_bytes);
            if (!PAIR && kb == 0) load_scales(scale_base + sbuf * BN, n0, &full_bar[s]);
            load_b(st, &full_bar[s], kb * BK, n0, n1);
          } else {
            expect(&full_bar[s], A_STAGE_BYTES + Map::B_BYTES + sc_bytes);
            if (!PAIR && kb == 0) load_scales(scale_base + sbuf * BN, n0, &full_bar[s]);
            load_a(st, &full_bar[s], kb * BK, m0);
            load_b(st + A_STAGE_BYTES, &full_bar[s], kb * BK, n0, n1);
          }
          if (++s == NSTAGE) { s = 0; ph ^= 1; }
        }
        if (!WRES && ++sbuf == Map::SCALE_BUFS) sbuf = 0;
      }
      GP_END(p_total, gp_p0); GP_STORE(3, p_empty); GP_STORE(4, p_total);
      if (!ok) {                       // give copies already in flight time to land before the CTA exits
        long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && rank == 0) {
      // s8 x s8 -> s32 | e4m3 x e4m3 -> f32 | f16 x f16 -> f32 (format code 0 means e4m3 resp. f16 in its kind)
      constexpr int MMA_M = PAIR ? 2 * BM : BM;          // a pair's MMA spans both CTAs' 128 rows
      constexpr uint32_t idesc = (KIND == KIND_I8) ? umma_idesc(2, 1, 1, MMA_M, BN) : umma_idesc(1, 0, 0, MMA_M, BN);
      // completion of the MMAs issued so far -> the barrier (of a pair: the same barrier in both CTAs)
      auto commit = [&](uint64_t* bar) {
        if constexpr (PAIR) umma_commit_pair_both(bar);
        else umma_commit(bar);
      };
      int s = 0; uint32_t ph = 0; bool ok = true;
      GP_DECL(m_total); GP_DECL(m_acc); GP_DECL(m_full); GP_DECL(m_res); GP_BEGIN(gp_m0);
      if (WRES && PAIR && !(kDiag && (p.ablate & 4))) {       // a pair waits for its whole W slice (one barrier) before the first MMA
        ok = mbar_wait(&res_full[0], 0, abort_flag, ST_TIMEOUT_MMA, (1u << 16) | 0x200, budget);
        tc_fence_after();
      }
      uint32_t rph = 0;
      Walk tw; tw.start(p);
      for (int it = 0; ok && tw.valid(p); ++it, tw.next(p)) {
        const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
        // (of a pair: the other CTA's epilogue warps arrive here too; what they hand over is tensor memory, ordered by the
        // tcgen05 fences on both sides)
        GP_BEGIN(gp_ta);
        if (!mbar_wait(&acc_empty[as], aph ^ 1, abort_flag, ST_TIMEOUT_MMA, (1u << 16) | 0x100 | as, budget)) { ok = false; break; }
        GP_END(m_acc, gp_ta);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        const bool rb_first = tw.first(), rb_last = tw.last();
        if (ARES && rb_first && it != 0) rph ^= 1;
        for (int kb = 0; kb < p.k_blocks && !(kDiag && (p.ablate & 4)); ++kb) {
          GP_BEGIN(gp_tr0);
          if constexpr (ARES) {
            if (rb_first && !mbar_wait(&res_full[kb], rph, abort_flag, ST_TIMEOUT_MMA, (1u << 16) | 0x300 | kb, budget)) { ok = false; break; }
          } else if constexpr (WRES && !PAIR) { // the W slice arrives during the first tile, K block by K block
            if (it == 0 && !mbar_wait(&res_full[kb], 0, abort_flag, ST_TIMEOUT_MMA, (1u << 16) | 0x200 | kb, budget)) { ok = false; break; }
          }
          GP_END(m_res, gp_tr0);
          GP_BEGIN(gp_tf);
          if (!mbar_wait(&full_bar[s], ph, abort_flag, ST_TIMEOUT_MMA, (1u << 16) | s, budget)) { ok = false; break; }
          GP_END(m_full, gp_tf);
          tc_fence_after();
          uint32_t a_addr, b_addr;
          const uint32_t st = smem_u32(ring + s * Map::STAGE_BYTES);
          if constexpr (WRES) { a_addr = st; b_addr = smem_u32(res_base + kb * Map::B_BYTES); }
          else if constexpr (ARES) { a_addr = smem_u32(res_base + kb * A_STAGE_BYTES); b_addr = st; }
          else { a_addr = st; b_addr = st + A_STAGE_BYTES; }
          const uint64_t a_desc = umma_smem_desc_sw128(a_addr);
          const uint64_t b_desc = umma_smem_desc_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t koff = (uint64_t)((k * UMMA_K) >> 4);
            if constexpr (PAIR) {
              if constexpr (KIND == KIND_I8) umma_i8_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
              else if constexpr (KIND == KIND_F16) umma_f16_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
              else umma_f8_pair(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
            } else {
              if constexpr (KIND == KIND_I8) umma_i8(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
              else if constexpr (KIND == KIND_F16) umma_f16(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
              else umma_f8(d_tmem, a_desc + koff, b_desc + koff, idesc, (kb | k) != 0);
            }
          }
          commit(&empty_bar[s]);               // ring stage reusable once these MMAs retire
          if (ARES && rb_last) commit(&res_empty[kb]);        // last reader of this A piece
          if (++s == NSTAGE) { s = 0; ph ^= 1; }
        }
        if (ok) commit(&acc_full[as]);          // accumulator complete
      }
      GP_END(m_total, gp_m0); GP_STORE(0, m_total); GP_STORE(1, m_acc); GP_STORE(2, m_full); GP_STORE(13, m_res);
    }
  } else if constexpr (FUSEQ) {
    // ------------------------------ activation quantiser (warps 2 and 3) ------------------------------
    // Per-token absmax quantisation of this CTA's next row block, fp16 -> int8, written straight into the resident
    // A block in the layout the MMAs read (rows of 128 bytes per K piece, 128-byte swizzle), with the arithmetic
    // of ptq_kernel: qs = fl(fl(1 / amax) * 127), q = rne(x * qs), scale = fl(1 / qs).  One row per warp and
    // round: lane l holds the 16 elements 16 l .. 16 l + 15 (K <= 512), i.e. chunk l % 8 of K piece l / 8.
    // The block can only be rewritten once the MMAs of the previous row block have retired, and the next MMAs wait
    // for it; the epilogue, which is what bounds this kernel, still has the last two tiles to drain meanwhile.
    const int wq = warp - 2;
    const int kvec = p.K >> 4;                          // lanes that hold data
    int rbi = 0;
    bool ok = true;
    for (int m_blk = blockIdx.x; ok && m_blk < p.m_blocks; m_blk += gridDim.x, ++rbi) {
      // the rows of the row block after this one go to L2 now (128-byte lines; 2 KiB per lane of this warp's half)
      {
        const long long nm = (long long)(m_blk + (int)gridDim.x) * BM;
        if (m_blk + (int)gridDim.x < p.m_blocks) {
          for (int r = wq * 64 + (lane >> 3); r < wq * 64 + 64; r += 4) {
            const long long row = nm + r;
            if (row < p.M && (lane & 7) * 64 < p.K)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(p.x_f16 + row * p.ldx + (lane & 7) * 64));
          }
        }
      }
      if (rbi > 0) {
        for (int kb = 0; kb < p.k_blocks; ++kb)
          if (!mbar_wait(&res_empty[kb], (uint32_t)(rbi - 1) & 1u, abort_flag, ST_TIMEOUT_PRODUCER, (0u << 16) | 0x400 | kb, budget)) { ok = false; break; }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      float* sa_dst = sa_s + (rbi & (Map::SA_BUFS - 1)) * BM;
      const long long row0 = (long long)m_blk * BM;
      const uint32_t dst_lane = (uint32_t)((lane >> 3) * A_STAGE_BYTES);      // K piece of this lane
      // rows wq, wq + 2, ... of the block, four per round so that their loads are in flight together
      for (int r0 = wq; r0 < BM; r0 += 8) {
        uint4 raw[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long row = row0 + r0 + 2 * j;
          raw[j][0] = raw[j][1] = make_uint4(0u, 0u, 0u, 0u);
          if (row < p.M && lane < kvec) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x_f16 + row * p.ldx + lane * 16);
            raw[j][0] = __ldg(src); raw[j][1] = __ldg(src + 1);
          }
        }
        // the four rows go through every stage together, so that their shuffle and reciprocal chains overlap
        float amax[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __half2 m2 = __float2half2_rn(0.f);
          const __half2* h = reinterpret_cast<const __half2*>(&raw[j][0]);
#pragma unroll
          for (int k = 0; k < 8; ++k) m2 = __hmax2(m2, __habs2(h[k]));
          amax[j] = fmaxf(__low2float(m2), __high2float(m2));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
#pragma unroll
          for (int j = 0; j < 4; ++j) amax[j] = fmaxf(amax[j], __shfl_xor_sync(0xffffffffu, amax[j], d));
        }
        float qs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) qs[j] = __fmul_rn(__frcp_rn(fmaxf(amax[j], 1e-8f)), 127.0f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = r0 + 2 * j;
          const __half2* h = reinterpret_cast<const __half2*>(&raw[j][0]);
          const float2 q2 = make_float2(qs[j], qs[j]);
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f0 = __half22float2(h[2 * k]), f1 = __half22float2(h[2 * k + 1]);
            const float2 a2 = __fmul2_rn(f0, q2), b2 = __fmul2_rn(f1, q2);
            uint32_t hi, lo;
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(__float2int_rn(b2.y)), "r"(__float2int_rn(b2.x)), "r"(0u));
            asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(lo) : "r"(__float2int_rn(a2.y)), "r"(__float2int_rn(a2.x)), "r"(hi));
            w[k] = lo;
          }
          if (lane < kvec)
            *reinterpret_cast<uint4*>(res_base + dst_lane + r * 128 + (((lane & 7) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if (lane < 4) {                                  // lane j reports row j of the round
          const int r = r0 + 2 * lane;
          const long long row = row0 + r;
          const float myqs = lane == 0 ? qs[0] : lane == 1 ? qs[1] : lane == 2 ? qs[2] : qs[3];
          const float sc = row < p.M ? __frcp_rn(myqs) : 0.f;
          sa_dst[r] = sc;
          if (p.scale_a_out && row < p.M) p.scale_a_out[row] = sc;
        }
      }
      fence_proxy_async_smem();                        // the stores above before the MMAs' reads of the block
      __syncwarp();
      if (lane == 0) {
        for (int kb = 0; kb < p.k_blocks; ++kb) mbar_arrive(&res_full[kb]);
        mbar_arrive(&sa_ready[rbi & (Map::SA_BUFS - 1)]);
      }
    }
  }
  } else if constexpr (EW == 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(EW12_EPI_REGS));
    // ------------------------------ epilogue, twelve warps ----------------------------------
    // Three warps per SM sub-partition (the eight-warp epilogue is bound by the latency of each warp's own chain:
    // tensor-memory load -> arithmetic -> staging -> store issue).  Warp e reads TMEM lane quarter e % 4.  The
    // quarter's work is a stream of items -- (tile, 64-column group): a head of the QKV projection, 64 gate + 64 up
    // columns of the SwiGLU -- dealt to its three warps in turn.  An item loads its accumulator columns, computes,
    // stages one pair of 16-row boxes and issues their TMA stores; a warp returns the accumulator stage to the MMA
    // warp when the columns of its last item of the tile are in registers.
    const int e = warp - FRONT_WARPS;      // 0..11
    const int q = warp & 3;                // TMEM lane quarter
    const int j = e >> 2;                  // which of the quarter's three warps
    uint8_t* out_buf = out_base + e * 2 * OUT_BUF_BYTES;
    // this thread's 128-byte box row (lanes 0-15: first box, 16-31: second); its 16-byte piece pc sits at
    // ((pc ^ (lane & 7)) << 4) in the row (128-byte swizzle)
    uint8_t* const stg_row = out_buf + (lane < 16 ? 0 : OUT_BUF_BYTES) + (lane & 15) * 128;
    const int stg_sw = lane & 7;
    float sa = 0.f;
    float2 sn2[EPI == EPI_ROTARY ? 16 : 1], cs2[EPI == EPI_ROTARY ? 16 : 1];
    int cur_m_blk = -1;
    bool trig_scaled = false;
    int sbuf = 0;
    int base3 = 0;                         // (tiles so far * ITEMS) % 3
    GP_DECL(e_total); GP_DECL(e_acc); GP_DECL(e_read); GP_DECL(e_ld); GP_BEGIN(gp_e0);
    Walk tw; tw.start(p);
    for (int it = 0; tw.valid(p); ++it, tw.next(p)) {
      const int m_blk = rowblk(tw.m), n_blk = tw.n;
      const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
      const int n0 = n_blk * OUT_COLS_PER_TILE;
      const int row_base = m_blk * BM + q * 32;
      int first = j - base3; if (first < 0) first += 3;          // this warp's first item of the tile
      base3 += ITEMS % 3; if (base3 >= 3) base3 -= 3;
      // per-row state of a new row block, asked for before the accumulator wait
      if (first < ITEMS && m_blk != cur_m_blk) {
        cur_m_blk = m_blk;
        const long long r = (long long)row_base + lane;
        sa = (r < p.M) ? (p.scale_a ? ldg_f_here(p.scale_a + r) : 1.f) : 0.f;
        if constexpr (EPI == EPI_ROTARY) {
          trig_scaled = false;
          const int pos = r < p.M ? (int)((r + p.row_offset) % p.seqlen) : 0;
          const float* s4 = p.sin_tab + (long long)pos * 32;
          const float* c4 = p.cos_tab + (long long)pos * 32;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(sn2[2 * k].x), "=f"(sn2[2 * k].y), "=f"(sn2[2 * k + 1].x), "=f"(sn2[2 * k + 1].y) : "l"(s4 + 4 * k));
            asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(cs2[2 * k].x), "=f"(cs2[2 * k].y), "=f"(cs2[2 * k + 1].x), "=f"(cs2[2 * k + 1].y) : "l"(c4 + 4 * k));
          }
        }
      }
      // every warp follows every tile's barrier (also tiles in which it has no item), so the phase it waits for is
      // always the next one
      GP_BEGIN(gp_tw);
      const bool got = mbar_wait(&acc_full[as], aph, abort_flag, ST_TIMEOUT_EPILOGUE, (2u << 16) | as, budget);
      GP_END(e_acc, gp_tw);
      uint32_t agreed = __all_sync(0xffffffffu, got) ? 1u : 0u;
      if (!agreed) break;
      asm volatile("" : "+r"(agreed));     // the scale address below stays dependent on the wait
      tc_fence_after();
      if constexpr (PAIR) {
        if (copy_scales && !(kDiag && (p.ablate & 4))) {
          const bool have = mbar_wait(&sc_full[sbuf], (uint32_t)(WRES ? 0 : it / Map::SCALE_BUFS) & 1u, abort_flag,
                                      ST_TIMEOUT_EPILOGUE, (2u << 16) | 0x600 | sbuf, budget);
          if (!__all_sync(0xffffffffu, have)) break;
        }
      }
      const uint32_t sc_tile = smem_u32(scale_base + sbuf * BN) + ((agreed - 1u) << 2);
      if (!WRES && ++sbuf == Map::SCALE_BUFS) sbuf = 0;
      const uint32_t t_tile = tmem_base + as * BN + ((uint32_t)(q * 32) << 16);
      const float2 sa2 = pk2(sa, sa);
      auto release_stage = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[as]), 0));
          else mbar_arrive(&acc_empty[as]);
        }
      };
      if (first >= ITEMS) release_stage();   // no item in this tile
#pragma unroll 1
      for (int c = first; c < ITEMS; c += 3) {
        const int n = n0 + 64 * c;           // first output column of the item
        const bool last_item = c + 3 >= ITEMS;
        auto release = [&]() { if (last_item) release_stage(); };
        if (row_base >= p.M || n >= p.N || (kDiag && (p.ablate & 2))) { release(); continue; }
        // the stores of this warp's previous item have read the staging boxes
        auto stage_begin = [&]() {
          GP_BEGIN(gp_tr);
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          GP_END(e_read, gp_tr);
        };
        auto put = [&](int piece, uint4 o) { *reinterpret_cast<uint4*>(stg_row + ((piece ^ stg_sw) << 4)) = o; };
        auto stage_end = [&]() {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && !(kDiag && (p.ablate & 1))) {
            // the two 16-row boxes lie one after the other: one store of a 32-row box (this form's output map), which
            // clips the rows past M
            tma_store_2d(&tm_c, out_buf, n, row_base);
            tma_store_commit();
          }
        };
        if constexpr (EPI == EPI_DEQUANT) {
          const uint32_t sc = sc_tile + 64 * c * 4;
          uint32_t va[32], vb[32];
          tmem_ld_32x32b_x32(t_tile + 64 * c, va);
          tmem_ld_32x32b_x32(t_tile + 64 * c + 32, vb);
          tmem_ld_wait(va, vb);
          release();
          stage_begin();
#pragma unroll
          for (int k = 0; k < 4; ++k) put(k, dequant_piece<KIND>(&va[8 * k], sa2, lds_f4_ro(sc + 32 * k), lds_f4_ro(sc + 32 * k + 16)));
#pragma unroll
          for (int k = 0; k < 4; ++k) put(4 + k, dequant_piece<KIND>(&vb[8 * k], sa2, lds_f4_ro(sc + 128 + 32 * k), lds_f4_ro(sc + 128 + 32 * k + 16)));
          stage_end();
        } else if constexpr (EPI == EPI_SILU) {
          // gate columns 64 c .. 64 c + 63 of the tile's first half, the matching up columns BN / 2 further on
          const uint32_t scg = sc_tile + 64 * c * 4, scu = scg + (BN / 2) * 4;
          const float2 sah2 = pk2(0.5f * sa, 0.5f * sa);      // the gate is dequantised straight to gate / 2 (exact halving)
          uint32_t g[16], u[16];
#pragma unroll
          for (int h = 0; h < 4; ++h) {                      // 16 output columns -> pieces 2 h, 2 h + 1
            tmem_ld_32x32b_x16(t_tile + 64 * c + 16 * h, g);
            tmem_ld_32x32b_x16(t_tile + BN / 2 + 64 * c + 16 * h, u);
            tmem_ld_wait(g, u);
            if (h == 0) stage_begin();
            if (h == 3) release();
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int k = 2 * h + kk;
              const float4 g_lo = lds_f4_ro(scg + 32 * k), g_hi = lds_f4_ro(scg + 32 * k + 16);
              const float4 u_lo = lds_f4_ro(scu + 32 * k), u_hi = lds_f4_ro(scu + 32 * k + 16);
              const float2 sg[4] = {{g_lo.x, g_lo.y}, {g_lo.z, g_lo.w}, {g_hi.x, g_hi.y}, {g_hi.z, g_hi.w}};
              const float2 su[4] = {{u_lo.x, u_lo.y}, {u_lo.z, u_lo.w}, {u_hi.x, u_hi.y}, {u_hi.z, u_hi.w}};
              uint32_t o[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 hv = dequant2<KIND>(g[8 * kk + 2 * i], g[8 * kk + 2 * i + 1], sah2, sg[i]);
                const float2 up = dequant2<KIND>(u[8 * kk + 2 * i], u[8 * kk + 2 * i + 1], sa2, su[i]);
                o[i] = pack_half2_from(fmul2(silu_from_half2(hv), up));
              }
              put(k, make_uint4(o[0], o[1], o[2], o[3]));
            }
          }
          stage_end();
        } else {
          // one 64-wide head: x0 = its columns 0..31, x1 = columns 32..63; piece k of x0 and piece k of x1 rotate
          // together.  Half a head (16 columns of each) is in registers at a time.
          const uint32_t sc = sc_tile + 64 * c * 4;
          const bool rotated = n < p.rot_cols;
          if (rotated && !trig_scaled) {          // sin and cos premultiplied by the token scale, once per row block
            trig_scaled = true;
#pragma unroll
            for (int k = 0; k < 16; ++k) { sn2[k] = fmul2(sn2[k], sa2); cs2[k] = fmul2(cs2[k], sa2); }
          }
          uint32_t x0[16], x1[16];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            GP_BEGIN(gp_tl);
            tmem_ld_32x32b_x16(t_tile + 64 * c + 16 * hh, x0);
            tmem_ld_32x32b_x16(t_tile + 64 * c + 32 + 16 * hh, x1);
            tmem_ld_wait(x0, x1);
            GP_END(e_ld, gp_tl);
            if (hh == 0) stage_begin(); else release();
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const int k = 2 * hh + kk;           // piece of x0 / x1
              const float4 a_lo = lds_f4_ro(sc + 32 * k), a_hi = lds_f4_ro(sc + 32 * k + 16);
              const float4 b_lo = lds_f4_ro(sc + 128 + 32 * k), b_hi = lds_f4_ro(sc + 128 + 32 * k + 16);
              if (rotated) {
                const float2 sb0[4] = {{a_lo.x, a_lo.y}, {a_lo.z, a_lo.w}, {a_hi.x, a_hi.y}, {a_hi.z, a_hi.w}};
                const float2 sb1[4] = {{b_lo.x, b_lo.y}, {b_lo.z, b_lo.w}, {b_hi.x, b_hi.y}, {b_hi.z, b_hi.w}};
                uint32_t o0[4], o1[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  // y = acc * sB[n];  out0 = y0*(sA cos) - y1*(sA sin),  out1 = y0*(sA sin) + y1*(sA cos), each as one
                  // rounded product and one fused multiply-add (the CPU model rounds at the same points)
                  const float2 y0 = fmul2(pk2(acc_to_float<KIND>(x0[8 * kk + 2 * i]), acc_to_float<KIND>(x0[8 * kk + 2 * i + 1])), sb0[i]);
                  const float2 y1 = fmul2(pk2(acc_to_float<KIND>(x1[8 * kk + 2 * i]), acc_to_float<KIND>(x1[8 * kk + 2 * i + 1])), sb1[i]);
                  const float2 c2 = cs2[4 * k + i], s2 = sn2[4 * k + i];
                  const float2 qa = fmul2(y1, s2), ta = fmul2(y1, c2);
                  o0[i] = pack_half2_from(__ffma2_rn(y0, c2, make_float2(-qa.x, -qa.y)));
                  o1[i] = pack_half2_from(__ffma2_rn(y0, s2, ta));
                }
                put(k, make_uint4(o0[0], o0[1], o0[2], o0[3]));
                put(4 + k, make_uint4(o1[0], o1[1], o1[2], o1[3]));
              } else {
                put(k, dequant_piece<KIND>(&x0[8 * kk], sa2, a_lo, a_hi));
                put(4 + k, dequant_piece<KIND>(&x1[8 * kk], sa2, b_lo, b_hi));
              }
            }
          }
          stage_end();
        }
      }
    }
    GP_END(e_total, gp_e0);
    if (lane == 0 && q == 0 && j < 2) { GP_STORE(5 + 4 * j, e_total); GP_STORE(6 + 4 * j, e_acc); GP_STORE(7 + 4 * j, e_read); GP_STORE(8 + 4 * j, e_ld); }
    if (lane == 0) tma_store_wait_all<0>();
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FUSEQ ? EPI_REGS_FUSEQ : EPI_REGS));
    // ------------------------------ epilogue ----------------------------------
    // Eight free-running warps.  Warp e reads TMEM lane quarter e % 4 (32 rows) and the column half e / 4
    // of every tile, in chunks: the TMEM load of chunk i+1 is in flight during the arithmetic of chunk i,
    // and the warp gives the accumulator stage back as soon as its last chunk sits in registers.  Warps
    // never synchronise with one another: each keeps its own copy of the channel scales it needs.
    const int e = warp - FRONT_WARPS;      // 0..7
    const int q = warp & 3;                // TMEM lane quarter this warp may read
    const int half = e >> 2;               // column half of the tile handled by this warp
    constexpr int WACC = BN / 2;                       // accumulator columns per warp and tile (dual: 64 gate + 64 up)
    constexpr int WOUT = OUT_COLS_PER_TILE / 2;        // output columns per warp and tile
    const int wout0 = half * WOUT;                     // first output column of this warp inside the tile
    const int acol0 = DUAL ? half * (BN / 4) : half * WACC;   // its first accumulator column (dual: of the gate part; up = + BN/2)
    uint8_t* out_buf = out_base + e * OUT_BUFS * OUT_BUF_BYTES;   // this warp's staging boxes
    int obuf = 0;
    int sbuf = 0;                          // channel-scale buffer of the current tile (the producer fills them in turn)
    // per-row state, fetched once per row block and kept in registers across its column blocks; the token
    // scale and the channel scales of the NEXT tile are fetched while the current tile is processed
    float sa = 0.f, sa_next = 0.f;
    int fq_rbi = 0;                        // FUSEQ: row blocks this warp has started
    float2 sn2[16], cs2[16];               // sin / cos row of this thread's token as fp32 pairs
    int cur_m_blk = -1;
    int trig_m_blk = -1;                   // row block whose sin / cos rows are in sn2 / cs2
    bool trig_scaled = false;              // ... already multiplied by the token scale
    // A pair of staging boxes holds 32 rows x 64 output columns: lanes 0-15 own the rows of the first box,
    // lanes 16-31 those of the second.  stg_off = byte offsets of the 8 16-byte pieces of this thread's row in
    // its box, in the 128-byte swizzle the TMA store expects (conflict-free for 16-byte stores by a warp).
    uint32_t stg_off[8];
#pragma unroll
    for (int pc = 0; pc < 8; ++pc) stg_off[pc] = (lane & 15) * 128 + ((pc ^ (lane & 7)) << 4);

    GP_DECL(e_total); GP_DECL(e_acc); GP_DECL(e_read); GP_DECL(e_ld); GP_BEGIN(gp_e0);
    Walk tw; tw.start(p);
    if constexpr (EPI != EPI_I32) {
      if (tw.valid(p)) {
        const int r = rowblk(tw.m) * BM + q * 32 + lane;
        if (r < p.M) sa_next = p.scale_a ? __ldg(p.scale_a + r) : 1.f;
      }
    }
    for (int it = 0; tw.valid(p); ++it) {
      const int m_blk = rowblk(tw.m), n_blk = tw.n;
      tw.next(p);                            // tw is now the NEXT tile
      const int nxt_m = rowblk(tw.m);        // its row block (meaningful while tw.valid)
      const int as = it & 1; const uint32_t aph = (it >> 1) & 1;
      const int m0 = m_blk * BM;
      const int n0 = n_blk * OUT_COLS_PER_TILE;
      const int row_base = m0 + q * 32;
      const int row = row_base + lane;
      const bool row_ok = row < p.M;

      // ---- per-tile prologue: everything that comes from global memory, before the accumulator wait ----
      bool new_row_block = false;            // FUSEQ: the token scale is picked up after the accumulator wait
      if constexpr (EPI != EPI_I32) {
        if (m_blk != cur_m_blk) {
          cur_m_blk = m_blk;
          if constexpr (FUSEQ) new_row_block = true; else sa = sa_next;
        }
        if constexpr (EPI == EPI_ROTARY) {
          // The angle rows cost 16 scattered 16-byte loads per thread.  Once this warp's columns lie past the
          // rotated ones (the V part of a QKV projection, walked last), the rows of the NEXT row block are
          // fetched already, a tile or more before they are needed; otherwise at the row block's first tile.
          int want = m_blk;
          if (n0 + wout0 >= p.rot_cols && tw.valid(p)) want = nxt_m;
          if (want != trig_m_blk) {
            trig_m_blk = want;
            trig_scaled = false;
            const long long r = (long long)want * BM + q * 32 + lane;
            const int pos = r < p.M ? (int)((r + p.row_offset) % p.seqlen) : 0;
            const float* s4 = p.sin_tab + (long long)pos * 32;
            const float* c4 = p.cos_tab + (long long)pos * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j) {     // straight into the registers that hold them: nothing waits for the data here
              asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(sn2[2 * j].x), "=f"(sn2[2 * j].y), "=f"(sn2[2 * j + 1].x), "=f"(sn2[2 * j + 1].y) : "l"(s4 + 4 * j));
              asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(cs2[2 * j].x), "=f"(cs2[2 * j].y), "=f"(cs2[2 * j + 1].x), "=f"(cs2[2 * j + 1].y) : "l"(c4 + 4 * j));
            }
          }
          // The rotated columns use sin and cos premultiplied by the token scale: folded in once per row block,
          // at the first tile in which this warp rotates (rows fetched ahead have arrived by then).
          if (!FUSEQ && trig_m_blk == m_blk && !trig_scaled && n0 + wout0 < p.rot_cols) {
            trig_scaled = true;
            const float2 s2 = pk2(sa, sa);
#pragma unroll
            for (int j = 0; j < 16; ++j) { sn2[j] = fmul2(sn2[j], s2); cs2[j] = fmul2(cs2[j], s2); }
          }
        }
        if (!FUSEQ && tw.valid(p) && nxt_m != m_blk) {
          const int r = nxt_m * BM + q * 32 + lane;
          sa_next = (r < p.M) ? (p.scale_a ? ldg_f_here(p.scale_a + r) : 1.f) : 0.f;
        }
      }

      // warp-uniform outcome of the bounded wait: the tcgen05.ld below needs the whole warp
      GP_BEGIN(gp_tw);
      const bool got = mbar_wait(&acc_full[as], aph, abort_flag, ST_TIMEOUT_EPILOGUE, (2u << 16) | as, budget);
      GP_END(e_acc, gp_tw);
      uint32_t agreed = __all_sync(0xffffffffu, got) ? 1u : 0u;
      if (!agreed) break;
      asm volatile("" : "+r"(agreed));   // opaque from here on: the scale address below must stay dependent on the wait
      tc_fence_after();
      if constexpr (FUSEQ && EPI != EPI_I32) {
        // token scales made on chip: written by the quantiser warps before the A block these MMAs read
        if (new_row_block) {
          const bool have = mbar_wait(&sa_ready[fq_rbi & (Map::SA_BUFS - 1)], (uint32_t)(fq_rbi / Map::SA_BUFS) & 1u, abort_flag,
                                      ST_TIMEOUT_EPILOGUE, (2u << 16) | 0x500, budget);
          if (!__all_sync(0xffffffffu, have)) break;
          sa = sa_s[(fq_rbi & (Map::SA_BUFS - 1)) * BM + q * 32 + lane];
          ++fq_rbi;
        }
        if constexpr (EPI == EPI_ROTARY) {
          if (trig_m_blk == m_blk && !trig_scaled && n0 + wout0 < p.rot_cols) {
            trig_scaled = true;
            const float2 s2 = pk2(sa, sa);
#pragma unroll
            for (int j = 0; j < 16; ++j) { sn2[j] = fmul2(sn2[j], s2); cs2[j] = fmul2(cs2[j], s2); }
          }
        }
      }
      if constexpr (PAIR && EPI != EPI_I32) {
        // of a pair, each CTA's scales report to a barrier of its own (buffer sbuf is filled for the (it / SCALE_BUFS)-th time)
        if (copy_scales && !(kDiag && (p.ablate & 4))) {
          const bool have = mbar_wait(&sc_full[sbuf], (uint32_t)(WRES ? 0 : it / Map::SCALE_BUFS) & 1u, abort_flag,
                                      ST_TIMEOUT_EPILOGUE, (2u << 16) | 0x600 | sbuf, budget);
          if (!__all_sync(0xffffffffu, have)) break;
        }
      }
      // The tile's channel scales landed with its first K block, before the MMAs that have now completed.
      // They are read with loads the compiler may move across the staging stores below (plain loads would
      // be kept in order with every store to shared memory); the address depends on the outcome of the
      // wait, so no read can move above it.  Index = column relative to this warp's first accumulator column.
      const uint32_t sc_addr = smem_u32(scale_base + sbuf * BN + acol0) + ((agreed - 1u) << 2);
      if (!WRES && ++sbuf == Map::SCALE_BUFS) sbuf = 0;
      auto scq = [&](int i) { return lds_f4_ro(sc_addr + i * 4); };      // scales of columns i..i+3
      auto scp = [&](int i) { return lds_f2_ro(sc_addr + i * 4); };      // ... i, i+1
      const uint32_t t_row = tmem_base + as * BN + ((uint32_t)(q * 32) << 16) + acol0;
      // hand the accumulator stage back to the MMA warp: called once per tile, right after the wait that
      // brought this warp's last accumulator chunk into registers
      auto release = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[as]), 0));    // the barrier of the CTA that issues the MMAs
          else mbar_arrive(&acc_empty[as]);
        }
      };

      if (row_base < p.M && !(kDiag && ((p.ablate & 2) || ((p.ablate & 8) && half == 1)))) {
        if constexpr (EPI == EPI_I32) {
          // raw accumulators, direct 16-byte stores
          auto emit = [&](const uint32_t (&v)[32], int c) {
            if (row_ok) {
              const int n = n0 + wout0 + c;
              int32_t* dst = reinterpret_cast<int32_t*>(p.C) + (long long)row * p.ldc + n;
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                if (n + j + 4 <= p.N) *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          };
          uint32_t va[32], vb[32];
          tmem_ld_32x32b_x32(t_row, va);
#pragma unroll
          for (int c = 0; c < WACC; c += 64) {
            tmem_ld_wait(va);
            tmem_ld_32x32b_x32(t_row + c + 32, vb);
            emit(va, c);
            tmem_ld_wait(vb);
            if (c + 64 < WACC) tmem_ld_32x32b_x32(t_row + c + 64, va); else release();
            emit(vb, c + 32);
          }
        } else if constexpr (EPI == EPI_ROTARY_GEN) {
          // Any head of 64 or 128 columns with its first 2 * rot_half columns rotated: x0 = columns [0, rot_half) of
          // the head, x1 = [rot_half, 2 rot_half), the rest of the head and every V column only dequantised
          // (cute/ampere_gemm_i8_rotary.py:362-393).  Same arithmetic, rounded at the same points, as EPI_ROTARY; 16
          // columns of x0 and the matching 16 of x1 at a time, sin / cos rows read per use, 32-byte stores straight
          // from registers (a rotated pair can lie 64 columns apart, further than one staging box is wide).
          const float2 sa2 = pk2(sa, sa);
          __half* drow = reinterpret_cast<__half*>(p.C) + (long long)row * p.ldc;
          const bool wide_ok = (reinterpret_cast<uintptr_t>(drow) & 31) == 0;
          auto store16 = [&](int n, const uint32_t (&o)[8]) {          // 16 fp16 at output column n
            if (!row_ok) return;
            __half* dst = drow + n;
            if (wide_ok && (n & 15) == 0) stg_v8(dst, make_uint4(o[0], o[1], o[2], o[3]), make_uint4(o[4], o[5], o[6], o[7]));
            else {
              *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(dst + 8) = make_uint4(o[4], o[5], o[6], o[7]);
            }
          };
          auto plain16 = [&](int lc) {                                   // local column lc of this warp's 128: dequant only
            uint32_t v[16], o[8];
            tmem_ld_32x32b_x16(t_row + lc, v);
            tmem_ld_wait(v);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = pack_half2_from(dequant2<KIND>(v[2 * i], v[2 * i + 1], sa2, scp(lc + 2 * i)));
            store16(n0 + wout0 + lc, o);
          };
          const long long pos = ((long long)row + p.row_offset) % p.seqlen;
          const float* srow = p.sin_tab + pos * p.rot_half;
          const float* crow = p.cos_tab + pos * p.rot_half;
#pragma unroll 1
          for (int hc = 0; hc < WACC; hc += p.head_dim) {             // the heads inside this warp's 128 columns
            const int nh = n0 + wout0 + hc;
            if (nh >= p.N) break;
            int done = 0;                                              // columns of the head finished so far
            if (nh < p.rot_cols) {
#pragma unroll 1
              for (int u = 0; u < p.rot_half; u += 16) {
                uint32_t x0[16], x1[16], o0[8], o1[8];
                tmem_ld_32x32b_x16(t_row + hc + u, x0);
                tmem_ld_32x32b_x16(t_row + hc + p.rot_half + u, x1);
                float4 sv[4], cv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  sv[i] = row_ok ? __ldg(reinterpret_cast<const float4*>(srow + u) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                  cv[i] = row_ok ? __ldg(reinterpret_cast<const float4*>(crow + u) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                tmem_ld_wait(x0, x1);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float4 s4 = sv[i >> 1], c4 = cv[i >> 1];
                  const float2 s2 = fmul2((i & 1) ? make_float2(s4.z, s4.w) : make_float2(s4.x, s4.y), sa2);   // sA sin
                  const float2 c2 = fmul2((i & 1) ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y), sa2);   // sA cos
                  const float2 y0 = fmul2(pk2(acc_to_float<KIND>(x0[2 * i]), acc_to_float<KIND>(x0[2 * i + 1])), scp(hc + u + 2 * i));
                  const float2 y1 = fmul2(pk2(acc_to_float<KIND>(x1[2 * i]), acc_to_float<KIND>(x1[2 * i + 1])), scp(hc + p.rot_half + u + 2 * i));
                  const float2 qa = fmul2(y1, s2), ta = fmul2(y1, c2);
                  o0[i] = pack_half2_from(__ffma2_rn(y0, c2, make_float2(-qa.x, -qa.y)));
                  o1[i] = pack_half2_from(__ffma2_rn(y0, s2, ta));
                }
                store16(nh + u, o0);
                store16(nh + p.rot_half + u, o1);
              }
              done = 2 * p.rot_half;
            }
#pragma unroll 1
            for (int lc = done; lc < p.head_dim; lc += 16) plain16(hc + lc);
          }
          release();
        } else if constexpr (EPI == EPI_SILU_MX) {
          // SwiGLU product quantised per 32 output columns: e = biased exponent of the block maximum,
          // scale byte = clamp(e - 8, 0, 254) (value 2^(byte-127)), elements = e4m3_rn_satfinite(v * 2^(127-byte)).
          // A thread holds whole 32-column blocks of its row, so the block maximum needs no exchange.
          const float2 sa2 = pk2(sa, sa);
          const float2 sah2 = pk2(0.5f * sa, 0.5f * sa);      // the gate is dequantised straight to gate / 2 (exact halving)
          auto emit = [&](const uint32_t (&g)[32], const uint32_t (&u)[32], int c) {
            const int n = n0 + wout0 + c;
            if (n + 32 <= p.N) {
              float o[32];
              float amax = 0.f;
#pragma unroll
              for (int j = 0; j < 32; j += 2) {
                const float2 hv = dequant2<KIND>(g[j], g[j + 1], sah2, scp(c + j));          // gate / 2
                const float2 uv = dequant2<KIND>(u[j], u[j + 1], sa2, scp(BN / 2 + c + j));
                const float2 ov = fmul2(silu_from_half2(hv), uv);
                o[j] = ov.x; o[j + 1] = ov.y;
                amax = fmaxf(amax, fmaxf(fabsf(o[j]), fabsf(o[j + 1])));
              }
              int eb = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 8;
              eb = max(0, min(254, eb));
              const float inv = __uint_as_float((uint32_t)(254 - eb) << 23);
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j] * inv, o[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(o[4 * j + 2] * inv, o[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                w[j] = lo | (hi << 16);
              }
              if (row_ok) {
                uint8_t* dst = reinterpret_cast<uint8_t*>(p.C) + (long long)row * p.ldc + n;
                *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
                p.out_scale[(long long)row * p.ld_scale + (n >> 5)] = (uint8_t)eb;
              }
            }
          };
          uint32_t ga[32], ua[32], gb[32], ub[32];
          tmem_ld_32x32b_x32(t_row, ga);
          tmem_ld_32x32b_x32(t_row + BN / 2, ua);
          tmem_ld_wait(ga, ua);
          tmem_ld_32x32b_x32(t_row + 32, gb);
          tmem_ld_32x32b_x32(t_row + BN / 2 + 32, ub);
          emit(ga, ua, 0);
          tmem_ld_wait(gb, ub);
          release();
          emit(gb, ub, 32);
        } else {
          const float2 sa2 = pk2(sa, sa);
          const float2 sah2 = pk2(0.5f * sa, 0.5f * sa);
          // The product path stages the tile in swizzled shared memory and leaves through TMA stores.  A library
          // built with -DGSB200_DIAG carries the body a second time, storing straight from registers.
          auto run_tile = [&](auto direct_tag) {
            constexpr bool DIRECT = decltype(direct_tag)::value;
            __half* drow0 = reinterpret_cast<__half*>(p.C) + (long long)row * p.ldc;
            // Output leaves in pairs of 32-column boxes (4 pieces of 8 fp16 per row and box): both boxes are
            // staged, then one proxy fence + one warp sync publish them to two TMA stores.  (Plain coalesced
            // global stores from the staged boxes were measured and are slower than the TMA stores.)
            int buf_a = 0, buf_b = 0;
            auto pair_begin = [&]() {
              buf_a = obuf; buf_b = (obuf + 1 == OUT_BUFS) ? 0 : obuf + 1;
              if constexpr (!DIRECT) {
                GP_BEGIN(gp_tr);
                if (lane == 0) tma_store_wait_read<OUT_BUFS - 2>();   // the stores that last used these two buffers have read them
                __syncwarp();
                GP_END(e_read, gp_tr);
              }
            };
            uint4 held[2];                       // direct stores: the even piece of a 32-byte sector waits for the odd one
            auto put = [&](int which, int n, int piece, uint4 o) {
              if constexpr (DIRECT) {
                if ((piece & 1) == 0) { held[which] = o; }
                else if (row_ok) {
                  __half* dst = drow0 + n + (piece - 1) * 8;
                  if (n + piece * 8 + 8 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) stg_v8(dst, held[which], o);
                  else {
                    if (n + piece * 8 <= p.N) *reinterpret_cast<uint4*>(dst) = held[which];
                    if (n + piece * 8 + 8 <= p.N) *reinterpret_cast<uint4*>(dst + 8) = o;
                  }
                }
              } else {
                *reinterpret_cast<uint4*>(out_buf + (lane < 16 ? buf_a : buf_b) * OUT_BUF_BYTES + stg_off[which * 4 + piece]) = o;
              }
            };
            auto pair_end = [&](int n_a, int n_b) {
              if constexpr (!DIRECT) {
                fence_proxy_async_smem();          // generic-proxy smem writes -> visible to the TMA engine
                __syncwarp();
                if (lane == 0 && !(kDiag && (p.ablate & 1))) {
                  tma_store_2d(&tm_c, out_buf + buf_a * OUT_BUF_BYTES, n_a, row_base); tma_store_commit();
                  if (row_base + OUT_BOX_ROWS < p.M) tma_store_2d(&tm_c, out_buf + buf_b * OUT_BUF_BYTES, n_a, row_base + OUT_BOX_ROWS);
                  tma_store_commit();          // always two groups per pair (the second may be empty): pair_begin counts groups
                }
                obuf = (buf_b + 1 == OUT_BUFS) ? 0 : buf_b + 1;
              }
            };

            if constexpr (EPI == EPI_DEQUANT || EPI == EPI_BIAS) {
              // chunks of 32 columns = one box; two chunks leave as a pair
              auto emit = [&](const uint32_t (&v)[32], int c, int which) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  if constexpr (EPI == EPI_BIAS)
                    put(which, n0 + wout0 + c, j >> 3, bias_piece<KIND>(&v[j], sa2, scq(c + j), scq(c + j + 4)));
                  else
                    put(which, n0 + wout0 + c, j >> 3, dequant_piece<KIND>(&v[j], sa2, scq(c + j), scq(c + j + 4)));
                }
              };
              uint32_t va[32], vb[32];
              tmem_ld_32x32b_x32(t_row, va);
#pragma unroll
              for (int c = 0; c < WACC; c += 64) {
                const int n = n0 + wout0 + c;
                const bool live = n < p.N;
                tmem_ld_wait(va);
                tmem_ld_32x32b_x32(t_row + c + 32, vb);
                if (live) { pair_begin(); emit(va, c, 0); }
                tmem_ld_wait(vb);
                if (c + 64 < WACC) tmem_ld_32x32b_x32(t_row + c + 64, va); else release();
                if (live) { emit(vb, c + 32, 1); pair_end(n, n + 32); }
              }
            } else if constexpr (EPI == EPI_ROTARY) {
              // 64-wide heads, x0 = columns 0..31, x1 = columns 32..63 of a head.  A chunk is half a head:
              // 16 columns of x0 and the matching 16 of x1, i.e. two pieces of each of the head's two boxes.
              auto ldh = [&](int c, int hh, uint32_t (&x0)[16], uint32_t (&x1)[16]) {
                tmem_ld_32x32b_x16(t_row + c + hh * 16, x0);
                tmem_ld_32x32b_x16(t_row + c + hh * 16 + 32, x1);
              };
              // c = local column of the head, hh = which half of x0 / x1 (a compile-time constant at each call)
              auto emit = [&](const uint32_t (&v0)[16], const uint32_t (&v1)[16], int c, int hh) {
                const int n = n0 + wout0 + c;
                if (n >= p.N) return;
                if (hh == 0) pair_begin();
                const int s0 = c + hh * 16;      // scale index of this half of x0; x1 is 32 columns on
                const int s1 = s0 + 32;
                if (n < p.rot_cols) {
#pragma unroll
                  for (int j = 0; j < 16; j += 8) {
                    const float4 a_lo = scq(s0 + j);
                    const float4 a_hi = scq(s0 + j + 4);
                    const float4 b_lo = scq(s1 + j);
                    const float4 b_hi = scq(s1 + j + 4);
                    const float2 sb0[4] = {{a_lo.x, a_lo.y}, {a_lo.z, a_lo.w}, {a_hi.x, a_hi.y}, {a_hi.z, a_hi.w}};
                    const float2 sb1[4] = {{b_lo.x, b_lo.y}, {b_lo.z, b_lo.w}, {b_hi.x, b_hi.y}, {b_hi.z, b_hi.w}};
                    uint32_t o0[4], o1[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      // y = acc * sB[n];  out0 = y0*(sA cos) - y1*(sA sin),  out1 = y0*(sA sin) + y1*(sA cos), each
                      // as one rounded product and one fused multiply-add (the CPU model rounds at the same points)
                      const float2 y0 = fmul2(pk2(acc_to_float<KIND>(v0[j + 2 * i]), acc_to_float<KIND>(v0[j + 2 * i + 1])), sb0[i]);
                      const float2 y1 = fmul2(pk2(acc_to_float<KIND>(v1[j + 2 * i]), acc_to_float<KIND>(v1[j + 2 * i + 1])), sb1[i]);
                      const float2 c2 = cs2[hh * 8 + (j >> 1) + i], s2 = sn2[hh * 8 + (j >> 1) + i];
                      const float2 qa = fmul2(y1, s2), ta = fmul2(y1, c2);
                      o0[i] = pack_half2_from(__ffma2_rn(y0, c2, make_float2(-qa.x, -qa.y)));
                      o1[i] = pack_half2_from(__ffma2_rn(y0, s2, ta));
                    }
                    put(0, n, hh * 2 + (j >> 3), make_uint4(o0[0], o0[1], o0[2], o0[3]));
                    put(1, n + 32, hh * 2 + (j >> 3), make_uint4(o1[0], o1[1], o1[2], o1[3]));
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 16; j += 8) {
                    put(0, n, hh * 2 + (j >> 3), dequant_piece<KIND>(&v0[j], sa2, scq(s0 + j), scq(s0 + j + 4)));
                    put(1, n + 32, hh * 2 + (j >> 3), dequant_piece<KIND>(&v1[j], sa2, scq(s1 + j), scq(s1 + j + 4)));
                  }
                }
                if (hh == 1) pair_end(n, n + 32);
              };
              uint32_t xa0[16], xa1[16], xb0[16], xb1[16];
              ldh(0, 0, xa0, xa1);
              // one head per trip and not unrolled: the body is large, and more straight-line code than the
              // instruction cache holds makes the warps stall on instruction fetch
#pragma unroll 1
              for (int c = 0; c < WACC; c += 64) {
                GP_BEGIN(gp_l0);
                tmem_ld_wait(xa0, xa1);
                GP_END(e_ld, gp_l0);
                ldh(c, 1, xb0, xb1);
                emit(xa0, xa1, c, 0);
                GP_BEGIN(gp_l1);
                tmem_ld_wait(xb0, xb1);
                GP_END(e_ld, gp_l1);
                if (c + 64 < WACC) ldh(c + 64, 0, xa0, xa1); else release();
                emit(xb0, xb1, c, 1);
              }
            } else {   // EPI_SILU: gate at local column c, up at BN/2 accumulator columns on; a chunk is one 32-column output box
              auto emit = [&](const uint32_t (&g)[32], const uint32_t (&u)[32], int c, int which) {
                const int n = n0 + wout0 + c;
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const float4 g_lo = scq(c + j);
                  const float4 g_hi = scq(c + j + 4);
                  const float4 u_lo = scq(BN / 2 + c + j);
                  const float4 u_hi = scq(BN / 2 + c + j + 4);
                  const float2 sg[4] = {{g_lo.x, g_lo.y}, {g_lo.z, g_lo.w}, {g_hi.x, g_hi.y}, {g_hi.z, g_hi.w}};
                  const float2 su[4] = {{u_lo.x, u_lo.y}, {u_lo.z, u_lo.w}, {u_hi.x, u_hi.y}, {u_hi.z, u_hi.w}};
                  uint32_t o[4];
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    // silu(gate) = h + h * tanh(h), h = gate / 2: the gate is dequantised straight to h (exact halving)
                    const float2 hv = dequant2<KIND>(g[j + 2 * i], g[j + 2 * i + 1], sah2, sg[i]);
                    const float2 up = dequant2<KIND>(u[j + 2 * i], u[j + 2 * i + 1], sa2, su[i]);
                    o[i] = pack_half2_from(fmul2(silu_from_half2(hv), up));
                  }
                  put(which, n, j >> 3, make_uint4(o[0], o[1], o[2], o[3]));
                }
              };
              uint32_t ga[32], ua[32], gb[32], ub[32];
              const int n = n0 + wout0;
              const bool live = n < p.N;
              tmem_ld_32x32b_x32(t_row, ga);
              tmem_ld_32x32b_x32(t_row + BN / 2, ua);
              tmem_ld_wait(ga, ua);
              tmem_ld_32x32b_x32(t_row + 32, gb);
              tmem_ld_32x32b_x32(t_row + BN / 2 + 32, ub);
              if (live) { pair_begin(); emit(ga, ua, 0, 0); }
              tmem_ld_wait(gb, ub);
              release();
              if (live) { emit(gb, ub, 32, 1); pair_end(n, n + 32); }
            }
          };
          if constexpr (kDiag) {
            if (p.direct_store) run_tile(true_tag{}); else run_tile(false_tag{});
          } else {
            run_tile(false_tag{});
          }
        }
      } else {
        release();
      }
    }
    GP_END(e_total, gp_e0);
    if (lane == 0 && q == 0) { GP_STORE(5 + 4 * half, e_total); GP_STORE(6 + 4 * half, e_acc); GP_STORE(7 + 4 * half, e_read); GP_STORE(8 + 4 * half, e_ld); }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  if constexpr (PAIR) {
    // neither CTA leaves (or frees tensor memory) while the other may still arrive at its barriers or its MMAs write here
    cluster_sync_all();
    if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
  } else {
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  }
}

}  // namespace gsb
