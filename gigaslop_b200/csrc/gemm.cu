// Host side of the tcgen05 GEMM family: argument validation, TMA tensor-map
// encoding and launch of the persistent kernel (one CTA per SM).
#include <cuda.h>

#include <atomic>

#include "capi_internal.h"
#include "diag.h"
#include "gemm_kernel.cuh"

namespace gsb {

// ---- tensor maps ---------------------------------------------------------------------------------
// cuTensorMapEncodeTiled is reached through the runtime's driver-entry-point query (no link-time libcuda
// dependency); the pointer is looked up once per process.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static std::atomic<EncodeTiledFn> fn{nullptr};
  EncodeTiledFn f = fn.load(std::memory_order_acquire);
  if (!f) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      f = reinterpret_cast<EncodeTiledFn>(p);
      fn.store(f, std::memory_order_release);
    }
  }
  return f;
}

// 2-D row-major tensor [rows, cols] of `esz`-byte elements, row stride ld_elems, box of box_cols x box_rows.
// A tensor map is a pure function of these arguments (it holds the address, not the data), so the last maps a
// host thread built are kept in a small per-thread table (set-associative): a caller that launches the same kernels on the same
// buffers step after step -- the per-timestep LSTM wrapper, a pipeline over a ring of buffers -- encodes nothing
// in steady state.  Per thread, so no lock and no sharing between the host threads that drive different GPUs.
struct TmapKey {
  const void* base; uint64_t rows, cols, ld; uint32_t box_cols, box_rows; int dt, esz, swz;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols &&
           box_rows == o.box_rows && dt == o.dt && esz == o.esz && swz == o.swz;
  }
};
constexpr int kTmapSets = 32, kTmapWays = 4;             // 128 maps per host thread, 4-way set-associative
struct TmapSlot { TmapKey key; CUtensorMap map; bool used; };
static std::atomic<unsigned long long> g_tmap_encodes{0};      // encodes since load (test / benchmark hook)

static inline uint64_t mix64(uint64_t x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 27; x *= 0x94D049BB133111EBull; x ^= x >> 31;
  return x;
}

bool tmap_2d(CUtensorMap* m, CUtensorMapDataType dt, int esz, const void* base, uint64_t rows, uint64_t cols,
             uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swz) {
  static thread_local TmapSlot cache[kTmapSets][kTmapWays];
  static thread_local unsigned victim[kTmapSets];
  const TmapKey key{base, rows, cols, ld_elems, box_cols, box_rows, (int)dt, esz, (int)swz};
  uint64_t h = mix64(reinterpret_cast<uintptr_t>(base));
  h = mix64(h ^ (rows * 0x9E3779B97F4A7C15ull) ^ (cols << 21) ^ (ld_elems << 42));
  h = mix64(h ^ ((uint64_t)box_rows << 8) ^ ((uint64_t)box_cols << 24) ^ ((uint64_t)dt << 40) ^ ((uint64_t)swz << 48));
  TmapSlot* set = cache[h % kTmapSets];
  for (int w = 0; w < kTmapWays; ++w)
    if (set[w].used && set[w].key == key) { *m = set[w].map; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * (uint64_t)esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "gigaslop_b200: cuTensorMapEncodeTiled failed (%d)\n", (int)r);
    return false;
  }
  g_tmap_encodes.fetch_add(1, std::memory_order_relaxed);
  int w = 0;
  while (w < kTmapWays && set[w].used) ++w;
  if (w == kTmapWays) w = (int)(victim[h % kTmapSets]++ % kTmapWays);     // round robin inside the set
  set[w].key = key; set[w].map = *m; set[w].used = true;
  return true;
}
unsigned long long tmap_encode_count() { return g_tmap_encodes.load(std::memory_order_relaxed); }

static bool make_map_2d(CUtensorMap* m, CUtensorMapDataType dt, int esz, const void* base, uint64_t rows,
                        uint64_t cols, uint64_t ld_elems, uint32_t box_cols, uint32_t box_rows,
                        CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  return tmap_2d(m, dt, esz, base, rows, cols, ld_elems, box_cols, box_rows, swz);
}

// ---- per-device state -------------------------------------------------------------------------
// Atomics: the contract allows one host thread per GPU, and two of them may meet here.
constexpr int kMaxDevices = 64;
constexpr int kVariantMinRowBlocks = 256;      // 128-row blocks from which the twelve-warp form is the default for the SwiGLU
constexpr int kPairMinRowBlocks = 16;          // ... and from which the streaming schedule runs as CTA pairs (measured down to M = 2048)
static std::atomic<int> g_dev_ok[kMaxDevices];       // 0 unknown, 1 ok, -1 unsupported
static std::atomic<int> g_dev_sms[kMaxDevices];

template <int KIND, int EPI>
static cudaError_t set_attr() {
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, EPI, SCHED_STREAM>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
  if (e != cudaSuccess) return e;
  constexpr int RES = (EPI == EPI_ROTARY || EPI == EPI_ROTARY_GEN || EPI == EPI_BIAS) ? SCHED_ARES : SCHED_WRES;
  return cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND, EPI, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              GEMM_SMEM_BYTES);
}

// ---- kernel variants -------------------------------------------------------------------------------
// The dequant / rotary / SwiGLU epilogues on 8-bit operands exist in four forms: eight or twelve epilogue warps,
// one CTA or a CTA pair per tile.
//   Twelve warps (three per SM sub-partition, working on 64-column items): the eight-warp epilogue is bound by the
//   latency of each warp's own chain, not by a shared resource, so more warps finish a tile sooner.  That form
//   re-splits its registers with setmaxnreg, which WAITS until the CTA's pool has them: it may only be launched when
//   the registers the kernel was compiled with, times its 512 threads, cover the re-split (checked here, once).
//   CTA pairs (tcgen05.mma.cta_group::2): two CTAs of a cluster share every MMA, 256 rows (128 each) x 256
//   accumulator columns, each CTA holding half of the tile's W rows: half the W traffic from L2 and a third less
//   shared-memory traffic per tile.
template <int KIND, int EPI, bool PAIR, int EW>
struct Variant {
  static constexpr int RES = (EPI == EPI_ROTARY || EPI == EPI_ROTARY_GEN || EPI == EPI_BIAS) ? SCHED_ARES : SCHED_WRES;
  static constexpr int THREADS = 32 * (FRONT_WARPS + EW);
  using Fn = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, GemmParams);
  static Fn kernel(bool resident) {
    return resident ? (Fn)gemm_tcgen05_kernel<KIND, EPI, RES, false, PAIR, EW>
                    : (Fn)gemm_tcgen05_kernel<KIND, EPI, SCHED_STREAM, false, PAIR, EW>;
  }
  static cudaLaunchConfig_t config(int grid, cudaStream_t st, cudaLaunchAttribute* attr) {
    attr->id = cudaLaunchAttributeClusterDimension;
    attr->val.clusterDim.x = PAIR ? 2 : 1; attr->val.clusterDim.y = 1; attr->val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
  }
  // Scheduling units (CTAs, or CTA pairs) that can be resident at once on the current device; 0 = this variant must
  // not be launched here.  Looked up once per device.
  static int capacity(bool resident) {
    static std::atomic<int> cap[kMaxDevices][2];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    int c = cap[dev][resident].load(std::memory_order_acquire);
    if (c == 0) {
      Fn k = kernel(resident);
      c = -1;
      cudaFuncAttributes fa{};
      bool ok = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES) == cudaSuccess &&
                cudaFuncGetAttributes(&fa, k) == cudaSuccess;
      if (ok && EW == 12) ok = fa.numRegs * THREADS >= EW12_REG_POOL_NEEDED && fa.numRegs * THREADS <= 65536;
      if (ok) {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (PAIR) {
          cudaLaunchAttribute attr;
          cudaLaunchConfig_t cfg = config(2 * (sms / 2), nullptr, &attr);
          int n = 0;
          if (cudaOccupancyMaxActiveClusters(&n, k, &cfg) == cudaSuccess && n > 0) c = n;
        } else if (sms > 0) {
          c = sms;
        }
      }
      (void)cudaGetLastError();
      cap[dev][resident].store(c, std::memory_order_release);
      if (getenv("GSB200_GEMM_VERBOSE"))
        fprintf(stderr, "gigaslop_b200: gemm variant pair=%d epilogue warps=%d: %d units resident (registers %d)\n", (int)PAIR, EW, c, fa.numRegs);
    }
    return c > 0 ? c : 0;
  }
  static cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb0, const CUtensorMap& tb1, const CUtensorMap& tc,
                            const GemmParams& p, int grid, bool resident, cudaStream_t st) {
    cudaLaunchAttribute attr;
    cudaLaunchConfig_t cfg = config(grid, st, &attr);
    return cudaLaunchKernelEx(&cfg, kernel(resident), ta, tb0, tb1, tc, p);
  }
};

// One of the variants, picked at run time: capacity (launch = false) or launch.
template <int KIND, int EPI>
static int variant_call(bool pair, bool ew12, bool launch, const CUtensorMap& ta, const CUtensorMap& tb0, const CUtensorMap& tb1,
                        const CUtensorMap& tc, const GemmParams& p, int grid, bool resident, cudaStream_t st) {
  if (pair && ew12) return launch ? (int)Variant<KIND, EPI, true, 12>::launch(ta, tb0, tb1, tc, p, grid, resident, st) : Variant<KIND, EPI, true, 12>::capacity(resident);
  if (pair) return launch ? (int)Variant<KIND, EPI, true, 8>::launch(ta, tb0, tb1, tc, p, grid, resident, st) : Variant<KIND, EPI, true, 8>::capacity(resident);
  if (ew12) return launch ? (int)Variant<KIND, EPI, false, 12>::launch(ta, tb0, tb1, tc, p, grid, resident, st) : Variant<KIND, EPI, false, 12>::capacity(resident);
  return launch ? (int)Variant<KIND, EPI, false, 8>::launch(ta, tb0, tb1, tc, p, grid, resident, st) : Variant<KIND, EPI, false, 8>::capacity(resident);
}
static int variant_dispatch(int kind, int epi, bool pair, bool ew12, bool launch, const CUtensorMap& ta, const CUtensorMap& tb0,
                            const CUtensorMap& tb1, const CUtensorMap& tc, const GemmParams& p, int grid, bool resident, cudaStream_t st) {
  const bool i8 = kind == KIND_I8;
  switch (epi) {
    case EPI_DEQUANT:
      return i8 ? variant_call<KIND_I8, EPI_DEQUANT>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st)
                : variant_call<KIND_F8, EPI_DEQUANT>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st);
    case EPI_ROTARY:
      return i8 ? variant_call<KIND_I8, EPI_ROTARY>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st)
                : variant_call<KIND_F8, EPI_ROTARY>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st);
    default:
      return i8 ? variant_call<KIND_I8, EPI_SILU>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st)
                : variant_call<KIND_F8, EPI_SILU>(pair, ew12, launch, ta, tb0, tb1, tc, p, grid, resident, st);
  }
}

// Process-wide override of the variant choice (-1 = by shape); the environment variables GSB200_GEMM_EW (8 / 12) and
// GSB200_GEMM_PAIR (0 / 1) give the initial value, read once.
static std::atomic<int> g_variant_ew{-2}, g_variant_pair{-2};       // -2 = environment not read yet
static int variant_setting(std::atomic<int>& v, const char* env) {
  int s = v.load(std::memory_order_relaxed);
  if (s == -2) {
    const char* e = getenv(env);
    s = (e && *e) ? atoi(e) : -1;
    v.store(s, std::memory_order_relaxed);
  }
  return s;
}
void set_gemm_variant(int epilogue_warps, int cta_pairs) {
  g_variant_ew.store(epilogue_warps, std::memory_order_relaxed);
  g_variant_pair.store(cta_pairs, std::memory_order_relaxed);
}

int32_t ensure_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return GSB200_ERR_DEVICE;
  const int known = g_dev_ok[dev].load(std::memory_order_acquire);
  if (known == 1) return GSB200_OK;
  if (known == -1) return GSB200_ERR_DEVICE;
  int major = 0, sms = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (major != 10) {
    fprintf(stderr, "gigaslop_b200: device %d is sm_%d*, this library only carries sm_100a code\n", dev, major * 10);
    g_dev_ok[dev].store(-1, std::memory_order_release);
    return GSB200_ERR_DEVICE;
  }
  cudaError_t errs[] = {
      set_attr<KIND_I8, EPI_I32>(),     set_attr<KIND_I8, EPI_DEQUANT>(), set_attr<KIND_I8, EPI_ROTARY>(),
      set_attr<KIND_I8, EPI_SILU>(),    set_attr<KIND_F8, EPI_DEQUANT>(), set_attr<KIND_F8, EPI_ROTARY>(),
      set_attr<KIND_F8, EPI_SILU>(),    set_attr<KIND_F8, EPI_SILU_MX>(), set_attr<KIND_F16, EPI_DEQUANT>(),
      set_attr<KIND_F16, EPI_BIAS>(),   set_attr<KIND_I8, EPI_ROTARY_GEN>(), set_attr<KIND_F8, EPI_ROTARY_GEN>()};
  for (cudaError_t er : errs)
    if (er != cudaSuccess) return cuda_status(er, "cudaFuncSetAttribute");
  {
    cudaError_t er = cudaFuncSetAttribute(gemm_tcgen05_kernel<KIND_I8, EPI_ROTARY, SCHED_ARES, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
    if (er != cudaSuccess) return cuda_status(er, "cudaFuncSetAttribute");
  }
  if (!encode_fn()) {
    fprintf(stderr, "gigaslop_b200: cuTensorMapEncodeTiled not available from the driver\n");
    return GSB200_ERR_DEVICE;
  }
  g_dev_sms[dev].store(sms, std::memory_order_relaxed);
  g_dev_ok[dev].store(1, std::memory_order_release);
  return GSB200_OK;
}

// Cap for the grids of the persistent GEMM kernels.  One value for the whole process (every device, every
// host thread); 0 = no cap.
static std::atomic<int> g_sm_limit{0};
void set_sm_limit(int sms) { g_sm_limit.store(sms, std::memory_order_relaxed); }

int sm_count_physical() {
  int dev = 0;
  cudaGetDevice(&dev);
  const int n = (dev >= 0 && dev < kMaxDevices) ? g_dev_sms[dev].load(std::memory_order_relaxed) : 0;
  return n > 0 ? n : 148;
}

int sm_count() {
  const int n = sm_count_physical();
  const int lim = g_sm_limit.load(std::memory_order_relaxed);
  return (lim > 0 && lim < n) ? lim : n;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int KIND, int EPI>
static cudaError_t launch_inst(const CUtensorMap& ta, const CUtensorMap& tb0, const CUtensorMap& tb1,
                               const CUtensorMap& tc, const GemmParams& p, int grid, bool resident, cudaStream_t st) {
  // resident-operand schedule: rotary and the bias epilogue keep A (activation-stationary: one CTA reads a row
  // block's A completely before it writes any of that row block's output, which is what lets the low-rank
  // projection keep its intermediate inside the output buffer), the others keep W (weight-stationary)
  constexpr int RES = (EPI == EPI_ROTARY || EPI == EPI_ROTARY_GEN || EPI == EPI_BIAS) ? SCHED_ARES : SCHED_WRES;
  if (resident) gemm_tcgen05_kernel<KIND, EPI, RES><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
  else gemm_tcgen05_kernel<KIND, EPI, SCHED_STREAM><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
  return cudaGetLastError();
}

int32_t launch_gemm(const GemmArgs& a, cudaStream_t st) {
  if (a.M == 0) return GSB200_OK;
  if (a.M < 0 || a.M > 0x7fffff00ll || a.N <= 0 || a.K <= 0) return GSB200_ERR_BAD_ARG;
  if (a.flags & ~(GSB200_FLAG_SCALAR_SCALE_B | GSB200_FLAG_OWN_ROW_BLOCKS | GSB200_DIAG_FLAG_MASK)) return GSB200_ERR_BAD_ARG;
  const bool force_streaming = (a.flags & GSB200_DIAG_FLAG_MASK & GSB200_DIAG_FLAG_STREAMING) != 0;
  const bool fused = a.x_f16 != nullptr;          // the int8 A operand is made on chip from fp16 activations
  if (fused) {
    if (a.kind != KIND_I8 || a.epi != EPI_ROTARY || a.A || a.scale_a) return GSB200_ERR_BAD_ARG;
    if (!aligned16(a.x_f16) || a.ldx < a.K || a.ldx % 8 != 0) return GSB200_ERR_BAD_ARG;
    if (a.K > RES_MAX_KBLOCKS * BK || a.K % BK != 0 || force_streaming) return GSB200_ERR_UNSUPPORTED;
  } else {
    if (!a.A || !aligned16(a.A) || a.lda < a.K || a.lda % 16 != 0) return GSB200_ERR_BAD_ARG;
  }
  if (!a.B0 || !a.C) return GSB200_ERR_BAD_ARG;
  if (!aligned16(a.B0) || !aligned16(a.C)) return GSB200_ERR_BAD_ARG;
  if (a.K % 16 != 0 || a.ldb < a.K || a.ldb % 16 != 0) return GSB200_ERR_BAD_ARG;
  if (a.ldc < a.N) return GSB200_ERR_BAD_ARG;
  const bool dual = a.epi == EPI_SILU || a.epi == EPI_SILU_MX;
  if (a.epi == EPI_I32) {
    if (a.N % 4 != 0 || a.ldc % 4 != 0) return GSB200_ERR_BAD_ARG;
  } else {
    if (a.N % 8 != 0 || a.ldc % 8 != 0) return GSB200_ERR_BAD_ARG;
    if (a.epi == EPI_BIAS && !a.scale_b0) return GSB200_ERR_BAD_ARG;                       // the bias vector
    if (a.epi != EPI_DEQUANT && a.epi != EPI_BIAS && ((!a.scale_a && !fused) || !a.scale_b0)) return GSB200_ERR_BAD_ARG;   // plain dequant: null = 1.0
    const bool scalar_b = (a.flags & GSB200_FLAG_SCALAR_SCALE_B) != 0;
    if (scalar_b && (a.epi != EPI_DEQUANT || !a.scale_b0)) return GSB200_ERR_BAD_ARG;
    if (a.scale_b0 && !scalar_b && (reinterpret_cast<uintptr_t>(a.scale_b0) & 15)) return GSB200_ERR_BAD_ARG;
  }
  if (dual) {
    if (!a.B1 || !aligned16(a.B1) || !a.scale_b1 || (reinterpret_cast<uintptr_t>(a.scale_b1) & 15))
      return GSB200_ERR_BAD_ARG;
  }
  if (a.epi == EPI_SILU_MX) {
    if (a.kind != KIND_F8 || a.N % 32 != 0 || !a.out_scale || a.ld_scale < a.N / 32 || a.ldc % 16 != 0)
      return GSB200_ERR_BAD_ARG;
  }
  int rot_cols = 0;
  bool general_rotary = false;
  if (a.epi == EPI_ROTARY) {
    if (!a.sin_tab || !a.cos_tab || !aligned16(a.sin_tab) || !aligned16(a.cos_tab)) return GSB200_ERR_BAD_ARG;
    if (a.seqlen < 1 || a.nhead < 1 || a.row_offset < 0) return GSB200_ERR_BAD_ARG;
    if (a.head_dim <= 0 || a.rotary_dim <= 0 || a.rotary_dim > a.head_dim || (a.rotary_dim & 1)) return GSB200_ERR_BAD_ARG;
    // heads of 64 or 128 columns, the first 32 / 64 / 96 / 128 of them rotated (pairs are handled 16 columns at a time)
    if ((a.head_dim != 64 && a.head_dim != 128) || a.rotary_dim % 32 != 0) return GSB200_ERR_UNSUPPORTED;
    rot_cols = 2 * a.nhead * a.head_dim;
    if (rot_cols > a.N || a.N % a.head_dim != 0) return GSB200_ERR_BAD_ARG;
    if (a.head_dim != 64 || a.rotary_dim != 64) {
      if (fused) return GSB200_ERR_UNSUPPORTED;         // the fused quantiser is built for the 64 / 64 epilogue only
      general_rotary = true;
    }
  }
  int32_t rc = ensure_device();
  if (rc != GSB200_OK) return rc;

  const int out_cols_per_tile = dual ? BN / 2 : BN;
  GemmParams p{};
  p.M = (int)a.M; p.N = a.N; p.K = a.K;
  p.m_blocks = (int)((a.M + BM - 1) / BM);
  p.n_blocks = (a.N + out_cols_per_tile - 1) / out_cols_per_tile;
  p.k_blocks = (a.K + BK - 1) / BK;
  p.C = a.C; p.ldc = a.ldc;
  p.out_scale = a.out_scale; p.ld_scale = a.ld_scale;
  p.scale_a = a.scale_a; p.scale_b0 = a.scale_b0; p.scale_b1 = a.scale_b1;
  p.scale_b_scalar = (a.flags & GSB200_FLAG_SCALAR_SCALE_B) ? 1 : 0;
  p.sin_tab = a.sin_tab; p.cos_tab = a.cos_tab;
  p.seqlen = a.seqlen > 0 ? a.seqlen : 1;
  p.rot_cols = rot_cols;
  p.head_dim = a.head_dim; p.rot_half = a.rotary_dim / 2;
  p.row_offset = (int)(a.row_offset % p.seqlen);
  p.direct_store = (a.flags & GSB200_DIAG_FLAG_MASK & GSB200_DIAG_FLAG_DIRECT_STORE) ? 1 : 0;
  p.ablate = ((a.flags & GSB200_DIAG_FLAG_MASK) >> 8) & 15;
  p.x_f16 = a.x_f16; p.ldx = a.ldx; p.scale_a_out = a.scale_a_out;
  const long long tiles = (long long)p.m_blocks * p.n_blocks;
  if (tiles > 0x7fffffffll) return GSB200_ERR_BAD_ARG;

  CUtensorMap ta, tb0, tb1, tc;
  const CUtensorMapDataType u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  bool ok = fused || make_map_2d(&ta, u8, 1, a.A, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)a.lda, BK, BM);
  ok = ok && make_map_2d(&tb0, u8, 1, a.B0, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.ldb, BK, BN / 2);
  ok = ok && make_map_2d(&tb1, u8, 1, dual ? a.B1 : a.B0, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.ldb, BK, BN / 2);
  if (a.epi != EPI_I32 && a.epi != EPI_SILU_MX)
    ok = ok && make_map_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.C, (uint64_t)a.M, (uint64_t)a.N,
                           (uint64_t)a.ldc, OUT_BOX_COLS, OUT_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    tc = ta;
  if (fused) ta = tb0;                            // never used by the fused kernel
  if (!ok) return GSB200_ERR_BAD_ARG;

  // One operand stays resident in shared memory whenever K <= 512 (its 4 K-pieces fit): the W slice for the
  // dequant / SwiGLU epilogues, the A row block for the rotary epilogue (whose per-row sin/cos state is then
  // fetched once per row block).  Larger K streams both operands.
  const bool resident = p.k_blocks <= RES_MAX_KBLOCKS && !force_streaming;
  int grid;
  p.m_major = 0;
  p.n_groups = 0;
  const bool a_stationary = a.epi == EPI_ROTARY || a.epi == EPI_BIAS;
  int sms = sm_count();
  if (a.sm_cap > 0 && a.sm_cap < sms) sms = a.sm_cap;
  if (a.epi == EPI_BIAS && !resident) return GSB200_ERR_UNSUPPORTED;     // only built for K <= 512 bytes of A per row
  // CTA pairs: 8-bit operands, the dequant / rotary / SwiGLU epilogues, at least two K blocks (the deeper rings' scale
  // buffers need that), and enough row blocks that pairs of SMs stay busy.  From here on a "row block" of the
  // schedule is the pair's 256 rows and `sms` counts pairs.
  bool pair = false, ew12 = false;
  const bool variants = !fused && !general_rotary && !p.direct_store && (a.kind == KIND_I8 || a.kind == KIND_F8) &&
                        (a.epi == EPI_DEQUANT || a.epi == EPI_ROTARY || a.epi == EPI_SILU);
  if (variants) {
    // Defaults, from measurements at the benchmark's sizes: twelve warps pay for the weight-stationary SwiGLU (the
    // heaviest epilogue per output), pairs for the streaming schedule with any of the three epilogues (K > 512: both
    // operands come from L2 for every tile, a single CTA asks for 96 bytes per clock where about 64 arrive, and a
    // pair halves the W part: 12-22 % at M = 65536); the activation-stationary rotary kernel takes both together (twelve
    // warps alone leave it waiting for operands, pairs alone for its epilogue; together 3 % at config 2 and less
    // power); everywhere else the eight-warp single-CTA kernel is as fast or faster.
    const int ew = variant_setting(g_variant_ew, "GSB200_GEMM_EW"), pm = variant_setting(g_variant_pair, "GSB200_GEMM_PAIR");
    const bool big = p.m_blocks >= kVariantMinRowBlocks;
    // twelve warps AND pairs, or neither (so not when the caller has fixed one of the two)
    const bool rotary_both = a.epi == EPI_ROTARY && resident && big && p.k_blocks >= 2 && sms >= 2 && ew < 0 && pm < 0;
    // ... and so does the weight-stationary dequant GEMM when its output is far larger than L2 (the hoisted LSTM
    // projection: 3 % at M = 262144, 5 % at a million rows, nothing at 131072)
    const bool huge_dequant_both = a.epi == EPI_DEQUANT && resident && p.m_blocks >= 2048 && p.n_blocks >= 4 &&
                                   p.k_blocks >= 2 && sms >= 2 && ew < 0 && pm < 0;
    const bool both = rotary_both || huge_dequant_both;
    ew12 = ew < 0 ? ((a.epi == EPI_SILU && resident && big) || both) : ew == 12;
    const bool want_pair = p.k_blocks >= 2 && sms >= 2 &&
                           (pm < 0 ? ((!resident && p.m_blocks >= kPairMinRowBlocks) || (both && ew12)) : pm == 1);
    if (ew12 && !variant_dispatch(a.kind, a.epi, false, true, false, ta, tb0, tb1, tc, p, 0, resident, st)) ew12 = false;
    if (want_pair) {
      int cap = variant_dispatch(a.kind, a.epi, true, ew12, false, ta, tb0, tb1, tc, p, 0, resident, st);
      if (cap > 0) {
        pair = true;
        sms = sms / 2 < cap ? sms / 2 : cap;
        p.m_blocks = (p.m_blocks + 1) / 2;
      }
    }
  }
  const long long sched_tiles = (long long)p.m_blocks * p.n_blocks;
  if (resident && !a_stationary) {
    int groups = sms / p.n_blocks;
    if (groups < 1) groups = 1;
    if (groups > p.m_blocks) groups = p.m_blocks;
    p.n_groups = groups;
    grid = groups * p.n_blocks;
  } else if (a_stationary) {
    p.m_major = 1;
    grid = p.m_blocks < sms ? p.m_blocks : sms;
    // the row blocks of the last, incomplete round are shared by as many CTAs as there are to go round
    const int rem = p.m_blocks % grid;
    p.ares_split = 1;
    // (not for the bias epilogue: the low-rank projection reads its A from inside the output rows it writes, which
    // only works while one CTA owns a row block)
    if (resident && !fused && a.epi == EPI_ROTARY && rem > 0 && !(a.flags & GSB200_FLAG_OWN_ROW_BLOCKS)) {
      int S = grid / rem;
      if (S > p.n_blocks) S = p.n_blocks;
      if (S > 1) p.ares_split = S;
    }
  } else {
    grid = (int)(sched_tiles < sms ? sched_tiles : sms);
  }
  cudaError_t e = cudaErrorInvalidValue;
  if (pair || ew12) {
    if (pair) grid *= 2;
    // the twelve-warp form stores a warp's 32 rows x 64 columns as ONE box
    if (ew12 && !make_map_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.C, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldc,
                             OUT_BOX_COLS, 2 * OUT_BOX_ROWS, CU_TENSOR_MAP_SWIZZLE_128B))
      return GSB200_ERR_BAD_ARG;
    e = (cudaError_t)variant_dispatch(a.kind, a.epi, pair, ew12, true, ta, tb0, tb1, tc, p, grid, resident, st);
    return cuda_status(e, "gemm launch");
  }
  if (a.kind == KIND_I8) {
    switch (a.epi) {
      case EPI_I32: e = launch_inst<KIND_I8, EPI_I32>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      case EPI_DEQUANT: e = launch_inst<KIND_I8, EPI_DEQUANT>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      case EPI_ROTARY:
        if (fused) {
          gemm_tcgen05_kernel<KIND_I8, EPI_ROTARY, SCHED_ARES, true><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb0, tb1, tc, p);
          e = cudaGetLastError();
        } else if (general_rotary) {
          e = launch_inst<KIND_I8, EPI_ROTARY_GEN>(ta, tb0, tb1, tc, p, grid, resident, st);
        } else {
          e = launch_inst<KIND_I8, EPI_ROTARY>(ta, tb0, tb1, tc, p, grid, resident, st);
        }
        break;
      case EPI_SILU: e = launch_inst<KIND_I8, EPI_SILU>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      default: return GSB200_ERR_BAD_ARG;
    }
  } else if (a.kind == KIND_F8) {
    switch (a.epi) {
      case EPI_DEQUANT: e = launch_inst<KIND_F8, EPI_DEQUANT>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      case EPI_ROTARY:
        e = general_rotary ? launch_inst<KIND_F8, EPI_ROTARY_GEN>(ta, tb0, tb1, tc, p, grid, resident, st)
                           : launch_inst<KIND_F8, EPI_ROTARY>(ta, tb0, tb1, tc, p, grid, resident, st);
        break;
      case EPI_SILU: e = launch_inst<KIND_F8, EPI_SILU>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      case EPI_SILU_MX: e = launch_inst<KIND_F8, EPI_SILU_MX>(ta, tb0, tb1, tc, p, grid, resident, st); break;
      default: return GSB200_ERR_BAD_ARG;
    }
  } else if (a.kind == KIND_F16) {
    if (a.epi == EPI_DEQUANT) e = launch_inst<KIND_F16, EPI_DEQUANT>(ta, tb0, tb1, tc, p, grid, resident, st);
    else if (a.epi == EPI_BIAS) e = launch_inst<KIND_F16, EPI_BIAS>(ta, tb0, tb1, tc, p, grid, resident, st);
    else return GSB200_ERR_BAD_ARG;
  } else {
    return GSB200_ERR_BAD_ARG;
  }
  return cuda_status(e, "gemm launch");
}

// ---- self-test of the bounded wait ------------------------------------------------------------
// One warp waits on an mbarrier that nothing ever arrives at.  With a small spin budget the
// wait gives up, records ST_TIMEOUT_EPILOGUE in the status word and the kernel returns
// normally: the give-up path is exercised without hanging or faulting the device.
__global__ void selftest_wait_timeout_kernel() {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  const AbortFlag abort_flag{smem_u32(&abort_word)};
  if (threadIdx.x == 0) { mbar_init(&bar, 1); abort_flag.set(0); fence_mbar_init(); }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, abort_flag, ST_TIMEOUT_EPILOGUE, 0xdead, spin_budget());
  __syncthreads();
}

int32_t selftest_wait_timeout(cudaStream_t st) {
  selftest_wait_timeout_kernel<<<1, 32, 0, st>>>();
  return cuda_status(cudaGetLastError(), "selftest launch");
}

// ---- status word --------------------------------------------------------------------------------
int32_t read_clear_status(uint32_t out[4]) {
  unsigned int h[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(h, g_status, sizeof(h));
  if (e != cudaSuccess) return cuda_status(e, "status read");
  for (int i = 0; i < 4; ++i) out[i] = h[i];
  if (h[0] != 0 || h[1] != 0) {
    unsigned int z[2] = {0, 0};
    e = cudaMemcpyToSymbol(g_status, z, sizeof(z));
    if (e != cudaSuccess) return cuda_status(e, "status clear");
  }
  return GSB200_OK;
}

int32_t set_spin_budget(uint32_t clocks) {
  cudaError_t e = cudaMemcpyToSymbol(g_status, &clocks, sizeof(clocks), 2 * sizeof(unsigned int));
  return cuda_status(e, "set spin budget");
}

}  // namespace gsb
