// Per-token (per-row) absmax quantisers: fp16/fp32 [M,K] -> int8 or E4M3 [M,K]
// plus one fp32 dequantisation scale per row.  HBM-bound: each row is read once
// with 16/32-byte vector loads, held in registers across the warp-shuffle max
// reduction, and written once with 8-byte stores.  One warp owns one row.
//
// The arithmetic order is part of the contract (results are bit-exact against the
// CPU reference): INT8 uses qs = (1/amax)*127, q = rne(x*qs), scale = 1/qs; FP8 has the kernel formulation (x * (448/amax)) and the torch formulation
// (x / (amax/448)).
#include <cuda_fp8.h>

#include "capi_internal.h"

namespace gsb {

constexpr int QUANT_WARPS = 8;

template <typename Tin>
__device__ __forceinline__ void load8(const Tin* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldg(reinterpret_cast<const float4*>(p + 4));
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  return m;
}

// Two int32 -> two saturated int8 in the low half of the result, the low half of `upper` above them:
// result = upper[15:0] << 16 | sat8(hi) << 8 | sat8(lo).
__device__ __forceinline__ uint32_t pack_sat_s8(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}
// q = clamp(rne(x * qs), -127, 127) for four values, packed little-endian.  |x| <= amax and qs = fl(fl(1/amax)*127)
// bound |x*qs| by 127.0001, so the rounded value never leaves [-127, 127]; the pack saturates all the same.
__device__ __forceinline__ uint32_t pack4_i8(float x0, float x1, float x2, float x3, float qs) {
  const float2 q2 = make_float2(qs, qs);
  const float2 a = __fmul2_rn(make_float2(x0, x1), q2), b = __fmul2_rn(make_float2(x2, x3), q2);
  const uint32_t hi = pack_sat_s8(__float2int_rn(b.y), __float2int_rn(b.x), 0u);     // round half to even
  return pack_sat_s8(__float2int_rn(a.y), __float2int_rn(a.x), hi);
}

__device__ __forceinline__ uint2 pack_i8(const float (&v)[8], float qs) {
  uint2 o;
  o.x = pack4_i8(v[0], v[1], v[2], v[3], qs);
  o.y = pack4_i8(v[4], v[5], v[6], v[7], qs);
  return o;
}

// FP8: mode 0 multiplies by inv = 448/amax; mode 1 divides by scale = amax/448 and clamps.
template <int MODE>
__device__ __forceinline__ float fp8_prescale(float x, float f) {
  if constexpr (MODE == 0) return __fmul_rn(x, f);
  else return fminf(fmaxf(__fdiv_rn(x, f), -448.f), 448.f);
}
template <int MODE>
__device__ __forceinline__ uint2 pack_e4m3(const float (&v)[8], float f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 pr = make_float2(fp8_prescale<MODE>(v[2 * i], f), fp8_prescale<MODE>(v[2 * i + 1], f));
    w[i] = __nv_cvt_float2_to_fp8x2(pr, __NV_SATFINITE, __NV_E4M3);    // rn, saturate to +-448
  }
  uint2 o;
  o.x = w[0] | (w[1] << 16);
  o.y = w[2] | (w[3] << 16);
  return o;
}

// FMT: 0 = int8, 1 = e4m3 kernel formulation, 2 = e4m3 torch formulation.
// NV > 0: the row (<= NV*256 elements) is cached in registers.  NV == 0: any K, second pass re-reads.
template <typename Tin, int FMT, int NV>
__global__ void __launch_bounds__(QUANT_WARPS * 32)
ptq_kernel(const Tin* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
           float* __restrict__ scale, long long M, int K) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (row >= M) return;
  const Tin* xr = x + row * ldx;
  uint8_t* qr = q + row * ldq;
  const int nvec = K >> 3;

  float vals[NV > 0 ? NV : 1][8];
  float amax = 0.f;
  constexpr bool HALF_CACHED = NV > 0 && sizeof(Tin) == 2;
  uint4 raw[HALF_CACHED ? NV : 1];       // fp16 rows are held as loaded: 8 halves per 16-byte vector
  if constexpr (HALF_CACHED) {
    // row maximum with packed half2 max / abs (exact: it is a maximum of the very same fp16 values)
    __half2 m2 = __float2half2_rn(0.f);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      raw[i] = make_uint4(0u, 0u, 0u, 0u);
      if (v < nvec) raw[i] = __ldg(reinterpret_cast<const uint4*>(xr + v * 8));
      const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) m2 = __hmax2(m2, __habs2(h[k]));
    }
    amax = fmaxf(__low2float(m2), __high2float(m2));
  } else if constexpr (NV > 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        load8<Tin>(xr + v * 8, vals[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[i][j]));
      }
    }
  } else {
    for (int v = lane; v < nvec; v += 32) {
      load8<Tin>(xr + v * 8, vals[0]);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[0][j]));
    }
  }
  amax = warp_max(amax);

  float f;   // factor applied to the elements
  float s;   // dequantisation scale written out
  if constexpr (FMT == 0) {
    amax = fmaxf(amax, 1e-8f);
    // the reference computes `127 / amax` with a Python scalar numerator, which PyTorch evaluates as
    // reciprocal(amax) * 127 (two roundings) -- reproduced here so every int8 value matches
    f = __fmul_rn(__frcp_rn(amax), 127.0f);
    s = __frcp_rn(f);
  } else {
    amax = fmaxf(amax, 1e-12f);
    s = __fdiv_rn(amax, 448.0f);
    f = (FMT == 1) ? __fdiv_rn(448.0f, amax) : s;
  }
  if (lane == 0) scale[row] = s;

  auto emit = [&](int v, const float (&vv)[8]) {
    uint2 o;
    if constexpr (FMT == 0) o = pack_i8(vv, f);
    else if constexpr (FMT == 1) o = pack_e4m3<0>(vv, f);
    else o = pack_e4m3<1>(vv, f);
    *reinterpret_cast<uint2*>(qr + v * 8) = o;
  };
  if constexpr (HALF_CACHED) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f2 = __half22float2(h[k]);
          vals[0][2 * k] = f2.x; vals[0][2 * k + 1] = f2.y;
        }
        emit(v, vals[0]);
      }
    }
  } else if constexpr (NV > 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) emit(v, vals[i]);
    }
  } else {
    for (int v = lane; v < nvec; v += 32) {
      load8<Tin>(xr + v * 8, vals[0]);
      emit(v, vals[0]);
    }
  }
}

template <typename Tin, int FMT>
static cudaError_t launch_fmt(const void* x, long long ldx, void* q, long long ldq, float* scale, long long M, int K,
                              cudaStream_t st) {
  const unsigned blocks = (unsigned)((M + QUANT_WARPS - 1) / QUANT_WARPS);
  const Tin* xp = static_cast<const Tin*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  if (K <= 512) ptq_kernel<Tin, FMT, 2><<<blocks, QUANT_WARPS * 32, 0, st>>>(xp, ldx, qp, ldq, scale, M, K);
  else if (K <= 1024) ptq_kernel<Tin, FMT, 4><<<blocks, QUANT_WARPS * 32, 0, st>>>(xp, ldx, qp, ldq, scale, M, K);
  else if (K <= 2048) ptq_kernel<Tin, FMT, 8><<<blocks, QUANT_WARPS * 32, 0, st>>>(xp, ldx, qp, ldq, scale, M, K);
  else ptq_kernel<Tin, FMT, 0><<<blocks, QUANT_WARPS * 32, 0, st>>>(xp, ldx, qp, ldq, scale, M, K);
  return cudaGetLastError();
}

// ---- MXFP8 activation quantiser: E4M3 elements + one E8M0 scale per 32 consecutive elements of a row -------
// scale byte = clamp(biased_exponent(block max) - 8, 0, 254), elements = e4m3_rn_satfinite(x * 2^(127-byte)).
// A lane owns 8 consecutive elements, so a 32-element block lives in 4 neighbouring lanes (two xor-shuffles).
template <typename Tin>
__global__ void __launch_bounds__(QUANT_WARPS * 32)
ptq_mx_kernel(const Tin* __restrict__ x, long long ldx, uint8_t* __restrict__ q, long long ldq,
              uint8_t* __restrict__ scales, long long lds, long long M, int K) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (row >= M) return;
  const Tin* xr = x + row * ldx;
  const int nvec = K >> 3;                         // K % 32 == 0 -> nvec % 4 == 0: the 4 lanes of a block agree on `v < nvec`
  for (int v0 = 0; v0 < nvec; v0 += 32) {
    const int v = v0 + lane;
    float vals[8];
    float amax = 0.f;
    if (v < nvec) {
      load8<Tin>(xr + v * 8, vals);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(vals[j]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (v < nvec) {
      int eb = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 8;
      eb = max(0, min(254, eb));
      const float inv = __uint_as_float((uint32_t)(254 - eb) << 23);
      *reinterpret_cast<uint2*>(q + row * ldq + v * 8) = pack_e4m3<0>(vals, inv);
      if ((lane & 3) == 0) scales[row * lds + (v >> 2)] = (uint8_t)eb;
    }
  }
}

int32_t launch_ptq_mx(const void* x, int x_dtype, long long ldx, uint8_t* q, long long ldq, uint8_t* scales,
                      long long lds, long long M, int K, cudaStream_t st) {
  if (M == 0) return GSB200_OK;
  if (!x || !q || !scales || M < 0 || K <= 0 || K % 32 != 0) return GSB200_ERR_BAD_ARG;
  if (ldx < K || ldq < K || ldq % 8 != 0 || lds < K / 32) return GSB200_ERR_BAD_ARG;
  if (x_dtype != GSB200_F16 && x_dtype != GSB200_F32) return GSB200_ERR_BAD_ARG;
  const int esz = x_dtype == GSB200_F16 ? 2 : 4;
  if ((ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
    return GSB200_ERR_BAD_ARG;
  if ((M + QUANT_WARPS - 1) / QUANT_WARPS > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  const unsigned blocks = (unsigned)((M + QUANT_WARPS - 1) / QUANT_WARPS);
  if (x_dtype == GSB200_F16)
    ptq_mx_kernel<__half><<<blocks, QUANT_WARPS * 32, 0, st>>>(static_cast<const __half*>(x), ldx, q, ldq, scales, lds, M, K);
  else
    ptq_mx_kernel<float><<<blocks, QUANT_WARPS * 32, 0, st>>>(static_cast<const float*>(x), ldx, q, ldq, scales, lds, M, K);
  return cuda_status(cudaGetLastError(), "ptq_mx launch");
}

int32_t launch_ptq(const void* x, int x_dtype, long long ldx, void* q, long long ldq, float* scale, long long M, int K,
                   int fmt, cudaStream_t st) {
  if (M == 0) return GSB200_OK;
  if (!x || !q || !scale || M < 0 || K <= 0) return GSB200_ERR_BAD_ARG;
  if (K % 8 != 0 || ldx < K || ldq < K || ldq % 8 != 0) return GSB200_ERR_BAD_ARG;
  const int esz = x_dtype == GSB200_F16 ? 2 : 4;
  if (x_dtype != GSB200_F16 && x_dtype != GSB200_F32) return GSB200_ERR_BAD_ARG;
  if ((ldx * esz) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
    return GSB200_ERR_BAD_ARG;
  if ((M + QUANT_WARPS - 1) / QUANT_WARPS > 0x7fffffffll) return GSB200_ERR_BAD_ARG;
  cudaError_t e;
  if (x_dtype == GSB200_F16) {
    if (fmt == 0) e = launch_fmt<__half, 0>(x, ldx, q, ldq, scale, M, K, st);
    else if (fmt == 1) e = launch_fmt<__half, 1>(x, ldx, q, ldq, scale, M, K, st);
    else if (fmt == 2) e = launch_fmt<__half, 2>(x, ldx, q, ldq, scale, M, K, st);
    else return GSB200_ERR_BAD_ARG;
  } else {
    if (fmt == 0) e = launch_fmt<float, 0>(x, ldx, q, ldq, scale, M, K, st);
    else if (fmt == 1) e = launch_fmt<float, 1>(x, ldx, q, ldq, scale, M, K, st);
    else if (fmt == 2) e = launch_fmt<float, 2>(x, ldx, q, ldq, scale, M, K, st);
    else return GSB200_ERR_BAD_ARG;
  }
  return cuda_status(e, "ptq launch");
}

}  // namespace gsb
