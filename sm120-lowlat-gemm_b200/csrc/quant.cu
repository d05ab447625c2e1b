// Activation quantizers for the W8A8 / W4A4 GEMMs, one CTA per row, the row read from global memory exactly once.
//
//   fp8 static     q = sat_e4m3(x * (1/scale))                      scale: one float on the device
//   fp8 per token  s[m] = max(amax(x[m]) / 448, min_scale);  q = sat_e4m3(x * (1/s[m]))
//   int8 per token s[m] = max(amax(x[m]) / 127, min_scale);  q = clamp(rint(x * (1/s[m])), +-127)
//   nvfp4          per 16 K: sf = e4m3(amax / 6 * g);  q = e2m1(x * (g / sf)), sf = 0 -> q = 0
//
// Arithmetic follows the reference kernels operation by operation (csrc/quant.cu:43-65 fp8, 67-82 int8, 85-114
// nvfp4): IEEE fp32 division for the scale and its reciprocal, one fp32 multiply per element, round-to-nearest-even
// saturating conversions. What differs is the data movement: 16-byte vector loads, the row kept in registers between
// the amax pass and the conversion pass, 8-byte stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "llg_internal.h"
#include "ptx_sm100.cuh"

namespace llg {
namespace {

constexpr int kThreadsSmall = 256;   // rows up to 16384 elements stay in registers with 256 threads
constexpr int kThreadsLarge = 1024;  // longer rows (up to 32768): same single pass, four units per thread (64 registers each)
constexpr int kUnitsLarge = 4;
constexpr int kUnitsCap = 8;  // 8-element units a thread may keep in registers: rows up to 8 * 8 * 256 = 16384

template <typename T>
__device__ __forceinline__ float as_f32(T v);
template <>
__device__ __forceinline__ float as_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float as_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float as_f32<float>(float v) { return v; }

// 8 consecutive elements starting at a 16-byte (32-byte for fp32) aligned address.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = as_f32(e[i]);
  }
}

template <int kThreads>
__device__ __forceinline__ float cta_max(float v) {
  __shared__ float part[kThreads / 32];
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) r = fmaxf(r, part[i]);
  __syncthreads();
  return r;
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)byte));
  return __half2float(__ushort_as_half((uint16_t)(h2 & 0xffffu)));
}

__device__ __forceinline__ uint32_t to_s8(float v, float inv) {
  const float r = fminf(fmaxf(rintf(__fmul_rn(v, inv)), -127.f), 127.f);
  return (uint32_t)(int)r & 0xffu;
}

struct QuantDev {
  const void* x;
  const void* up;   // gated input: the row is silu(x) * up, rounded to the input type, before it is quantised
  void* act;        // optional copy of that row in the input type (mode NONE writes only this)
  void* q;
  void* sf;
  const float* scale_in;
  float* scale_out;
  int64_t ldx, ldup, ldact, ldq, ldsf;
  float min_scale;
  int K;
};

constexpr int kModeNone = 4;  // gated activation only, no quantisation

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }

// silu(g) * u in fp32, rounded once to the activation type: the value a separate activation kernel would have stored
template <typename T>
__device__ __forceinline__ float gated(float g, float u) {
  return round_to<T>(__fdiv_rn(g, 1.f + expf(-g)) * u);
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    T e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) e[i] = __float2half_rn(f[i]);
      else e[i] = __float2bfloat16_rn(f[i]);
    }
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(e);
  }
}

// MODE: LLG_QUANT_*. VEC: rows are 16-byte aligned with K % 8 == 0 and the q rows 8-byte aligned, and the row fits the
// register budget -> single pass with vector access. Otherwise a scalar two-pass walk that accepts anything.
template <typename T, int MODE, bool VEC, bool GATED, int kThreads>
__global__ void __launch_bounds__(kThreads) quant_rows_kernel(const QuantDev p) {
  const int m = blockIdx.x;
  // let the kernel behind this one (normally the GEMM that consumes q) start streaming its weight right away, then
  // wait for the producer of x
  pdl_trigger();
  pdl_wait();
  const T* x = static_cast<const T*>(p.x) + (int64_t)m * p.ldx;
  const T* up = GATED ? static_cast<const T*>(p.up) + (int64_t)m * p.ldup : nullptr;
  T* act = (GATED && p.act) ? static_cast<T*>(p.act) + (int64_t)m * p.ldact : nullptr;
  // one unit of 8 input values (vector path) / one value (scalar path), gated when asked
  auto fetch8 = [&](int e0, float (&f)[8]) {
    load8(x + e0, f);
    if constexpr (GATED) {
      float u[8];
      load8(up + e0, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = gated<T>(f[i], u[i]);
      if (act) store8(act + e0, f);
    }
  };
  auto fetch1 = [&](int e) -> float {
    float v = as_f32(x[e]);
    if constexpr (GATED) {
      v = gated<T>(v, as_f32(up[e]));
      if (act) {
        if constexpr (sizeof(T) == 4) act[e] = v;
        else if constexpr (std::is_same<T, __half>::value) act[e] = __float2half_rn(v);
        else act[e] = __float2bfloat16_rn(v);
      }
    }
    return v;
  };
  if constexpr (MODE == kModeNone) {
    if constexpr (VEC) {
      for (int u8 = threadIdx.x; u8 < (p.K >> 3); u8 += kThreads) {
        float f[8];
        fetch8(u8 * 8, f);
      }
    } else {
      for (int k = threadIdx.x; k < p.K; k += kThreads) fetch1(k);
    }
    return;
  }
  uint8_t* q = static_cast<uint8_t*>(p.q) + (int64_t)m * p.ldq;
  const int tid = threadIdx.x;

  if constexpr (MODE == LLG_QUANT_NVFP4) {
    uint8_t* sf = static_cast<uint8_t*>(p.sf) + (int64_t)m * p.ldsf;
    const float g = *p.scale_in;
    const int nblk = p.K >> 4;
    for (int b = tid; b < nblk; b += kThreads) {
      float v[16];
      if constexpr (VEC) {
        float lo[8], hi[8];
        fetch8(b * 16, lo);
        fetch8(b * 16 + 8, hi);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[e] = lo[e]; v[8 + e] = hi[e]; }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = fetch1(b * 16 + e);
      }
      float a = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) a = fmaxf(a, fabsf(v[e]));
      const uint32_t s8 = cvt_e4m3x2(__fmul_rn(__fdiv_rn(a, 6.f), g), 0.f) & 0xffu;
      const float sfv = e4m3_to_f32(s8);
      const float inv = sfv > 0.f ? __fdiv_rn(g, sfv) : 0.f;
      uint32_t w0 = 0, w1 = 0;
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        w0 |= cvt_e2m1x2(__fmul_rn(v[e], inv), __fmul_rn(v[e + 1], inv)) << (4 * e);
        w1 |= cvt_e2m1x2(__fmul_rn(v[8 + e], inv), __fmul_rn(v[9 + e], inv)) << (4 * e);
      }
      *reinterpret_cast<uint2*>(q + b * 8) = make_uint2(w0, w1);  // q rows are 8-byte aligned by contract
      sf[b] = (uint8_t)s8;
    }
    return;
  } else {
    constexpr bool kInt8 = MODE == LLG_QUANT_INT8_PER_TOKEN;
    constexpr bool kPerToken = MODE != LLG_QUANT_FP8_STATIC;
    constexpr float kTop = kInt8 ? 127.f : 448.f;
    if constexpr (VEC) {
      const int units = p.K >> 3;
      constexpr int kUnits = kThreads == kThreadsLarge ? kUnitsLarge : kUnitsCap;
      float r[kUnits][8];
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < kUnits; ++j) {
        const int u = tid + j * kThreads;
        if (u < units) {
          fetch8(u * 8, r[j]);
          if constexpr (kPerToken) {
#pragma unroll
            for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(r[j][e]));
          }
        }
      }
      float scale;
      if constexpr (kPerToken) {
        a = cta_max<kThreads>(a);
        scale = fmaxf(__fdiv_rn(a, kTop), p.min_scale);
        if (tid == 0) p.scale_out[m] = scale;
      } else {
        scale = *p.scale_in;
      }
      const float inv = __fdiv_rn(1.f, scale);
#pragma unroll
      for (int j = 0; j < kUnits; ++j) {
        const int u = tid + j * kThreads;
        if (u < units) {
          uint32_t w0, w1;
          if constexpr (kInt8) {
            w0 = to_s8(r[j][0], inv) | (to_s8(r[j][1], inv) << 8) | (to_s8(r[j][2], inv) << 16) | (to_s8(r[j][3], inv) << 24);
            w1 = to_s8(r[j][4], inv) | (to_s8(r[j][5], inv) << 8) | (to_s8(r[j][6], inv) << 16) | (to_s8(r[j][7], inv) << 24);
          } else {
            w0 = cvt_e4m3x2(__fmul_rn(r[j][0], inv), __fmul_rn(r[j][1], inv)) |
                 (cvt_e4m3x2(__fmul_rn(r[j][2], inv), __fmul_rn(r[j][3], inv)) << 16);
            w1 = cvt_e4m3x2(__fmul_rn(r[j][4], inv), __fmul_rn(r[j][5], inv)) |
                 (cvt_e4m3x2(__fmul_rn(r[j][6], inv), __fmul_rn(r[j][7], inv)) << 16);
          }
          *reinterpret_cast<uint2*>(q + u * 8) = make_uint2(w0, w1);
        }
      }
    } else {
      float scale;
      if constexpr (kPerToken) {
        float a = 0.f;
        for (int k = tid; k < p.K; k += kThreads) a = fmaxf(a, fabsf(fetch1(k)));
        a = cta_max<kThreads>(a);
        scale = fmaxf(__fdiv_rn(a, kTop), p.min_scale);
        if (tid == 0) p.scale_out[m] = scale;
      } else {
        scale = *p.scale_in;
      }
      const float inv = __fdiv_rn(1.f, scale);
      for (int k = tid; k < p.K; k += kThreads) {
        const float xv = fetch1(k);
        if constexpr (kInt8) q[k] = (uint8_t)to_s8(xv, inv);
        else q[k] = (uint8_t)(cvt_e4m3x2(__fmul_rn(xv, inv), 0.f) & 0xffu);
      }
    }
  }
}

inline bool mult(int64_t v, int64_t n) { return v % n == 0; }
inline bool ptr_aligned(const void* p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

template <typename T, int MODE>
cudaError_t launch_mode(const llg_quant_args& a, const GatedExtra& g, cudaStream_t s) {
  QuantDev p{};
  p.x = a.x; p.q = a.q; p.sf = a.sf_out; p.scale_in = a.scale_in; p.scale_out = a.scale_out;
  p.ldx = a.ldx; p.ldq = a.ldq; p.ldsf = a.ldsf; p.min_scale = a.min_scale; p.K = a.K;
  p.up = g.up; p.ldup = g.ldup; p.act = g.act; p.ldact = g.ldact;
  const int64_t in_align = sizeof(T) == 4 ? 32 : 16;
  const int64_t esz = sizeof(T);
  bool vec = ptr_aligned(a.x, in_align) && mult(a.ldx * esz, in_align) && mult(a.K, 8);
  if (MODE != kModeNone) vec = vec && ptr_aligned(a.q, 8) && mult(a.ldq, 8);
  if (g.up) vec = vec && ptr_aligned(g.up, in_align) && mult(g.ldup * esz, in_align);
  if (g.act) vec = vec && ptr_aligned(g.act, in_align) && mult(g.ldact * esz, in_align);
  const bool large = a.K > kUnitsCap * 8 * kThreadsSmall;
  if (MODE != LLG_QUANT_NVFP4 && MODE != kModeNone) vec = vec && a.K <= kUnitsLarge * 8 * kThreadsLarge;
  const dim3 grid(a.M), one(1, 1, 1);
  const bool pdl = pdl_on();
#define LLG_QLAUNCH(V, G, TH) launch_ex(quant_rows_kernel<T, MODE, V, G, TH>, grid, dim3(TH), 0, s, pdl, one, p)
  if (g.up) {
    if (vec) return large ? LLG_QLAUNCH(true, true, kThreadsLarge) : LLG_QLAUNCH(true, true, kThreadsSmall);
    return LLG_QLAUNCH(false, true, kThreadsSmall);
  }
  if constexpr (MODE == kModeNone) {
    return cudaErrorInvalidValue;
  } else {
    if (vec) return large ? LLG_QLAUNCH(true, false, kThreadsLarge) : LLG_QLAUNCH(true, false, kThreadsSmall);
    return LLG_QLAUNCH(false, false, kThreadsSmall);
  }
#undef LLG_QLAUNCH
}

template <typename T>
cudaError_t launch_type(const llg_quant_args& a, const GatedExtra& g, cudaStream_t s) {
  switch (a.mode) {
    case LLG_QUANT_FP8_STATIC: return launch_mode<T, LLG_QUANT_FP8_STATIC>(a, g, s);
    case LLG_QUANT_FP8_PER_TOKEN: return launch_mode<T, LLG_QUANT_FP8_PER_TOKEN>(a, g, s);
    case LLG_QUANT_INT8_PER_TOKEN: return launch_mode<T, LLG_QUANT_INT8_PER_TOKEN>(a, g, s);
    case LLG_QUANT_NVFP4: return launch_mode<T, LLG_QUANT_NVFP4>(a, g, s);
    case kModeNone: return launch_mode<T, kModeNone>(a, g, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t quant_launch(const llg_quant_args& a, const GatedExtra& g, cudaStream_t s) {
  switch (a.in_dtype) {
    case LLG_DT_BF16: return launch_type<__nv_bfloat16>(a, g, s);
    case LLG_DT_F16: return launch_type<__half>(a, g, s);
    case LLG_DT_F32: return launch_type<float>(a, g, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace llg
