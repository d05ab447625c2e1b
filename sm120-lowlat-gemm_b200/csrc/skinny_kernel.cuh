// Skinny streaming GEMV on CUDA cores: y[M,N] = x[M,K] @ w[N,K]^T, bf16 or f16, M <= 16, fp32 accumulation.
//
// Summation-order contract (the same one the reference documents in csrc/gemv.cuh:6-12, so results are bit-identical
// to it and do not depend on M or on the tile knobs):
//   * a weight row is shared by LPR lanes; lane `sl` accumulates the 16-byte vectors vbeg+sl, vbeg+sl+LPR, ... in
//     increasing order, the 8 elements of a vector in order, with one fused multiply-add each (the product of two
//     16-bit floats is exact in fp32, so this equals multiply-then-add);
//   * the LPR lane sums are combined by an xor butterfly with offsets LPR/2, ..., 1;
//   * split-K partials are added in split order 0, 1, ..., ksplit-1 starting from partial 0.
// K is split at vector granularity: split s covers vectors [kv*s/ksplit, kv*(s+1)/ksplit), kv = K/8.
//
// Data movement: every lane keeps U x R 16-byte streaming loads (no L1 allocation, 256-byte L2 sectors) in flight;
// activations are re-read through L1. With PDL the first weight loads are issued before the dependency wait.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "llg_internal.h"
#include "ptx_sm100.cuh"

namespace llg {

template <bool F16>
__device__ __forceinline__ void widen16x8(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (F16) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    } else {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

template <bool F16>
__device__ __forceinline__ void skinny_store(const SkinnyDev& p, int m, int n, float v) {
  const int64_t at = (int64_t)m * p.ldy + n;
  if (p.out_fp32) static_cast<float*>(p.y)[at] = v;
  else if constexpr (F16) static_cast<__half*>(p.y)[at] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p.y)[at] = __float2bfloat16_rn(v);
}

// In-order sum of `n` partials spaced `stride` floats apart, at most 8 loads in flight.
__device__ __forceinline__ float ordered_sum_l2(const float* src, int n, int64_t stride) {
  float s = 0.f;
  for (int base = 0; base < n; base += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (base + j < n) v[j] = __ldcg(src + (int64_t)(base + j) * stride);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (base + j < n) s = (base + j == 0) ? v[j] : s + v[j];
  }
  return s;
}

// MT token capacity (M <= MT), R weight rows per lane group, U vectors in flight per row and lane, LPR lanes per row.
template <int MT, int R, int U, int LPR, bool F16>
__global__ void __launch_bounds__(256) skinny_kernel(const SkinnyDev p) {
  constexpr int kGroups = 32 / LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / LPR, sl = lane % LPR;
  const int rows_cta = (blockDim.x >> 5) * kGroups * R;
  const int cta_row0 = blockIdx.x * rows_cta;
  const int row0 = cta_row0 + (warp * kGroups + grp) * R;
  const int split = blockIdx.y;
  const int kv = p.K >> 3;
  const int vbeg = (int)((int64_t)kv * split / p.ksplit), vend = (int)((int64_t)kv * (split + 1) / p.ksplit);

  const uint16_t* const xbase = static_cast<const uint16_t*>(p.x);
  const uint16_t* wrow[R];
  bool live[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    live[r] = row0 + r < p.N;
    wrow[r] = static_cast<const uint16_t*>(p.w) + (int64_t)(live[r] ? row0 + r : 0) * p.ldw;
  }

  float acc[R][MT];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  if (p.pdl_early) pdl_trigger();
  bool synced = false;
  for (int v0 = vbeg + sl; v0 < vend; v0 += LPR * U) {
    uint4 raw[U][R];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int v = v0 + u * LPR;
        raw[u][r] = (v < vend && live[r]) ? ld_stream16(wrow[r] + (int64_t)v * 8) : make_uint4(0, 0, 0, 0);
      }
    if (!synced) {  // weights never depend on the previous kernel; activations may
      pdl_wait();
      synced = true;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * LPR;
      if (v < vend) {
        float wf[R][8];
#pragma unroll
        for (int r = 0; r < R; ++r) widen16x8<F16>(raw[u][r], wf[r]);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < p.M) {
            float xf[8];
            widen16x8<F16>(__ldg(reinterpret_cast<const uint4*>(xbase + (int64_t)m * p.ldx + (int64_t)v * 8)), xf);
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[r][m] = __fmaf_rn(wf[r][e], xf[e], acc[r][m]);
          }
        }
      }
    }
  }
  pdl_wait();
  if (!p.pdl_early) pdl_trigger();
  l2_prefetch_share(p.pf, p.pf_bytes, blockIdx.x + (int64_t)gridDim.x * blockIdx.y, (int64_t)gridDim.x * gridDim.y,
                    threadIdx.x, blockDim.x);

#pragma unroll
  for (int off = LPR / 2; off >= 1; off >>= 1)
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], off);

  // every lane of the group now holds every sum; lane (r*MT+m) % LPR writes entry (r, m)
  if (p.ksplit == 1) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (sl == (r * MT + m) % LPR && m < p.M && live[r]) skinny_store<F16>(p, m, row0 + r, acc[r][m]);
    return;
  }

  if (p.cluster) {
    // The ksplit CTAs of a column form a cluster; each parks [rows_cta][M] partials in its own shared memory and
    // CTA k of the cluster finishes slice k of the column, reading the ranks in split order.
    extern __shared__ float parked[];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (sl == (r * MT + m) % LPR && m < p.M) parked[(row0 + r - cta_row0) * p.M + m] = acc[r][m];
    cluster_arrive();
    cluster_wait();
    const int nrows = min(rows_cta, p.N - cta_row0);
    const int total = nrows * p.M, share = (total + p.ksplit - 1) / p.ksplit;
    const int lo = (int)cluster_ctarank() * share, hi = min(total, lo + share);
    const uint32_t base = smem_u32(parked);
    for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) {
      uint32_t bits[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.ksplit) bits[k] = ld_cluster_u32(cluster_map_shared(base + (uint32_t)i * 4u, (uint32_t)k));
      float s = __uint_as_float(bits[0]);
#pragma unroll
      for (int k = 1; k < 8; ++k)
        if (k < p.ksplit) s += __uint_as_float(bits[k]);
      skinny_store<F16>(p, i % p.M, cta_row0 + i / p.M, s);
    }
    cluster_arrive();  // partials stay alive until every CTA of the cluster has read them
    cluster_wait();
    return;
  }

  // workspace split-K: publish, count arrivals per column, the last CTA of the column reduces in split order
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (sl == (r * MT + m) % LPR && m < p.M && live[r])
        p.ws[((int64_t)split * p.M + m) * p.N + row0 + r] = acc[r][m];
  __shared__ unsigned last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&p.counters[blockIdx.x], 1u) == (unsigned)(p.ksplit - 1);
  __syncthreads();
  if (!last) return;
  __threadfence();
  const int nrows = min(rows_cta, p.N - cta_row0);
  const int64_t plane = (int64_t)p.M * p.N;
  for (int i = threadIdx.x; i < nrows * p.M; i += blockDim.x) {
    const int m = i / nrows, n = cta_row0 + i % nrows;
    skinny_store<F16>(p, m, n, ordered_sum_l2(p.ws + (int64_t)m * p.N + n, p.ksplit, plane));
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0u;
}

inline int skinny_bucket(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }

template <int MT, int R, int U, int LPR>
cudaError_t skinny_launch_one(const SkinnyDev& p, int warps, bool f16, bool pdl, cudaStream_t s) {
  const int rows_cta = warps * (32 / LPR) * R;
  const dim3 grid((p.N + rows_cta - 1) / rows_cta, p.ksplit);
  SkinnyDev q = p;
  q.pdl_early = (int64_t)grid.x * grid.y <= sm_count();
  const size_t smem = q.cluster ? (size_t)rows_cta * p.M * sizeof(float) : 0;
  const dim3 cluster(1, q.cluster ? (unsigned)p.ksplit : 1u, 1);  // the ksplit CTAs of one column
  if (f16) return launch_ex(skinny_kernel<MT, R, U, LPR, true>, grid, dim3(warps * 32), smem, s, pdl, cluster, q);
  return launch_ex(skinny_kernel<MT, R, U, LPR, false>, grid, dim3(warps * 32), smem, s, pdl, cluster, q);
}

template <int MT, int LPR>
cudaError_t skinny_launch_tile(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  switch (rows * 16 + unroll) {
    case 0x12: return skinny_launch_one<MT, 1, 2, LPR>(p, warps, f16, pdl, s);
    case 0x14: return skinny_launch_one<MT, 1, 4, LPR>(p, warps, f16, pdl, s);
    case 0x18: return skinny_launch_one<MT, 1, 8, LPR>(p, warps, f16, pdl, s);
    case 0x22: return skinny_launch_one<MT, 2, 2, LPR>(p, warps, f16, pdl, s);
    case 0x24: return skinny_launch_one<MT, 2, 4, LPR>(p, warps, f16, pdl, s);
    case 0x42: return skinny_launch_one<MT, 4, 2, LPR>(p, warps, f16, pdl, s);
    default: return cudaErrorInvalidValue;
  }
}

template <int LPR>
cudaError_t skinny_launch_lpr(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  switch (skinny_bucket(p.M)) {
    case 1: return skinny_launch_tile<1, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 2: return skinny_launch_tile<2, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 4: return skinny_launch_tile<4, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 8: return skinny_launch_tile<8, LPR>(p, rows, unroll, warps, f16, pdl, s);
    default: return skinny_launch_tile<16, LPR>(p, rows, unroll, warps, f16, pdl, s);
  }
}

}  // namespace llg
