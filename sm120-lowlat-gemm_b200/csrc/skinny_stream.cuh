// Skinny streaming GEMV for sm_100a on the CUDA cores: y[M,N] = x[M,K] @ w[N,K]^T, bf16 or f16, M <= 16, fp32 sums.
//
// What is fixed (the order contract of the reference, csrc/gemv.cuh:6-12, so that results are bit-identical to it, to
// the CPU oracle, and across every M and tile knob):
//   * the K range of a split is cut into 16-byte vectors; "virtual lane" sl of a row's LPR lanes owns vectors
//     vbeg+sl, vbeg+sl+LPR, ... and adds them in that order, the 8 elements of a vector in order, one fused
//     multiply-add each into one fp32 sum per (row, token, virtual lane);
//   * the LPR sums of a row are combined by an xor butterfly with offsets LPR/2, ..., 1;
//   * split-K partials are added in split order 0, 1, ..., ksplit-1. Split s covers vectors
//     [kv*s/ksplit, kv*(s+1)/ksplit), kv = K/8.
//
// Everything else is this kernel's own design for B200:
//   * Persistent, one wave: blockIdx.x owns a contiguous range of about N / gridDim.x rows, so every SM streams the
//     same number of weight bytes; blockIdx.y is the K split.
//   * Weights never pass through registers on their way in: a producer warp brings one K chunk of every row of the
//     range into a ring of shared-memory stages with ONE tiled TMA load per stage (a box of rows x chunk bytes, no
//     swizzle, no multicast), completion counted on an mbarrier. Per-row bulk copies were measured first: about 50 ns
//     per request and SM, which capped the kernel at 3 TB/s. The producer starts before the programmatic-dependent-
//     launch wait - weights do not depend on the previous kernel - so the ring is full when the activations become
//     readable.
//   * Activations come through the same ring, not once per lane and token from global memory: a second TMA box per
//     stage (tokens x chunk bytes), issued after the dependency wait. Two converter warps widen it to fp32 inside
//     shared memory, once per stage and CTA, in the order the compute warps read it, so a compute thread spends one
//     16-byte shared load per two packed multiply-adds of each row it carries and no conversion instruction on x.
//     (Widening x in registers instead was measured: the conversions are repeated by every thread and by the rows a
//     warp holds side by side, and from 4 tokens on they, not memory, set the time.)
//   * A thread owns TWO virtual lanes of a row, p and p + LPR/2 - the partners of the butterfly's first level - and
//     advances both sums with one packed fma.rn.f32x2 (each half is an IEEE fused multiply-add, so the bits are
//     those of two scalar fmaf). The LPR/2 threads of a row are lanes of one warp: the first butterfly level is an
//     add inside the thread, the others are shuffles; no shared memory and no barrier between warps is needed to finish
//     a row. A warp works on 64/LPR rows side by side and on up to R such row groups, which share the widened
//     activations.
//   * Lanes of a row read contiguous weights and contiguous activations: conflict-free.
//   * Vectors past the end of the split are neutralised exactly: their activations are replaced by +0 and their
//     weights by -0, and fma(-0, +0, s) returns s for every s.
//   * Every wait is bounded; on expiry the role records a status code, raises the CTA's abort word and all roles
//     drain.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "llg_internal.h"
#include "ptx_sm100.cuh"

namespace llg {

constexpr int kSkConverterWarps = 2;
constexpr int kSkHelperWarps = 1 + kSkConverterWarps;  // the producer and the converters
constexpr int kSkHeaderBytes = 512;
constexpr int kSkMaxStages = 12;

struct SkinnyHeader {
  uint64_t landed[kSkMaxStages]; // the stage's two TMA boxes (weights, activations) have arrived
  uint64_t full[kSkMaxStages];   // ... and the activations are widened
  uint64_t empty[kSkMaxStages];  // every compute warp is done with the stage
  uint32_t abort;
  uint32_t last;
};
static_assert(sizeof(SkinnyHeader) <= kSkHeaderBytes, "header too large");

// Registers decide how many compute warps a CTA may have: a thread carries R * MT packed sums. Registers are handed
// out per four warps, so 16 warps in all leave 128 per thread and 12 leave 168.
template <int MT, int R>
struct SkinnyGeo {
  static constexpr int kMaxComputeWarps = (R * MT >= 16 ? 12 : 16) - kSkHelperWarps;
  static constexpr int kMaxThreads = (kMaxComputeWarps + kSkHelperWarps) * 32;
};

template <bool F16>
__device__ __forceinline__ float sk_lo(uint32_t w) {
  if constexpr (F16) return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
  else return __uint_as_float(w << 16);
}
template <bool F16>
__device__ __forceinline__ float sk_hi(uint32_t w) {
  if constexpr (F16) return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
  else return __uint_as_float(w & 0xffff0000u);
}

template <bool F16>
__device__ __forceinline__ void sk_emit(const SkinnyDev& p, int m, int n, float v) {
  const int64_t at = (int64_t)m * p.ldy + n;
  if (p.out_fp32) static_cast<float*>(p.y)[at] = v;
  else if constexpr (F16) static_cast<__half*>(p.y)[at] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p.y)[at] = __float2bfloat16_rn(v);
}

// One round (LPR vectors of K) of one thread: its two vectors of up to R rows against the widened activations.
// Element order inside a sum: the 8 elements of the vector, in order (q = element pair, then low, then high).
// xs points at the round's first 16-byte entry for this thread: entry ((m * 4 + q) * HP) further on holds
// {a[2q], b[2q], a[2q+1], b[2q+1]} of token m, a / b = the thread's first / second vector.
//
// Fast body: exactly L live row groups, exactly MT tokens, every vector inside the split - no predicate anywhere, so
// nothing is issued that does not count. wsrc points at the thread's first vector of the round in its first row group;
// group_stride steps to the next group; the second vector lies `second` bytes on.
template <int MT, int R, int L, int HP, bool F16>
__device__ __forceinline__ void sk_round_fast(const uint8_t* wsrc, int group_stride, int second, const float4* xs,
                                              float2 (&acc)[R][MT]) {
  uint4 ra[L], rb[L];
#pragma unroll
  for (int u = 0; u < L; ++u) {
    ra[u] = *reinterpret_cast<const uint4*>(wsrc + (size_t)u * group_stride);
    rb[u] = *reinterpret_cast<const uint4*>(wsrc + (size_t)u * group_stride + second);
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 w0[L], w1[L];
#pragma unroll
    for (int u = 0; u < L; ++u) {
      const uint32_t aw = q == 0 ? ra[u].x : q == 1 ? ra[u].y : q == 2 ? ra[u].z : ra[u].w;
      const uint32_t bw = q == 0 ? rb[u].x : q == 1 ? rb[u].y : q == 2 ? rb[u].z : rb[u].w;
      w0[u] = make_float2(sk_lo<F16>(aw), sk_lo<F16>(bw));
      w1[u] = make_float2(sk_hi<F16>(aw), sk_hi<F16>(bw));
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float4 xv = xs[(m * 4 + q) * HP];
#pragma unroll
      for (int u = 0; u < L; ++u) acc[u][m] = __ffma2_rn(w0[u], make_float2(xv.x, xv.y), acc[u][m]);
#pragma unroll
      for (int u = 0; u < L; ++u) acc[u][m] = __ffma2_rn(w1[u], make_float2(xv.z, xv.w), acc[u][m]);
    }
  }
}

// Guarded body for everything else: fewer than MT tokens, or the last, partial round of a split, whose vectors past
// the split's end are neutralised (weights -0 here, activations +0 by the converters: fma(-0, +0, s) = s for every s).
template <int MT, int R, int HP, bool F16>
__device__ __forceinline__ void sk_round_guarded(const uint8_t* wsrc, int group_stride, int second, const float4* xs,
                                                 int nlive, int M, bool a_off, bool b_off, float2 (&acc)[R][MT]) {
  uint4 ra[R], rb[R];
#pragma unroll
  for (int u = 0; u < R; ++u) {
    ra[u] = rb[u] = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);
    if (u < nlive) {
      if (!a_off) ra[u] = *reinterpret_cast<const uint4*>(wsrc + (size_t)u * group_stride);
      if (!b_off) rb[u] = *reinterpret_cast<const uint4*>(wsrc + (size_t)u * group_stride + second);
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 w0[R], w1[R];
#pragma unroll
    for (int u = 0; u < R; ++u) {
      const uint32_t aw = q == 0 ? ra[u].x : q == 1 ? ra[u].y : q == 2 ? ra[u].z : ra[u].w;
      const uint32_t bw = q == 0 ? rb[u].x : q == 1 ? rb[u].y : q == 2 ? rb[u].z : rb[u].w;
      w0[u] = make_float2(sk_lo<F16>(aw), sk_lo<F16>(bw));
      w1[u] = make_float2(sk_hi<F16>(aw), sk_hi<F16>(bw));
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < M) {
        const float4 xv = xs[(m * 4 + q) * HP];
#pragma unroll
        for (int u = 0; u < R; ++u) {
          if (u < nlive) {
            acc[u][m] = __ffma2_rn(w0[u], make_float2(xv.x, xv.y), acc[u][m]);
            acc[u][m] = __ffma2_rn(w1[u], make_float2(xv.z, xv.w), acc[u][m]);
          }
        }
      }
    }
  }
}

// MT: token capacity (M <= MT). R: row groups a warp carries at once. LPR: virtual lanes per row (order contract).
template <int MT, int R, int LPR, bool F16>
__global__ void __launch_bounds__(SkinnyGeo<MT, R>::kMaxThreads, 1)
skinny_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const SkinnyDev p) {
  constexpr int HP = LPR / 2;   // threads per row; each owns virtual lanes pp and pp + HP
  constexpr int RS = 32 / HP;   // rows a warp works on side by side
  extern __shared__ __align__(128) uint8_t sk_smem[];
  SkinnyHeader* const hdr = reinterpret_cast<SkinnyHeader*>(sk_smem);
  uint8_t* const stage0 = sk_smem + kSkHeaderBytes;
  volatile uint32_t* const abort_word = &hdr->abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NC = (int)(blockDim.x >> 5) - kSkHelperWarps;
  const int S = p.stages, J = p.rounds, M = p.M;
  const int split = blockIdx.y;
  const int rb = (int)((int64_t)p.N * blockIdx.x / gridDim.x), re = (int)((int64_t)p.N * (blockIdx.x + 1) / gridDim.x);
  const int nrows = re - rb;
  const int kv = p.K >> 3;
  const int vbeg = (int)((int64_t)kv * split / p.ksplit), vend = (int)((int64_t)kv * (split + 1) / p.ksplit);
  const int nrounds = (vend - vbeg + LPR - 1) / LPR;
  const int nst = (nrounds + J - 1) / J;                       // stages per pass over K
  const int npass = (nrows + p.rows_pass - 1) / p.rows_pass;   // passes over K (one, unless the range is long)
  const int total = npass * nst;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&hdr->landed[s]), 1);
      mbar_init(smem_u32(&hdr->full[s]), kSkConverterWarps);
      mbar_init(smem_u32(&hdr->empty[s]), (uint32_t)NC);
    }
    hdr->abort = 0u;
    hdr->last = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  __syncthreads();
  pdl_trigger();  // one wave by construction: the next kernel's CTAs may take the SMs as they free up

  if (warp == 0) {
    // ================================ producer: weights and activations ================================
    // The warp walks the loop together; one elected lane issues. A box is always transferred whole (rows or K past
    // the tensor read as zero, rows past this CTA's range are the neighbour's and are never used), so the byte count
    // a stage waits for is constant.
    const bool leader = elect_one();
    const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
    const uint32_t tx = (uint32_t)(p.w_box_bytes + p.x_box_bytes);
    auto load_w = [&](int g) {
      const int pass = g / nst, st = g - pass * nst, s = g % S;
      const uint32_t bar = smem_u32(&hdr->landed[s]);
      mbar_expect_tx(bar, tx);  // the activations follow (load_x)
      tma_load_2d(smem_u32(stage0 + (size_t)s * p.stage_bytes), &tmW, bar, (vbeg + st * J * LPR) * 4, rb + pass * p.rows_pass, pol_w);
    };
    auto load_x = [&](int g) {
      const int st = g % nst, s = g % S;
      tma_load_2d(smem_u32(stage0 + (size_t)s * p.stage_bytes + p.xraw_off), &tmX, smem_u32(&hdr->landed[s]),
                  (vbeg + st * J * LPR) * 4, 0, pol_x);
    };
    // fill the ring with weights, which never depend on the previous kernel; its output x follows after the wait
    const int npre = total < S ? total : S;
    if (leader)
      for (int g = 0; g < npre; ++g) load_w(g);
    pdl_wait();
    if (leader)
      for (int g = 0; g < npre; ++g) load_x(g);
    bool ok = true;
    for (int g = npre; g < total; ++g) {
      ok = mbar_wait(smem_u32(&hdr->empty[g % S]), ((g / S) & 1) ^ 1, abort_word);
      if (!ok) break;
      if (leader) {
        load_w(g);
        load_x(g);
      }
    }
    if (!ok) {
      if (lane == 0) atomicCAS(p.status, 0u, (unsigned)ST_SKINNY_PRODUCER_WAIT);
      // copies already issued must land before the CTA's shared memory goes away: they take microseconds
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000ll) {}
    }
    __syncwarp();
    l2_prefetch_share(p.pf, p.pf_bytes, blockIdx.x + (int64_t)gridDim.x * blockIdx.y, (int64_t)gridDim.x * gridDim.y, lane, 32);
  } else if (warp < kSkHelperWarps) {
    // ================================ activation converters ================================
    // Widened layout of a stage's x: for round j, token m, element pair q and thread pp of a row, 16 bytes
    // {a[2q], b[2q], a[2q+1], b[2q+1]} in fp32, a = vector of virtual lane pp, b = that of lane pp + HP; vectors past
    // the split's end become +0.
    const int ct = (warp - 1) * 32 + lane;
    constexpr int kCt = kSkConverterWarps * 32;
    bool ok = true;
    for (int g = 0; g < total; ++g) {
      const int s = g % S, st = g % nst;
      ok = mbar_wait(smem_u32(&hdr->landed[s]), (g / S) & 1, abort_word);
      if (!ok) break;
      const int v0 = vbeg + st * J * LPR;
      const int jn = min(J, nrounds - st * J);
      const uint8_t* const raw = stage0 + (size_t)s * p.stage_bytes + p.xraw_off;
      float4* const xs = reinterpret_cast<float4*>(stage0 + (size_t)s * p.stage_bytes + p.xslot_off);
      const int items = jn * M * HP;
      for (int it = ct; it < items; it += kCt) {
        const int pp = it % HP, jm = it / HP, m = jm % M, j = jm / M;
        const int la = j * LPR + pp, lb = la + HP;  // vectors counted from the stage's start
        uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
        if (v0 + la < vend) a = *reinterpret_cast<const uint4*>(raw + (size_t)m * p.xraw_pitch + (size_t)la * 16);
        if (v0 + lb < vend) b = *reinterpret_cast<const uint4*>(raw + (size_t)m * p.xraw_pitch + (size_t)lb * 16);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
          xs[(jm * 4 + q) * HP + pp] = make_float4(sk_lo<F16>(aw[q]), sk_lo<F16>(bw[q]), sk_hi<F16>(aw[q]), sk_hi<F16>(bw[q]));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&hdr->full[s]));
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0u, (unsigned)ST_SKINNY_CONVERT_WAIT);
  } else {
    // ================================ compute warps ================================
    const int cw = warp - kSkHelperWarps;
    const int rl = lane / HP, pp = lane % HP;
    float* const parked = reinterpret_cast<float*>(stage0 + (size_t)S * p.stage_bytes);  // cluster split-K only
    pdl_wait();  // outputs and split-K buffers may still be in use by the previous kernel
    bool ok = true;
    for (int pass = 0; pass < npass && ok; ++pass) {
      const int r0 = pass * p.rows_pass, nr = min(p.rows_pass, nrows - r0);
      // row group u of this warp holds rows (u * NC + cw) * RS + [0, RS) of the pass; groups past the end are skipped
      int nlive = 0;
#pragma unroll
      for (int u = 0; u < R; ++u) nlive += ((u * NC + cw) * RS < nr) ? 1 : 0;
      float2 acc[R][MT];
#pragma unroll
      for (int u = 0; u < R; ++u)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[u][m] = make_float2(0.f, 0.f);

      for (int st = 0; st < nst; ++st) {
        const int g = pass * nst + st, s = g % S;
        // the converters' arrival says the activations are widened; the TMA barrier itself makes the weights, written
        // by the copy engine, visible to this thread
        ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word) &&
             mbar_wait(smem_u32(&hdr->landed[s]), (g / S) & 1, abort_word);
        if (!ok) break;
        const uint8_t* const wst = stage0 + (size_t)s * p.stage_bytes;
        const float4* const xs0 = reinterpret_cast<const float4*>(wst + p.xslot_off) + pp;
        const int v0 = vbeg + st * J * LPR;
        const int jn = nlive > 0 ? min(J, nrounds - st * J) : 0;  // a warp without rows only hands the stage back
        // rounds whose vectors all lie inside the split take the unguarded body when every token slot is in use
        const int jfull = min(jn, (vend - v0) / LPR);
        const uint8_t* const wsrc0 = wst + (size_t)((cw * RS + rl) * p.pitch) + (size_t)pp * 16;
        const int group_stride = NC * RS * p.pitch;
        const int xround = M * 4 * HP;  // 16-byte entries of widened activations per round
        int j = 0;
        if (M == MT) {
          for (; j < jfull; ++j) {
            const uint8_t* const wsrc = wsrc0 + (size_t)j * (LPR * 16);
            const float4* const xs = xs0 + (size_t)j * xround;
            if (nlive == 1) sk_round_fast<MT, R, 1, HP, F16>(wsrc, group_stride, HP * 16, xs, acc);
            if constexpr (R >= 2) {
              if (nlive == 2) sk_round_fast<MT, R, 2, HP, F16>(wsrc, group_stride, HP * 16, xs, acc);
            }
            if constexpr (R >= 4) {
              if (nlive == 3) sk_round_fast<MT, R, 3, HP, F16>(wsrc, group_stride, HP * 16, xs, acc);
              if (nlive == 4) sk_round_fast<MT, R, 4, HP, F16>(wsrc, group_stride, HP * 16, xs, acc);
            }
          }
        }
        for (; j < jn; ++j) {
          const int va = v0 + j * LPR + pp;  // this thread's first vector of the round
          sk_round_guarded<MT, R, HP, F16>(wsrc0 + (size_t)j * (LPR * 16), group_stride, HP * 16, xs0 + (size_t)j * xround, nlive, M,
                                           va >= vend, va + HP >= vend, acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&hdr->empty[s]));
      }
      if (!ok) break;
      // butterfly: offset LPR/2 is the add of the thread's two halves, the rest are shuffles among the row's threads
#pragma unroll
      for (int u = 0; u < R; ++u) {
        if (u < nlive) {
          const int i = (u * NC + cw) * RS + rl;
          const int n = rb + r0 + i;
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            if (m < M) {
              float t = __fadd_rn(acc[u][m].x, acc[u][m].y);
#pragma unroll
              for (int off = HP / 2; off >= 1; off >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, off));
              if (i < nr && pp == m % HP) {  // every thread of the row holds t; they take turns storing
                if (p.ksplit == 1) sk_emit<F16>(p, m, n, t);
                else if (p.cluster) parked[(r0 + i) * M + m] = t;
                else p.ws[((int64_t)split * M + m) * p.N + n] = t;
              }
            }
          }
        }
      }
    }
    if (!ok && lane == 0) atomicCAS(p.status, 0u, (unsigned)ST_SKINNY_COMPUTE_WAIT);
  }

  if (p.ksplit == 1) return;

  if (p.cluster) {
    // The ksplit CTAs of a row range form a cluster (1, ksplit, 1); every thread of each passes both barriers. CTA k
    // finishes share k of the range's [row][token] entries, reading the parked partials in split order.
    cluster_arrive();
    cluster_wait();
    const uint32_t base = smem_u32(stage0 + (size_t)S * p.stage_bytes);
    const int count = nrows * M, share = (count + p.ksplit - 1) / p.ksplit;
    const int lo = (int)cluster_ctarank() * share, hi = min(count, lo + share);
    for (int i = lo + tid; i < hi; i += (int)blockDim.x) {
      uint32_t bits[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.ksplit) bits[k] = ld_cluster_u32(cluster_map_shared(base + (uint32_t)i * 4u, (uint32_t)k));
      float sum = __uint_as_float(bits[0]);
#pragma unroll
      for (int k = 1; k < 8; ++k)
        if (k < p.ksplit) sum = __fadd_rn(sum, __uint_as_float(bits[k]));
      sk_emit<F16>(p, i % M, rb + i / M, sum);
    }
    cluster_arrive();  // parked partials stay readable until every CTA of the cluster has finished
    cluster_wait();
    return;
  }

  // Workspace split-K: each writer fences its partials, the CTA counts itself in, and the CTA that completes the range's
  // count adds the ksplit planes in order and returns the counter to zero for the next launch.
  __threadfence();
  __syncthreads();
  if (tid == 0) hdr->last = atomicAdd(&p.counters[blockIdx.x], 1u) == (unsigned)(p.ksplit - 1) ? 1u : 0u;
  __syncthreads();
  if (!hdr->last) return;
  __threadfence();
  const int64_t plane = (int64_t)M * p.N;
  for (int i = tid; i < nrows * M; i += (int)blockDim.x) {
    const int m = i / nrows, n = rb + i % nrows;
    const float* const src = p.ws + (int64_t)m * p.N + n;
    float sum = 0.f;
    for (int k0 = 0; k0 < p.ksplit; k0 += 8) {  // eight partials in flight, added in split order
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k0 + k < p.ksplit) v[k] = __ldcg(src + (int64_t)(k0 + k) * plane);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k0 + k < p.ksplit) sum = (k0 + k == 0) ? v[k] : __fadd_rn(sum, v[k]);
    }
    sk_emit<F16>(p, m, n, sum);
  }
  if (tid == 0) p.counters[blockIdx.x] = 0u;
}

// ---------------------------------------------------------------------------------------------------------------
// host side

inline int sk_bucket(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }

// Opts the kernel in to large dynamic shared memory once per device (one bit per device, set atomically; the flag is
// a static of this template, so every kernel has its own), then launches it.
template <auto Kernel>
cudaError_t sk_go(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl, dim3 cluster, const CUtensorMap& tw,
                  const CUtensorMap& tx, const SkinnyDev& p) {
  static std::atomic<uint64_t> done{0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !((done.load(std::memory_order_acquire) >> dev) & 1ull)) {
    e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  }
  return launch_ex(Kernel, grid, block, smem, stream, pdl, cluster, tw, tx, p);
}

// Geometry of one launch. `rows`, `unroll`, `warps` are the caller's tile knobs (they never change a result bit):
//   rows   -> row groups a warp carries at once (clamped so that rows * token bucket <= 32 packed sums per thread)
//   unroll -> rounds of LPR vectors per pipeline stage (unroll / 2, at most 1 KB of K per row and stage)
//   warps  -> warps per CTA (2 * warps, three of them helpers; at most 16, or 12 when a thread carries 16 or more
//             packed sums); up to 8 warps per CTA two CTAs share an SM
template <int MT, int R, int LPR>
cudaError_t sk_launch_one(const SkinnyDev& in, int unroll, int warps, bool f16, bool pdl, cudaStream_t stream) {
  constexpr int HP = LPR / 2, RS = 32 / HP;
  SkinnyDev p = in;
  const int sms = sm_count() > 0 ? sm_count() : 1;
  // 2 * warps warps per CTA, three of them helpers. CTAs of at most 8 warps run two to an SM (registers and shared
  // memory are budgeted for it): the ring of one streams while the other computes or finishes, and in a chain of
  // dependent launches the next kernel's CTAs fill their rings beside the last CTAs of this one.
  int nc = 2 * warps - kSkHelperWarps;
  if (nc > SkinnyGeo<MT, R>::kMaxComputeWarps) nc = SkinnyGeo<MT, R>::kMaxComputeWarps;
  if (nc < 1) nc = 1;
  const int occ = nc + kSkHelperWarps <= 8 ? 2 : 1;
  // one wave of CTAs; a range is never empty; with the workspace split-K one counter per range must exist
  int64_t gx = (int64_t)sms * occ / p.ksplit;
  if (gx < 1) gx = 1;
  if (gx > p.N) gx = p.N;
  if (p.ksplit > 1 && !p.cluster && gx > in.max_ranges) gx = in.max_ranges;
  if (gx < 1) return cudaErrorInvalidValue;
  // cluster split-K parks [rows of the range][M] floats in shared memory: keep that below 48 KB
  if (p.cluster) {
    const int64_t need = ((int64_t)p.N * p.M * 4 + 48 * 1024 - 1) / (48 * 1024);
    if (gx < need) gx = need;
    if (gx > p.N) return cudaErrorInvalidConfiguration;
  }
  const int range = (int)((p.N + gx - 1) / gx);
  const int parked = p.cluster ? (range * p.M * 4 + 127) / 128 * 128 : 0;
  int J = unroll / 2 < 1 ? 1 : unroll / 2;
  if (J * LPR > 64) J = 64 / LPR;  // a TMA box is at most 256 four-byte elements wide
  const int budget = (occ == 2 ? 107 : 216) * 1024 - kSkHeaderBytes - parked;
  // a stage: the weight box (whole row groups, so that lanes of a partly filled group stay inside it), the activation
  // box, and the activations widened to fp32
  auto w_bytes_of = [&](int rp, int j) { return ((rp + RS - 1) / RS * RS * j * LPR * 16 + 127) / 128 * 128; };
  auto x_bytes_of = [&](int j) { return (p.M * j * LPR * 16 + 127) / 128 * 128; };
  auto stage_bytes_of = [&](int rp, int j) { return w_bytes_of(rp, j) + x_bytes_of(j) + j * p.M * LPR * 32; };
  // passes of equal length, so one box height serves them all
  int cap = nc * RS * R;
  if (cap > 256) cap = 256;
  int npass = (range + cap - 1) / cap;
  int rows_pass = (range + npass - 1) / npass;
  while (J > 1 && 3 * stage_bytes_of(rows_pass, J) > budget) J >>= 1;
  while (rows_pass > RS && 2 * stage_bytes_of(rows_pass, J) > budget) rows_pass = (rows_pass + 1) / 2;
  if (2 * stage_bytes_of(rows_pass, J) > budget) return cudaErrorInvalidConfiguration;
  p.rounds = J;
  p.rows_pass = rows_pass;
  p.pitch = J * LPR * 16;
  p.xraw_off = w_bytes_of(rows_pass, J);
  p.xraw_pitch = J * LPR * 16;
  p.xslot_off = p.xraw_off + x_bytes_of(J);
  p.stage_bytes = stage_bytes_of(rows_pass, J);
  p.w_box_bytes = rows_pass * p.pitch;
  p.x_box_bytes = p.M * p.xraw_pitch;
  // as deep as shared memory allows: the ring is what keeps enough bytes in flight per SM to cover the loaded latency
  // of HBM (about 2 us at full rate, some 90 KB per SM)
  int S = budget / p.stage_bytes;
  if (S > kSkMaxStages) S = kSkMaxStages;
  if (S < 2) return cudaErrorInvalidConfiguration;
  p.stages = S;
  // tensor maps over four-byte elements: box = chunk x rows, dense rows in shared memory, zero fill outside the tensor
  CUtensorMap tw, tx;
  if (!make_dense_map(&tw, p.w, (int64_t)p.K * 2, p.N, p.ldw * 2, p.pitch, rows_pass, true) ||
      !make_dense_map(&tx, p.x, (int64_t)p.K * 2, p.M, p.ldx * 2, p.xraw_pitch, p.M, false))
    return cudaErrorInvalidValue;
  const size_t smem = (size_t)kSkHeaderBytes + (size_t)S * p.stage_bytes + parked;
  const dim3 grid((unsigned)gx, (unsigned)p.ksplit), block((unsigned)((nc + kSkHelperWarps) * 32));
  const dim3 cluster(1, p.cluster ? (unsigned)p.ksplit : 1u, 1);
  if (f16) return sk_go<skinny_stream_kernel<MT, R, LPR, true>>(grid, block, smem, stream, pdl, cluster, tw, tx, p);
  return sk_go<skinny_stream_kernel<MT, R, LPR, false>>(grid, block, smem, stream, pdl, cluster, tw, tx, p);
}

template <int MT, int LPR>
cudaError_t sk_launch_rows(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  int r = rows;
  while (r * MT > 32) r >>= 1;  // at most 32 packed sums per thread
  if constexpr (MT <= 8) {
    if (r >= 4) return sk_launch_one<MT, 4, LPR>(p, unroll, warps, f16, pdl, s);
  }
  if (r >= 2) return sk_launch_one<MT, 2, LPR>(p, unroll, warps, f16, pdl, s);
  return sk_launch_one<MT, 1, LPR>(p, unroll, warps, f16, pdl, s);
}

template <int LPR>
cudaError_t sk_launch_lpr(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  switch (sk_bucket(p.M)) {
    case 1: return sk_launch_rows<1, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 2: return sk_launch_rows<2, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 4: return sk_launch_rows<4, LPR>(p, rows, unroll, warps, f16, pdl, s);
    case 8: return sk_launch_rows<8, LPR>(p, rows, unroll, warps, f16, pdl, s);
    default: return sk_launch_rows<16, LPR>(p, rows, unroll, warps, f16, pdl, s);
  }
}

}  // namespace llg
