// One-shot all-reduce (sum) of a small activation tensor across the GPUs of one node, over peer memory.
//
// Used at the two row-parallel boundaries of a tensor-parallel decode layer, where the payload is only M x hidden
// 16-bit values (16 KB per token at hidden 8192): pure latency. Every rank has written its partial into its own
// symmetric buffer (peer-mapped memory); each rank then reads all partials with plain 16-byte peer loads and adds them
// in rank order in fp32, so every rank obtains the same bits, run after run. No multicast, no TMA, no NVLS.
//
// Synchronisation: each CTA (or row) exchanges one signal with the same CTA on every peer. A signal is a system-scope
// add of 1 to a counter in the peer's memory, sent after a system-scope fence and without waiting for a reply; the
// receiver keeps, in its own memory, how many signals it has consumed from each peer and spins until the counter has
// passed that number. Counters only grow (compared through their wrapped difference), nothing is reset, so a captured
// launch replays as often as wanted as long as every rank replays the same sequence. Every spin is bounded; on
// expiry the kernel records a status code and carries on without waiting (the result is then undefined, the device
// stays usable). Buffers must alternate between consecutive all-reduces (the caller uses two): a rank may still be
// reading a peer's buffer of all-reduce n while that peer already writes the buffer of n+1.
// Flag memory per rank: 2 * slots * world words, zero before the first call - [slot][peer] arrival counters, written
// by the peers, then [slot][peer] consumed counts, private to the rank.
//
// The reference has no collective of any kind; this stands where NCCL's all_reduce would be called.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "llg_internal.h"
#include "ptx_sm100.cuh"

namespace llg {
namespace {

constexpr int kArThreads = 256;
std::atomic<long long> g_spin_cycles{2000000000ll};  // ~1 s; llg_set_wait_limit() shortens it for failure tests

__device__ __forceinline__ void flag_send(uint32_t* counter) {
  atomicAdd_system(counter, 1u);  // result unused: a reduction, nothing comes back over the link
}
// Waits until `counter` (written by one peer) has passed this rank's count of consumed signals, which it advances.
__device__ __forceinline__ bool flag_recv(const uint32_t* counter, uint32_t* consumed, long long limit) {
  const uint32_t want = *consumed + 1u;
  *consumed = want;
  const long long t0 = clock64();
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    if ((int32_t)(seen - want) >= 0) return true;
    if (clock64() - t0 > limit) return false;
  }
}
// One signal to and one from peer `peer`, for slot `slot` (a CTA or a row) of `slots`.
__device__ __forceinline__ bool exchange(uint32_t* const* flags, int slot, int slots, int peer, int rank, int world,
                                         long long limit) {
  __threadfence_system();
  flag_send(flags[peer] + (int64_t)slot * world + rank);
  uint32_t* const mine = flags[rank];
  const bool ok = flag_recv(mine + (int64_t)slot * world + peer, mine + ((int64_t)slots + slot) * world + peer, limit);
  __threadfence_system();
  return ok;
}

struct ArDev {
  const void* const* buffers;   // [world] device pointers, one symmetric buffer per rank (index = rank)
  uint32_t* const* flags;       // [world] device pointers to each rank's flag words: [ctas][world]
  void* out;
  int64_t vecs;                 // 16-byte vectors to reduce
  int rank, world, dtype;
  unsigned* status;
  long long spin;               // bound of every wait for a peer's signal, in cycles
};

template <int DT>
__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4& v, bool first) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  if constexpr (DT == LLG_DT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = first ? __uint_as_float(w[i]) : acc[i] + __uint_as_float(w[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float lo, hi;
      if constexpr (DT == LLG_DT_BF16) {
        lo = __uint_as_float(w[i] << 16);
        hi = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        lo = t.x;
        hi = t.y;
      }
      acc[2 * i] = first ? lo : acc[2 * i] + lo;
      acc[2 * i + 1] = first ? hi : acc[2 * i + 1] + hi;
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArDev p) {
  const int tid = threadIdx.x, cta = blockIdx.x;
  pdl_trigger();  // the GEMM behind this kernel may start streaming its weight
  pdl_wait();     // the GEMM before it must have finished writing this rank's partial
  // ---- all partials of this CTA's peers are written: exchange flags ----
  if (tid < p.world) {
    if (!exchange(p.flags, cta, LLG_AR_MAX_CTAS, tid, p.rank, p.world, p.spin))  // tell peer `tid`, hear from peer `tid`
      atomicCAS(p.status, 0u, (unsigned)ST_ALLREDUCE_WAIT);
  }
  __syncthreads();
  // ---- reduce this CTA's share in rank order ----
  const int64_t per = (p.vecs + gridDim.x - 1) / gridDim.x;
  const int64_t lo = per * cta, hi = lo + per < p.vecs ? lo + per : p.vecs;
  for (int64_t i = lo + tid; i < hi; i += kArThreads) {
    uint4 v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.world) v[r] = __ldcv(static_cast<const uint4*>(p.buffers[r]) + i);  // volatile: never a stale cached line
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.world) accumulate<DT>(acc, v[r], r == 0);
    uint4 o;
    if constexpr (DT == LLG_DT_F32) {
      o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
    } else if constexpr (DT == LLG_DT_BF16) {
      __nv_bfloat162 t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) t[j] = __halves2bfloat162(__float2bfloat16_rn(acc[2 * j]), __float2bfloat16_rn(acc[2 * j + 1]));
      o = *reinterpret_cast<const uint4*>(t);
    } else {
      __half2 t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) t[j] = __halves2half2(__float2half_rn(acc[2 * j]), __float2half_rn(acc[2 * j + 1]));
      o = *reinterpret_cast<const uint4*>(t);
    }
    static_cast<uint4*>(p.out)[i] = o;
  }
}

// ---- all-reduce fused with the per-token FP8 quantizer --------------------------------------------------------------
// One CTA per row (token): the row's partials are added in rank order in fp32 and rounded to the activation type -
// the very values the stand-alone all-reduce would have stored - and the quantizer's arithmetic follows on them in
// registers (scale = max(amax / 448, min_scale), IEEE division for the scale and its reciprocal, one multiply per
// element, cvt.rn.satfinite.e4m3x2), so (q, scale) equal quantize_fp8(all_reduce(x)) bit for bit while one kernel and
// one dependent launch disappear from the chain. The rounded sum itself is stored too when the caller asks for it.
constexpr int kArqThreads = 1024, kArqUnits = 2;  // rows up to 1024 * 2 * 8 = 16384 elements

struct ArqDev {
  const void* const* buffers;
  uint32_t* const* flags;
  void* out;             // optional [rows, cols] rounded sum (same type as the partials), may be null
  unsigned char* q;      // [rows, ldq] e4m3 bytes
  float* scale_out;      // [rows]
  int64_t ldq;
  int cols, rank, world;
  float min_scale;
  unsigned* status;
  long long spin;
};

template <int DT>
__global__ void __launch_bounds__(kArqThreads) allreduce_quant_fp8_kernel(const ArqDev p) {
  const int tid = threadIdx.x, row = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  __shared__ float red[kArqThreads / 32];
  if (tid < p.world) {
    if (!exchange(p.flags, row, LLG_AR_MAX_CTAS, tid, p.rank, p.world, p.spin)) atomicCAS(p.status, 0u, (unsigned)ST_ALLREDUCE_WAIT);
  }
  __syncthreads();
  const int units = p.cols >> 3;  // 8 values = 16 bytes per unit
  float r[kArqUnits][8];
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < kArqUnits; ++j) {
    const int u = tid + j * kArqThreads;
    if (u < units) {
      const int64_t i = (int64_t)row * units + u;
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.world) v[k] = __ldcv(static_cast<const uint4*>(p.buffers[k]) + i);
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.world) accumulate<DT>(acc, v[k], k == 0);
      uint4 o;
      if constexpr (DT == LLG_DT_BF16) {
        __nv_bfloat162 t[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) t[e] = __halves2bfloat162(__float2bfloat16_rn(acc[2 * e]), __float2bfloat16_rn(acc[2 * e + 1]));
        o = *reinterpret_cast<const uint4*>(t);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          r[j][2 * e] = __bfloat162float(t[e].x);
          r[j][2 * e + 1] = __bfloat162float(t[e].y);
        }
      } else {
        __half2 t[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) t[e] = __halves2half2(__float2half_rn(acc[2 * e]), __float2half_rn(acc[2 * e + 1]));
        o = *reinterpret_cast<const uint4*>(t);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(t[e]);
          r[j][2 * e] = f.x;
          r[j][2 * e + 1] = f.y;
        }
      }
      if (p.out) static_cast<uint4*>(p.out)[i] = o;
#pragma unroll
      for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(r[j][e]));
    }
  }
  // row maximum over the CTA
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
  if ((tid & 31) == 0) red[tid >> 5] = a;
  __syncthreads();
  a = red[tid & 31];  // kArqThreads / 32 == 32 partial maxima
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
  const float scale = fmaxf(__fdiv_rn(a, 448.f), p.min_scale);
  if (tid == 0) p.scale_out[row] = scale;
  const float inv = __fdiv_rn(1.f, scale);
  unsigned char* const q = p.q + (int64_t)row * p.ldq;
#pragma unroll
  for (int j = 0; j < kArqUnits; ++j) {
    const int u = tid + j * kArqThreads;
    if (u < units) {
      const uint32_t w0 = cvt_e4m3x2(__fmul_rn(r[j][0], inv), __fmul_rn(r[j][1], inv)) |
                          (cvt_e4m3x2(__fmul_rn(r[j][2], inv), __fmul_rn(r[j][3], inv)) << 16);
      const uint32_t w1 = cvt_e4m3x2(__fmul_rn(r[j][4], inv), __fmul_rn(r[j][5], inv)) |
                          (cvt_e4m3x2(__fmul_rn(r[j][6], inv), __fmul_rn(r[j][7], inv)) << 16);
      *reinterpret_cast<uint2*>(q + u * 8) = make_uint2(w0, w1);
    }
  }
}

// ---- consumer of pushed partials -------------------------------------------------------------------------------------
// The row-parallel GEMM of every rank has stored its [rows, cols] partial into region `src` of THIS rank's receive
// buffer and signalled each row (umma_gemm.cuh, push mode). One CTA per row waits for the `world` signals of its row,
// adds the local copies in rank order in fp32 and rounds to the activation type - the all-reduce's result, bit for bit
// what allreduce_oneshot_kernel produces - then, all optional and in this order: adds the residual (fp32 add of the two
// 16-bit values, one rounding: what a separate elementwise add would store), stores the new hidden state, and runs the
// per-token FP8 quantizer on it. Nothing crosses NVLink here; the pull round trip of the other kernels is gone.
struct RlDev {
  const unsigned char* recv;   // world regions of region_bytes each
  int64_t region_bytes;
  uint32_t* flags;             // this rank's flag words: [slots][world] arrivals, then [slots][world] consumed counts
  void* out;                   // optional [rows, cols] result in the partials' type
  const void* residual;        // optional [rows, cols], same type
  unsigned char* q;            // optional [rows, ldq] e4m3 bytes
  float* scale_out;
  int64_t ldq;
  int cols, world;
  float min_scale;
  unsigned* status;
  long long spin;
};

template <int DT>
__global__ void __launch_bounds__(kArqThreads) reduce_local_kernel(const RlDev p) {
  const int tid = threadIdx.x, row = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  __shared__ float red[kArqThreads / 32];
  if (tid < p.world) {
    if (!flag_recv(p.flags + (int64_t)row * p.world + tid, p.flags + ((int64_t)LLG_AR_MAX_CTAS + row) * p.world + tid, p.spin))
      atomicCAS(p.status, 0u, (unsigned)ST_ALLREDUCE_WAIT);
  }
  __syncthreads();  // the waiters' acquire loads, then this barrier: every thread may now read the partials
  const int units = p.cols >> 3;
  float r[kArqUnits][8];
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < kArqUnits; ++j) {
    const int u = tid + j * kArqThreads;
    if (u < units) {
      const int64_t i = (int64_t)row * units + u;
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.world) v[k] = __ldcv(reinterpret_cast<const uint4*>(p.recv + (int64_t)k * p.region_bytes) + i);
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < p.world) accumulate<DT>(acc, v[k], k == 0);
      uint4 res = make_uint4(0u, 0u, 0u, 0u);
      if (p.residual) res = __ldg(static_cast<const uint4*>(p.residual) + i);
      const uint32_t rw[4] = {res.x, res.y, res.z, res.w};
      uint32_t ow[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float lo, hi, rlo, rhi;
        if constexpr (DT == LLG_DT_BF16) {
          const __nv_bfloat162 t = __halves2bfloat162(__float2bfloat16_rn(acc[2 * e]), __float2bfloat16_rn(acc[2 * e + 1]));
          lo = __bfloat162float(t.x), hi = __bfloat162float(t.y);
          rlo = __uint_as_float(rw[e] << 16), rhi = __uint_as_float(rw[e] & 0xffff0000u);
          if (p.residual) {
            const __nv_bfloat162 s2 = __halves2bfloat162(__float2bfloat16_rn(__fadd_rn(lo, rlo)), __float2bfloat16_rn(__fadd_rn(hi, rhi)));
            lo = __bfloat162float(s2.x), hi = __bfloat162float(s2.y);
            ow[e] = *reinterpret_cast<const uint32_t*>(&s2);
          } else {
            ow[e] = *reinterpret_cast<const uint32_t*>(&t);
          }
        } else {
          const __half2 t = __halves2half2(__float2half_rn(acc[2 * e]), __float2half_rn(acc[2 * e + 1]));
          const float2 f = __half22float2(t);
          lo = f.x, hi = f.y;
          const float2 rf = __half22float2(*reinterpret_cast<const __half2*>(&rw[e]));
          rlo = rf.x, rhi = rf.y;
          if (p.residual) {
            const __half2 s2 = __halves2half2(__float2half_rn(__fadd_rn(lo, rlo)), __float2half_rn(__fadd_rn(hi, rhi)));
            const float2 g = __half22float2(s2);
            lo = g.x, hi = g.y;
            ow[e] = *reinterpret_cast<const uint32_t*>(&s2);
          } else {
            ow[e] = *reinterpret_cast<const uint32_t*>(&t);
          }
        }
        r[j][2 * e] = lo;
        r[j][2 * e + 1] = hi;
      }
      if (p.out) static_cast<uint4*>(p.out)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
#pragma unroll
      for (int e = 0; e < 8; ++e) a = fmaxf(a, fabsf(r[j][e]));
    }
  }
  if (!p.q) return;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
  if ((tid & 31) == 0) red[tid >> 5] = a;
  __syncthreads();
  a = red[tid & 31];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
  const float scale = fmaxf(__fdiv_rn(a, 448.f), p.min_scale);
  if (tid == 0) p.scale_out[row] = scale;
  const float inv = __fdiv_rn(1.f, scale);
  unsigned char* const q = p.q + (int64_t)row * p.ldq;
#pragma unroll
  for (int j = 0; j < kArqUnits; ++j) {
    const int u = tid + j * kArqThreads;
    if (u < units) {
      const uint32_t w0 = cvt_e4m3x2(__fmul_rn(r[j][0], inv), __fmul_rn(r[j][1], inv)) |
                          (cvt_e4m3x2(__fmul_rn(r[j][2], inv), __fmul_rn(r[j][3], inv)) << 16);
      const uint32_t w1 = cvt_e4m3x2(__fmul_rn(r[j][4], inv), __fmul_rn(r[j][5], inv)) |
                          (cvt_e4m3x2(__fmul_rn(r[j][6], inv), __fmul_rn(r[j][7], inv)) << 16);
      *reinterpret_cast<uint2*>(q + u * 8) = make_uint2(w0, w1);
    }
  }
}

}  // namespace

long long ar_spin_cycles() { return g_spin_cycles.load(std::memory_order_relaxed); }
void set_ar_spin_cycles(long long cycles) { g_spin_cycles.store(cycles, std::memory_order_relaxed); }

cudaError_t reduce_local_launch(const void* recv, int64_t region_bytes, uint32_t* flags, void* out, const void* residual,
                                void* q, int64_t ldq, float* scale_out, int rows, int cols, int dtype, float min_scale,
                                int world, unsigned* status, cudaStream_t s) {
  RlDev p{static_cast<const unsigned char*>(recv), region_bytes, flags, out, residual, static_cast<unsigned char*>(q),
          scale_out, ldq, cols, world, min_scale, status, ar_spin_cycles()};
  const bool pdl = pdl_on();
  const dim3 grid(rows), block(kArqThreads), one(1, 1, 1);
  switch (dtype) {
    case LLG_DT_BF16: return launch_ex(reduce_local_kernel<LLG_DT_BF16>, grid, block, 0, s, pdl, one, p);
    case LLG_DT_F16: return launch_ex(reduce_local_kernel<LLG_DT_F16>, grid, block, 0, s, pdl, one, p);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t allreduce_quant_fp8_launch(const void* const* buffers, uint32_t* const* flags, void* out, void* q, int64_t ldq,
                                       float* scale_out, int rows, int cols, int dtype, float min_scale, int rank,
                                       int world, unsigned* status, cudaStream_t s) {
  ArqDev p{buffers, flags, out, static_cast<unsigned char*>(q), scale_out, ldq, cols, rank, world, min_scale, status, ar_spin_cycles()};
  const bool pdl = pdl_on();
  const dim3 grid(rows), block(kArqThreads), one(1, 1, 1);
  switch (dtype) {
    case LLG_DT_BF16: return launch_ex(allreduce_quant_fp8_kernel<LLG_DT_BF16>, grid, block, 0, s, pdl, one, p);
    case LLG_DT_F16: return launch_ex(allreduce_quant_fp8_kernel<LLG_DT_F16>, grid, block, 0, s, pdl, one, p);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t allreduce_launch(const void* const* buffers, uint32_t* const* flags, void* out, int64_t vecs, int rank,
                             int world, int dtype, int ctas, unsigned* status, cudaStream_t s) {
  ArDev p{buffers, flags, out, vecs, rank, world, dtype, status, ar_spin_cycles()};
  const bool pdl = pdl_on();
  const dim3 grid(ctas), block(kArThreads), one(1, 1, 1);
  switch (dtype) {
    case LLG_DT_BF16: return launch_ex(allreduce_oneshot_kernel<LLG_DT_BF16>, grid, block, 0, s, pdl, one, p);
    case LLG_DT_F16: return launch_ex(allreduce_oneshot_kernel<LLG_DT_F16>, grid, block, 0, s, pdl, one, p);
    case LLG_DT_F32: return launch_ex(allreduce_oneshot_kernel<LLG_DT_F32>, grid, block, 0, s, pdl, one, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace llg
