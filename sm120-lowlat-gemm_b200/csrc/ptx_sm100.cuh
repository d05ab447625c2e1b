// Inline-PTX building blocks for sm_100a: mbarrier, TMA (non-multicast), tcgen05 (TMEM, MMA, commit, ld/st),
// thread-block-cluster shared memory, programmatic dependent launch and L2 prefetch.
//
// Replaces the role of the reference's csrc/ptx.cuh:18-215 (cp.async / ldmatrix / mma.sync wrappers) and
// csrc/pdl.cuh:17-35; none of those instruction forms are used here.
//
// Every wait in this file is bounded: a wait that runs out of time returns false, the caller records a status code
// and leaves the kernel in an orderly way (no trap, no endless spin).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llg {

// ---------------------------------------------------------------------------------------------------------------
// misc

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------------------------
// programmatic dependent launch + L2 prefetch

// Blocks until the grid this launch depends on has finished and its writes are visible (no-op without PDL).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Allows the next kernel of the stream to start its pre-wait part.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Fire-and-forget pull of share `part` of `parts` of [ptr, ptr+bytes) into L2, 16 KB per instruction, issued by
// `nthreads` cooperating threads of which the caller is number `t`. ptr must be 16-byte aligned.
__device__ __forceinline__ void l2_prefetch_share(const void* ptr, int64_t bytes, int64_t part, int64_t parts, int t,
                                                  int nthreads) {
  if (ptr == nullptr || bytes < 16) return;
  const int64_t units = bytes >> 4;
  const int64_t lo = units * part / parts * 16, hi = units * (part + 1) / parts * 16;
  for (int64_t off = lo + (int64_t)t * 16384; off < hi; off += (int64_t)nthreads * 16384) {
    const uint32_t n = (uint32_t)(hi - off < 16384 ? hi - off : 16384);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(static_cast<const char*>(ptr) + off), "r"(n)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------------------
// mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// About one second at B200 clocks; far beyond any legitimate wait of these kernels (tens of microseconds).
constexpr long long kWaitCycles = 2000000000ll;

// Bounded wait for phase `parity` of an mbarrier. `abort_word` is a shared-memory word that any thread of the CTA
// sets once it gave up; other waiters then give up as well, so that the CTA drains instead of spinning.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 63u) == 0u) {
      if (*abort_word != 0u) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_word = 1u;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// TMA: 2-D tiled load into this CTA's shared memory, completion counted on an mbarrier (no multicast anywhere)

// Bring one box of a tiled map into L2 only (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(m), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// x = innermost coordinate (bytes here, always a multiple of 16), y = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05 operands).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------------------
// cp.async (only for data TMA cannot carry: 4-byte-aligned block-scale rows)

__device__ __forceinline__ void cp_async4_zfill(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 4u : 0u;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
// Arrives on the mbarrier once all earlier cp.async of this thread have landed (does not change the pending count).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tcgen05: tensor memory

__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 bit x 16 columns: thread i of the warp receives lane (base lane + i), columns [col, col+16).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 32 bit x 8 columns store: thread i writes lane (base lane + i), columns [col, col+8).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// tcgen05: descriptors and MMA issue

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes, TMA 128-byte swizzle, tile base
// 1024-byte aligned. Groups of 8 rows are 1024 bytes apart (stride byte offset); the leading byte offset is unused
// for swizzled K-major layouts. Bits 46-47 = 1 mark the sm_100 descriptor version, bits 61-63 = 2 select the
// 128-byte swizzle.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Descriptor of a 32-row x 16-byte block of unswizzled shared memory (8-row groups 128 bytes apart), the source
// format of tcgen05.cp.32x128b.
__device__ __forceinline__ uint64_t umma_desc_plain128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)(128u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
#define LLG_MMA_SS(KINDSTR)                                                                              \
  asm volatile(                                                                                          \
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                  \
      "tcgen05.mma.cta_group::1.kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),           \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                                               \
      : "memory")

__device__ __forceinline__ void mma_ss_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  LLG_MMA_SS("f16");
}
__device__ __forceinline__ void mma_ss_f8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  LLG_MMA_SS("f8f6f4");
}
__device__ __forceinline__ void mma_ss_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  LLG_MMA_SS("i8");
}
#undef LLG_MMA_SS

// D[tmem] (+)= A[tmem] * B[smem] (A was widened into tensor memory by the converter warps).
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled NVFP4: e2m1 operands, one ue4m3 scale per 16 K (4 per MMA of K=64) read from tensor memory.
__device__ __forceinline__ void mma_ss_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::
          "r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated into all four 32-lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Arrives on the mbarrier when every MMA (and tcgen05.cp) this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Instruction descriptor (dense, K-major A and B): accumulator format at bits 4-5 (1 = f32, 2 = s32), A format at
// 7-9, B format at 10-12, N/8 at 17-22, M/16 at 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m,
                                                  uint32_t n) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Block-scaled variant: no accumulator-format field; scale format at bit 23 (0 = ue4m3); scale ids 0.
__host__ __device__ constexpr uint32_t umma_idesc_bs(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
  return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------------------------
// thread-block cluster

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------------------------
// global loads / conversions

// 16-byte streaming weight load: read-only path, no L1 allocation, 256-byte L2 sector prefetch.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Two floats -> two e4m3 bytes (lo in the low byte), round to nearest even, saturating to +-448.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// Two floats -> one byte of two e2m1 nibbles (lo in the low nibble), round to nearest even, saturating to +-6.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{\n\t.reg .b8 b;\n\t.reg .b16 h;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\t"
      "mov.b16 h, {b, b};\n\t"
      "cvt.u32.u16 %0, h;\n\t}\n"
      : "=r"(r)
      : "f"(hi), "f"(lo));
  return r & 0xffu;
}

// ---------------------------------------------------------------------------------------------------------------
// CTA pairs (cta_group::2): the two CTAs of a cluster (1 x 2) run one 256-row MMA. Each holds its 128 rows of A, its
// half of B and its 128 lanes of the accumulator; the CTA of cluster rank 0 issues the MMAs for both. Loads never use
// multicast: each CTA fetches its own operands and reports the bytes to the issuing CTA's barrier.

// One warp of EACH CTA of the pair executes the allocation (same warp index, same holder address) and the release.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t holder_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 2-D tiled load into THIS CTA's shared memory whose bytes are counted on `bar`, a shared::cluster address that may
// lie in the other CTA of the pair (mapa).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// D[tmem of both CTAs] (+)= A * B with both operands in the shared memory of both CTAs (same offsets in each).
#define LLG_MMA_SS_PAIR(KINDSTR)                                                                         \
  asm volatile(                                                                                          \
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                                  \
      "tcgen05.mma.cta_group::2.kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),           \
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                                               \
      : "memory")
__device__ __forceinline__ void mma_pair_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  LLG_MMA_SS_PAIR("f16");
}
__device__ __forceinline__ void mma_pair_f8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  LLG_MMA_SS_PAIR("f8f6f4");
}
__device__ __forceinline__ void mma_pair_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  LLG_MMA_SS_PAIR("i8");
}
#undef LLG_MMA_SS_PAIR

// Arrives on the mbarrier at this shared-memory offset in every CTA of `cta_mask` once the pair's MMAs issued so far
// have completed (a barrier signal fanned out to both CTAs; no data moves).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask)
               : "memory");
}

// Arrive on an mbarrier of any CTA of the cluster (address from cluster_map_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

}  // namespace llg
