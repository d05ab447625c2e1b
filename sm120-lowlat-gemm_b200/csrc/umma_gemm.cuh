// Tensor-core GEMM for sm_100a: C[p,q] = sum_k A[p,k] B[q,k], both operands K-contiguous.
//
// One CTA computes a 128 x BQ output tile for one K partition:
//   warp 0      TMA producer: 128-byte-swizzled tiles of A and B into a ring of shared-memory stages
//   warp 1      allocates tensor memory and issues tcgen05.mma (accumulator lives in tensor memory)
//   warps 2-5   epilogue: tcgen05.ld the accumulator, scale / bias / convert / store, split-K reduction; while it
//               has nothing to do, one of them asks for the CTA's later weight stages to be brought into L2
//   warps 6-    helpers, only for some kinds: NVFP4 - four warps put the block scales of every stage into the layout
//               the MMA's scale copy reads; W8A16 / W4A16 - 8 warps widen the weight tile exactly into tensor
//               memory (the MMA then takes A from there), in two groups that take alternate stages
// The host maps (activation, weight) onto (A, B): with few tokens the weight is A ("swap": its rows fill the 128
// MMA rows, the tokens sit on the narrow N side and y is stored transposed).
//
// Reference behaviour reproduced (not its implementation): operand orientation and epilogue of
// csrc/tc_gemm.cuh:146-168,411-425; workspace split-K with last-arriver in-order reduction and counter reset
// (:462-500); cluster split-K over distributed shared memory, bit-identical to the workspace path (:427-460);
// weight-first streaming before the PDL dependency wait and the pdl_early rule (:386-409, 533); zero contribution
// of K tails and out-of-range rows (here by TMA zero fill instead of predicated cp.async, :213-255).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>

#include "llg_internal.h"
#include "ptx_sm100.cuh"

namespace llg {

constexpr int kBP = 128;
constexpr int kAtomBytes = 128;           // bytes of K per row in one swizzle atom
constexpr int kAAtomTile = kBP * 128;     // one A atom tile in shared memory
constexpr int kHeaderBytes = 2048;
constexpr int kSfLag = 3;                 // block-scale cp.async groups kept in flight per thread

template <int FAM, int BQ, int ATOMS>
struct Geo {
  static constexpr bool kMixed = FAM == FAM_W8A16 || FAM == FAM_W4A16;
  static constexpr bool kNvf4 = FAM == FAM_NVF4;
  static constexpr bool kIntAcc = FAM == FAM_I8;
  static constexpr bool kHelpers = kMixed || kNvf4;              // warps 6..: converter / block-scale feeder
  // helper threads per tile row: the widening is ALU work, so several warps share each 32-lane quarter of tensor memory
  static constexpr int kParts = FAM == FAM_W4A16 ? 2 : FAM == FAM_W8A16 ? 2 : 1;
  static constexpr int kHelperThreads = kHelpers ? 128 * kParts : 0;
  // the converter warps of the mixed kinds form two groups that take alternate stages (each owns one of the two widened
  // A buffers), so the waits and the store latency of one stage overlap the arithmetic of the next; within a group
  // kSubParts threads share a row
  static constexpr int kGroups = kMixed ? 2 : 1;
  static constexpr int kSubParts = kParts / kGroups;
  static constexpr int kThreads = 192 + kHelperThreads;
  static constexpr int kBPerA = FAM == FAM_W8A16 ? 2 : FAM == FAM_W4A16 ? 4 : 1;  // B atoms per A atom
  static constexpr int kBAtomTile = BQ * 128;
  static constexpr int kABytes = ATOMS * kAAtomTile;
  static constexpr int kBBytes = ATOMS * kBPerA * kBAtomTile;
  static constexpr int kSfA = (kNvf4 || FAM == FAM_W4A16) ? ATOMS * 2048 : 0;  // 128 rows x 16 scale bytes per atom
  static constexpr int kSfB = kNvf4 ? ATOMS * 2048 : 0;
  static constexpr int kAOff = 0, kBOff = kABytes, kSfAOff = kBOff + kBBytes, kSfBOff = kSfAOff + kSfA;
  static constexpr int kStageBytes = (kSfBOff + kSfB + 1023) / 1024 * 1024;
  static constexpr uint32_t kTxBytes = kABytes + kBBytes;
  // tensor-memory columns: accumulator buffers first, then widened-A buffers or block-scale columns
  static constexpr int kAccCols = BQ < 32 ? 32 : BQ;
  static constexpr int kAColsAtom = FAM == FAM_W8A16 ? 64 : FAM == FAM_W4A16 ? 128 : 0;  // widened A, 2 K per column
  static constexpr int kABufs = 2;
  static constexpr int kSfColsStage = kNvf4 ? ATOMS * 4 * 8 : 0;  // per MMA 4 columns for A scales + 4 for B
  static constexpr int kOtherCols = (kMixed ? kABufs * ATOMS * kAColsAtom : 0) + 2 * kSfColsStage;
  static constexpr int kAccBufs = 2 * kAccCols + kOtherCols <= 512 ? 2 : 1;  // two: epilogue overlaps the next item
  static constexpr int kNeedCols = kAccBufs * kAccCols + kOtherCols;
  static constexpr int kTmemCols = kNeedCols <= 32 ? 32 : kNeedCols <= 64 ? 64 : kNeedCols <= 128 ? 128
                                   : kNeedCols <= 256 ? 256 : 512;
  static constexpr bool kValid = kNeedCols <= 512 && (!kNvf4 || BQ <= 128) && kStageBytes * 2 <= kSmemBudget;
};

struct SmemHeader {
  uint64_t full[LLG_MAX_STAGES];     // TMA bytes of a stage have landed
  uint64_t empty[LLG_MAX_STAGES];    // the MMAs that read a stage have completed
  uint64_t sf_full[LLG_MAX_STAGES];  // block scales of a stage are in shared memory (128 arrivals)
  uint64_t acc_full[2];              // every MMA of the item that used this accumulator buffer has completed
  uint64_t acc_empty[2];             // the epilogue has read the buffer out (128 arrivals)
  uint64_t a_full[2];                // widened A buffer written to tensor memory (128 arrivals)
  uint64_t a_empty[2];               // MMAs reading a widened A buffer have completed
  uint32_t tmem_base;
  uint32_t abort;
  uint32_t last;
  uint32_t trace_slot;
  uint32_t prod_stage;               // first item: stages the producer has issued (0 until the dependency resolved)
  // column-side epilogue factors (scale, bias as fp32) of the tile in flight, tiles up to 64 columns wide; two sets,
  // so that the fetch for the next item never overwrites what a slower epilogue warp still reads
  alignas(16) float colf[2][2][64];
};
static_assert(sizeof(SmemHeader) <= kHeaderBytes, "header too large");

__device__ __forceinline__ void give_up(const TcDev& prm, uint32_t code) { atomicCAS(prm.status, 0u, code); }

// Element i of a scale vector that may be absent (1), a scalar or a full vector. Written as selects and a predicated
// load rather than branches: the epilogue runs as one warp per scheduler, where a branch is paid in full.
__device__ __forceinline__ float tc_vec(const float* p, int len, int i) {
  const float* const at = p + (len > 1 ? i : 0);
  return len == 0 ? 1.f : __ldg(at);
}
__device__ __forceinline__ float tc_bias(const TcDev& prm, int i) {
  const bool wide = prm.bias_dtype == LLG_DT_F32;
  const float f = wide ? __ldg(static_cast<const float*>(prm.bias) + i) : 0.f;
  const unsigned short h = wide ? (unsigned short)0 : __ldg(static_cast<const unsigned short*>(prm.bias) + i);
  const float from_bf16 = __uint_as_float((uint32_t)h << 16);
  const float from_f16 = __half2float(__ushort_as_half(h));
  return wide ? f : (prm.bias_dtype == LLG_DT_BF16 ? from_bf16 : from_f16);
}

// v = ((acc * alpha) * row_scale[p]) * col_scale[q] (+ bias), every operation individually rounded.
template <bool INT_ACC>
__device__ __forceinline__ float tc_finish(const TcDev& prm, float alpha, int p, int q, uint32_t bits) {
  const float acc = INT_ACC ? (float)(int32_t)bits : __uint_as_float(bits);
  float v = __fmul_rn(__fmul_rn(__fmul_rn(acc, alpha), tc_vec(prm.row_scale, prm.row_scale_len, p)),
                      tc_vec(prm.col_scale, prm.col_scale_len, q));
  if (prm.bias_dtype != LLG_DT_NONE) v = __fadd_rn(v, tc_bias(prm, prm.bias_on_p ? p : q));
  return v;
}
// Same arithmetic with the row-side factors (row scale, bias when it is indexed by p) already in registers.
template <bool INT_ACC>
__device__ __forceinline__ float tc_finish_row(const TcDev& prm, float alpha, float rs, float bias_p, int q, uint32_t bits) {
  const float acc = INT_ACC ? (float)(int32_t)bits : __uint_as_float(bits);
  float v = __fmul_rn(__fmul_rn(__fmul_rn(acc, alpha), rs), tc_vec(prm.col_scale, prm.col_scale_len, q));
  if (prm.bias_dtype != LLG_DT_NONE) v = __fadd_rn(v, prm.bias_on_p ? bias_p : tc_bias(prm, q));
  return v;
}
__device__ __forceinline__ void tc_store_to(void* y, int out_dtype, int64_t at, float v) {
  // three predicated stores of which one executes (the type is uniform over the grid)
  if (out_dtype == LLG_DT_BF16) static_cast<__nv_bfloat16*>(y)[at] = __float2bfloat16_rn(v);
  if (out_dtype == LLG_DT_F16) static_cast<__half*>(y)[at] = __float2half_rn(v);
  if (out_dtype == LLG_DT_F32) static_cast<float*>(y)[at] = v;
}
// One finished output element. In push mode it goes to every rank's copy of this rank's partial (plain stores into
// peer-mapped memory; the transfer so overlaps the tiles that are still being computed) instead of to y.
__device__ __forceinline__ void tc_store(const TcDev& prm, int p, int q, float v) {
  const int64_t at = prm.swap ? (int64_t)q * prm.ldy + p : (int64_t)p * prm.ldy + q;
  if (prm.push_n == 0) {
    tc_store_to(prm.y, prm.out_dtype, at, v);
    return;
  }
#pragma unroll
  for (int d = 0; d < 8; ++d)
    if (d < prm.push_n) tc_store_to(prm.push_y[d], prm.out_dtype, at, v);
}

// Column-side factors of 16 consecutive columns: scale (1 when absent) and bias as fp32 (0 when absent or indexed by
// p). The kind of vector is decided once per call, so the 16 loads are straight-line code: the epilogue runs as one
// warp per scheduler with nothing to hide a branch behind.
__device__ __forceinline__ void tc_col_factors(const TcDev& prm, int q_first, float (&cs)[16], float (&cb)[16]) {
  const int last = prm.Q - 1;
  if (prm.col_scale_len > 1) {
#pragma unroll
    for (int c = 0; c < 16; ++c) cs[c] = __ldg(prm.col_scale + min(q_first + c, last));
  } else {
    const float one = prm.col_scale_len == 1 ? __ldg(prm.col_scale) : 1.f;
#pragma unroll
    for (int c = 0; c < 16; ++c) cs[c] = one;
  }
  if (prm.bias_dtype == LLG_DT_NONE || prm.bias_on_p) {
#pragma unroll
    for (int c = 0; c < 16; ++c) cb[c] = 0.f;
  } else if (prm.bias_dtype == LLG_DT_BF16) {
#pragma unroll
    for (int c = 0; c < 16; ++c) cb[c] = __bfloat162float(static_cast<const __nv_bfloat16*>(prm.bias)[min(q_first + c, last)]);
  } else if (prm.bias_dtype == LLG_DT_F16) {
#pragma unroll
    for (int c = 0; c < 16; ++c) cb[c] = __half2float(static_cast<const __half*>(prm.bias)[min(q_first + c, last)]);
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c) cb[c] = __ldg(static_cast<const float*>(prm.bias) + min(q_first + c, last));
  }
}

// The same two factors for one column (scale in .x, bias in .y).
__device__ __forceinline__ float2 tc_col_factor(const TcDev& prm, int q) {
  float2 f;
  f.x = tc_vec(prm.col_scale, prm.col_scale_len, q);
  f.y = (prm.bias_dtype != LLG_DT_NONE && !prm.bias_on_p) ? tc_bias(prm, q) : 0.f;
  return f;
}

__device__ __forceinline__ void tc_put(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void tc_put(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void tc_put(float* p, float v) { *p = v; }

// 16 finished values of one accumulator row, stored transposed: element c goes to y[q_first + c][p] (the lanes of a
// warp hold consecutive p, so every store instruction writes one contiguous run).
template <typename T>
__device__ __forceinline__ void tc_emit_transposed(void* y, int64_t ldy, int p, int q_first, int nvalid, const float (&o)[16]) {
  T* const dst = static_cast<T*>(y) + (int64_t)q_first * ldy + p;
#pragma unroll
  for (int c = 0; c < 16; ++c)
    if (c < nvalid) tc_put(dst + (int64_t)c * ldy, o[c]);
}
__device__ __forceinline__ void tc_emit_transposed_any(void* y, int out_dtype, int64_t ldy, int p, int q_first, int nvalid,
                                                       const float (&o)[16]) {
  if (out_dtype == LLG_DT_BF16) tc_emit_transposed<__nv_bfloat16>(y, ldy, p, q_first, nvalid, o);
  else if (out_dtype == LLG_DT_F16) tc_emit_transposed<__half>(y, ldy, p, q_first, nvalid, o);
  else tc_emit_transposed<float>(y, ldy, p, q_first, nvalid, o);
}

// ---- exact widening of 8-bit / 4-bit floats to 16-bit pairs ---------------------------------------------------------

// four e4m3 bytes -> (k0,k1) and (k2,k3) as bf16x2 / f16x2
template <bool BF16>
__device__ __forceinline__ void widen_e4m3x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  if constexpr (BF16) {
    // byte s eeee mmm -> bf16 bits with the sign at 15 and exponent+mantissa at 4..10, which reads as the value times
    // 2^-120; the multiply by 2^120 is exact (also for e4m3 subnormals, which become bf16 subnormals). With the
    // byte b in the low bits of a 16-bit lane, b * 16 puts everything four bits up and (b & 0x80) * 240 moves the
    // sign from bit 11 to bit 15; multiplies run on another pipe than the logic operations.
    uint32_t a, b;
    asm("prmt.b32 %0, %1, 0, 0x4140;" : "=r"(a) : "r"(w));
    asm("prmt.b32 %0, %1, 0, 0x4342;" : "=r"(b) : "r"(w));
    const uint32_t ta = (a & 0x00800080u) * 240u + a * 16u, tb = (b & 0x00800080u) * 240u + b * 16u;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(ta), "r"(0x7b807b80u));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(tb), "r"(0x7b807b80u));
  } else {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((uint16_t)(w & 0xffffu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((uint16_t)(w >> 16)));
  }
}
// Eight e2m1 nibbles of one word (nibble i = K element i) -> four 16-bit pairs (k, k+1), times the block-scale pair.
//   f16:  the hardware conversion, then one exact multiply (<= 6 significant bits, magnitudes in [2^-10, 2688]).
//   bf16: nibble s e e m -> bf16 bits with the magnitude at 6..8, which reads as the value times 2^-126 (e = 0 lands
//         in the bf16 subnormals, matching e2m1's 0 / 0.5). The scale pair arrives multiplied by 2^118, so the one
//         multiply yields value * scale * 2^-8 exactly (>= 2^-18: never subnormal); the epilogue multiplies the
//         accumulator by 2^8, which is exact. The bit moves use a multiply (another pipe than the logic operations).
template <bool BF16>
__device__ __forceinline__ void widen_e2m1x8(uint32_t w, uint32_t scale2, uint32_t* o) {
  if constexpr (BF16) {
    const uint32_t lo = w & 0x0f0f0f0fu, hi = (w >> 4) & 0x0f0f0f0fu;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // bytes: [even nibble, 0, odd nibble, 0]; a selector with bit 3 set replicates the (clear) top bit of a byte
      uint32_t x;
      asm("prmt.b32 %0, %1, %2, %3;" : "=r"(x) : "r"(lo), "r"(hi), "r"((uint32_t)(j | 0x80 | ((4 + j) << 8) | 0x8000)));
      const uint32_t t = (x * 0x1040u) & 0x81c081c0u;  // magnitude << 6, sign << 12
      asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[j]) : "r"(t), "r"(scale2));
    }
  } else {
    uint32_t r0, r1, r2, r3;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
        : "r"(w));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(o[0]) : "r"(r0), "r"(scale2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(o[1]) : "r"(r1), "r"(scale2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(o[2]) : "r"(r2), "r"(scale2));
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(o[3]) : "r"(r3), "r"(scale2));
  }
}
// Four e4m3 block-scale bytes -> four replicated 16-bit pairs (s, s); for bf16 each carries the extra 2^118 (see above).
template <bool BF16>
__device__ __forceinline__ void widen_scales4(uint32_t sc4, uint32_t* s) {
  uint32_t p01, p23;
  widen_e4m3x4<BF16>(sc4, p01, p23);
  if constexpr (BF16) {
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p01) : "r"(p01), "r"(0x7a807a80u));  // 2^118: at most 448 * 2^118 < 2^127
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p23) : "r"(p23), "r"(0x7a807a80u));
  }
  s[0] = __byte_perm(p01, 0u, 0x1010);
  s[1] = __byte_perm(p01, 0u, 0x3232);
  s[2] = __byte_perm(p23, 0u, 0x1010);
  s[3] = __byte_perm(p23, 0u, 0x3232);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// W8A16: one thread's share of a stage: chunks [part * kChunks, +kChunks) of row r of every atom, 16 e4m3 bytes each,
// widened into 8 columns (2 K per column) of the thread's lane of tensor memory.
template <class G, int ATOMS, bool BF16>
__device__ __forceinline__ void w8_widen_stage(uint32_t st, uint32_t abuf, int r, int part) {
  constexpr int kChunks = 8 / G::kSubParts;
#pragma unroll
  for (int a = 0; a < ATOMS; ++a) {
    // all of the atom's shared-memory reads first, so that their latencies overlap instead of each sitting in front
    // of its own conversion (the loads and the tensor-memory stores are ordered instructions)
    uint4 raw[kChunks];
#pragma unroll
    for (int cc = 0; cc < kChunks; ++cc) {
      const int c = part * kChunks + cc;
      raw[cc] = lds128(st + G::kAOff + a * kAAtomTile + r * 128 + ((c ^ (r & 7)) << 4));
    }
#pragma unroll
    for (int cc = 0; cc < kChunks; ++cc) {
      const int c = part * kChunks + cc;
      uint32_t o[8];
      widen_e4m3x4<BF16>(raw[cc].x, o[0], o[1]);
      widen_e4m3x4<BF16>(raw[cc].y, o[2], o[3]);
      widen_e4m3x4<BF16>(raw[cc].z, o[4], o[5]);
      widen_e4m3x4<BF16>(raw[cc].w, o[6], o[7]);
      tmem_st8(abuf + a * G::kAColsAtom + c * 8, o);
    }
  }
}

// W4A16: one thread's share of a stage. Row r of every atom is 128 bytes = 8 chunks of 32 K elements; chunk c holds
// scale blocks 2c and 2c+1, i.e. bytes 2c and 2c+1 of the row's 16 scale bytes. The thread owns chunks
// [part * kChunks, +kChunks) and writes them, widened and scaled, to its lane of tensor memory (2 K per column).
template <class G, int ATOMS, bool BF16>
__device__ __forceinline__ void w4_widen_stage(uint32_t st, uint32_t abuf, int r, int part) {
  constexpr int kChunks = 8 / G::kSubParts;
  static_assert(kChunks % 2 == 0, "scales are fetched four at a time");
#pragma unroll
  for (int a = 0; a < ATOMS; ++a) {
    // the atom's shared-memory reads first (weights and scales), then the arithmetic: see w8_widen_stage
    uint4 raw[kChunks];
    uint32_t sc4[kChunks / 2];
#pragma unroll
    for (int cp = 0; cp < kChunks / 2; ++cp) {
      const int c0 = part * kChunks + 2 * cp;
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sc4[cp]) : "r"(st + G::kSfAOff + a * 2048 + r * 16 + 2 * c0));
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c0 + cc;
        raw[2 * cp + cc] = lds128(st + G::kAOff + a * kAAtomTile + r * 128 + ((c ^ (r & 7)) << 4));
      }
    }
#pragma unroll
    for (int cp = 0; cp < kChunks / 2; ++cp) {
      const int c0 = part * kChunks + 2 * cp;
      uint32_t sc[4];
      widen_scales4<BF16>(sc4[cp], sc);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c0 + cc;
        const uint4 rw = raw[2 * cp + cc];
        uint32_t o[8];
        widen_e2m1x8<BF16>(rw.x, sc[cc * 2], o);
        widen_e2m1x8<BF16>(rw.y, sc[cc * 2], o + 4);
        tmem_st8(abuf + a * G::kAColsAtom + c * 16, o);
        widen_e2m1x8<BF16>(rw.z, sc[cc * 2 + 1], o);
        widen_e2m1x8<BF16>(rw.w, sc[cc * 2 + 1], o + 4);
        tmem_st8(abuf + a * G::kAColsAtom + c * 16 + 8, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Work decomposition. An item is one (output tile, K partition). Without cluster split-K the kernel is persistent: the
// grid holds at most as many CTAs as fit on the GPU at once and CTA c works on items c, c + grid, c + 2*grid, ...;
// the TMA ring, the stage counters and (where tensor memory allows) two accumulator buffers carry across items, so
// the loads of the next item and the epilogue of the previous one overlap the MMAs of the current one. With cluster
// split-K every CTA owns exactly one item (tile = blockIdx.x, partition = rank in the cluster).

#ifdef LLG_TRACE
// Timeline probes for a diagnostic build only (never compiled into the shipped library).
extern __device__ unsigned long long g_trace[16384 * 8];
extern __device__ unsigned int g_trace_count;
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define LLG_STAMP(slot, k) do { if ((slot) < 16384u) g_trace[(slot) * 8 + (k)] = gtime(); } while (0)
#else
#define LLG_STAMP(slot, k) do { } while (0)
#endif

struct Item {
  int p0, q0, split, kt_beg, ntiles;
  unsigned tile;
};

template <int BQ, int ATOMS>
__device__ __forceinline__ Item decode_item(const TcDev& prm, int item) {
  const int tiles_p = (prm.P + prm.p_rows - 1) / prm.p_rows, tiles_q = (prm.Q + BQ - 1) / BQ;
  const int ntile = tiles_p * tiles_q;
  Item w;
  int tile;
  if (prm.cluster) {
    tile = blockIdx.x;
    w.split = blockIdx.z;
  } else {
    tile = item % ntile;
    w.split = item / ntile;
  }
  w.tile = (unsigned)tile;
  w.p0 = (tile % tiles_p) * prm.p_rows;
  w.q0 = (tile / tiles_p) * BQ;
  const int nk = (prm.k_atoms + ATOMS - 1) / ATOMS;
  w.kt_beg = (int)((int64_t)nk * w.split / prm.ksplit);
  w.ntiles = (int)((int64_t)nk * (w.split + 1) / prm.ksplit) - w.kt_beg;
  return w;
}

template <int FAM, int BQ, int ATOMS>
__global__ void __launch_bounds__(Geo<FAM, BQ, ATOMS>::kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmT, const TcDev prm) {
  using G = Geo<FAM, BQ, ATOMS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_base = smem_u32(smem_raw);
  const uint32_t base = (raw_base + 1023u) & ~1023u;
  SmemHeader* const hdr = reinterpret_cast<SmemHeader*>(smem_raw + (base - raw_base));
  const uint32_t stage0 = base + kHeaderBytes;
  volatile uint32_t* const abort_word = &hdr->abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ksplit = prm.ksplit;
  const int S = prm.stages;
  const int n_items = prm.n_items;
  const int item0 = prm.cluster ? 0 : (int)blockIdx.x;
  const int item_step = prm.cluster ? n_items : (int)gridDim.x;  // cluster mode: exactly one pass

#ifdef LLG_TRACE
  if (tid == 0) {
    hdr->trace_slot = atomicAdd(&g_trace_count, 1u);
    LLG_STAMP(hdr->trace_slot, 0);
    if (hdr->trace_slot < 16384u) g_trace[hdr->trace_slot * 8 + 7] = ((unsigned long long)gridDim.x << 32) | blockIdx.x;
  }
#endif
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), 1);
      mbar_init(smem_u32(&hdr->empty[s]), 1);
      mbar_init(smem_u32(&hdr->sf_full[s]), 128);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&hdr->acc_full[b]), 1);
      mbar_init(smem_u32(&hdr->acc_empty[b]), 128);
      mbar_init(smem_u32(&hdr->a_full[b]), G::kMixed ? G::kHelperThreads / G::kGroups : 128);
      mbar_init(smem_u32(&hdr->a_empty[b]), 1);
    }
    hdr->abort = 0u;
    hdr->prod_stage = 0u;
    hdr->last = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if ((FAM == FAM_W4A16 || G::kNvf4) && prm.sf_tma) tma_prefetch_desc(&tmS);
    if (G::kNvf4 && prm.sf_tma) tma_prefetch_desc(&tmT);
  }
  if (prm.pdl_early) pdl_trigger();
  uint32_t tmem = 0;
  if (warp == 0) {
    // the producer needs only the barriers it has just initialised: it announces them and starts streaming while
    // the other warps still set up tensor memory
    __syncwarp();
    asm volatile("bar.arrive 3, %0;" ::"r"(G::kThreads) : "memory");
  } else {
    if (warp == 1) {
      tmem_alloc(smem_u32(&hdr->tmem_base), G::kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    asm volatile("bar.sync 3, %0;" ::"r"(G::kThreads) : "memory");
    tc_fence_after();
    tmem = hdr->tmem_base;
  }

  constexpr uint32_t kABufCol = G::kAccBufs * G::kAccCols;  // mixed kinds: widened A buffers
  constexpr uint32_t kSfCol = G::kAccBufs * G::kAccCols;    // nvfp4: block-scale columns
  const bool a_first = prm.a_is_weight != 0;                // which operand may stream before the dependency wait

  if (warp == 0) {
    // ================================ TMA producer ================================
    // The whole warp walks the loop (addresses, counters and waits stay warp-uniform, so the compiler can keep them in
    // uniform registers); only the elected lane issues the copies.
    {
      const bool leader = elect_one();
      const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
      // an A box holds p_rows rows (<= 128): the rows of the 128-row MMA tile below it keep stale data and produce
      // accumulator rows nobody reads
      // block scales with 16-byte aligned rows: the 16 scale bytes per row and atom travel with the tile, as
      // [row][16 bytes] boxes (W4A16 reads them as they are, NVFP4's helpers reorder them for the MMA)
      const bool sf_tma = (FAM == FAM_W4A16 || G::kNvf4) && prm.sf_tma;
      const uint32_t tx_bytes = (uint32_t)(ATOMS * prm.p_rows * (sf_tma ? 144 : 128)) + (uint32_t)G::kBBytes +
                                (G::kNvf4 && sf_tma ? (uint32_t)(ATOMS * BQ * 16) : 0u);
      auto load_a = [&](const Item& w, int it, uint32_t g) {
        const uint32_t s = g % S, st = stage0 + s * G::kStageBytes, bar = smem_u32(&hdr->full[s]);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_2d(st + G::kAOff + a * kAAtomTile, &tmA, bar, ((w.kt_beg + it) * ATOMS + a) * kAtomBytes, w.p0,
                      a_first ? pol_w : pol_x);
          if constexpr (FAM == FAM_W4A16 || G::kNvf4) {
            if (sf_tma)
              tma_load_2d(st + G::kSfAOff + a * 2048, &tmS, bar, ((w.kt_beg + it) * ATOMS + a) * 16, w.p0,
                          a_first ? pol_w : pol_x);
          }
        }
      };
      auto load_b = [&](const Item& w, int it, uint32_t g) {
        const uint32_t s = g % S, st = stage0 + s * G::kStageBytes, bar = smem_u32(&hdr->full[s]);
#pragma unroll
        for (int a = 0; a < ATOMS * G::kBPerA; ++a)
          tma_load_2d(st + G::kBOff + a * G::kBAtomTile, &tmB, bar,
                      ((w.kt_beg + it) * ATOMS * G::kBPerA + a) * kAtomBytes, w.q0, a_first ? pol_x : pol_w);
        if constexpr (G::kNvf4) {
          if (sf_tma) {
#pragma unroll
            for (int a = 0; a < ATOMS; ++a)
              tma_load_2d(st + G::kSfBOff + a * 2048, &tmT, bar, ((w.kt_beg + it) * ATOMS + a) * 16, w.q0,
                          a_first ? pol_x : pol_w);
          }
        }
      };
      uint32_t g = 0;
      bool ok = true, first = true;
      for (int item = item0; item < n_items && ok; item += item_step) {
        const Item w = decode_item<BQ, ATOMS>(prm, item);
        int it = 0;
        if (first) {
          // the ring is empty: fill it with weight tiles before waiting for the previous kernel, then add the
          // activation tiles of the same stages
          const int npre = w.ntiles < S ? w.ntiles : S;
          if (leader) {
            for (int i = 0; i < npre; ++i) {
              mbar_expect_tx(smem_u32(&hdr->full[i]), tx_bytes);
              if (a_first) load_a(w, i, (uint32_t)i); else load_b(w, i, (uint32_t)i);
            }
          }
          LLG_STAMP(hdr->trace_slot, 1);
          pdl_wait();
          LLG_STAMP(hdr->trace_slot, 2);
          if (leader) {
            for (int i = 0; i < npre; ++i) {
              if (a_first) load_b(w, i, (uint32_t)i); else load_a(w, i, (uint32_t)i);
            }
          }
          it = npre;
          g = (uint32_t)npre;
          first = false;
          if (prm.pf_pace > 0 && leader) *reinterpret_cast<volatile uint32_t*>(&hdr->prod_stage) = (uint32_t)npre;
        }
        for (; it < w.ntiles; ++it, ++g) {
          const uint32_t s = g % S;
          if (g >= (uint32_t)S) {
            ok = mbar_wait(smem_u32(&hdr->empty[s]), ((g / S) & 1) ^ 1, abort_word);
            if (!ok) { give_up(prm, ST_PRODUCER_EMPTY_WAIT); break; }
          }
          if (leader) {
            mbar_expect_tx(smem_u32(&hdr->full[s]), tx_bytes);
            load_a(w, it, g);
            load_b(w, it, g);
            if (prm.pf_pace > 0 && item == item0) *reinterpret_cast<volatile uint32_t*>(&hdr->prod_stage) = (uint32_t)(it + 1);
          }
        }
      }
      if (first) pdl_wait();
      if (!ok) {
        // leave only after the copies already issued have landed (bounded): shared memory must not be written
        // after the CTA has gone
        for (int s = 0; s < S; ++s) {
          const long long t0 = clock64();
          while (!mbar_try(smem_u32(&hdr->full[s]), 0) && !mbar_try(smem_u32(&hdr->full[s]), 1) &&
                 clock64() - t0 < kWaitCycles / 16) {}
        }
      }
    }
    __syncwarp();
    if (!prm.pdl_early) pdl_trigger();
    l2_prefetch_share(prm.pf, prm.pf_bytes, blockIdx.x + (int64_t)gridDim.x * blockIdx.z, (int64_t)gridDim.x * gridDim.z,
                      lane, 32);
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    // Warp-uniform loop, one elected lane issues (always the same lane, so tcgen05.commit covers its MMAs).
    {
      const bool leader = elect_one();
      const uint32_t idesc = prm.idesc;
      // descriptors of stage 0; a stage or an atom further on only adds to the 14-bit address field (never overflows:
      // shared memory ends below 256 KB)
      const uint64_t adesc0 = umma_desc_sw128(stage0 + G::kAOff), bdesc0 = umma_desc_sw128(stage0 + G::kBOff);
      const uint64_t sfa0 = umma_desc_plain128(stage0 + G::kSfAOff), sfb0 = umma_desc_plain128(stage0 + G::kSfBOff);
      bool ok = true;
      uint32_t g = 0, n_acc = 0;
      for (int item = item0; item < n_items && ok; item += item_step) {
        const Item w = decode_item<BQ, ATOMS>(prm, item);
        if (w.ntiles <= 0) continue;
        const uint32_t ab = n_acc % G::kAccBufs, acc = tmem + ab * G::kAccCols;
        if (n_acc >= (uint32_t)G::kAccBufs) {  // the epilogue must have drained this buffer
          ok = mbar_wait(smem_u32(&hdr->acc_empty[ab]), ((n_acc / G::kAccBufs) & 1) ^ 1, abort_word);
          if (!ok) { give_up(prm, ST_MMA_FULL_WAIT); break; }
          tc_fence_after();
        }
        for (int it = 0; it < w.ntiles; ++it, ++g) {
          const uint32_t s = g % S, st = stage0 + s * G::kStageBytes;
          ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word);
          if constexpr (G::kNvf4) ok = ok && mbar_wait(smem_u32(&hdr->sf_full[s]), (g / S) & 1, abort_word);
          if constexpr (G::kMixed) ok = ok && mbar_wait(smem_u32(&hdr->a_full[g & 1]), (g >> 1) & 1, abort_word);
          if (!ok) { give_up(prm, ST_MMA_FULL_WAIT); break; }
          tc_fence_after();
#ifdef LLG_TRACE
          if (g == 0) LLG_STAMP(hdr->trace_slot, 3);
#endif
          if (leader) {
          if constexpr (G::kMixed) {
            const uint32_t abuf = tmem + kABufCol + (g & 1u) * ATOMS * G::kAColsAtom;
            constexpr int kMmaPerAtom = G::kAColsAtom / 8;  // K = 16 per MMA, 8 columns of widened A
#pragma unroll
            for (int a = 0; a < ATOMS; ++a)
#pragma unroll
              for (int j = 0; j < kMmaPerAtom; ++j) {
                const uint64_t bdesc = bdesc0 + (uint64_t)((s * G::kStageBytes + (a * G::kBPerA + j / 4) * G::kBAtomTile) >> 4) + (uint64_t)((j % 4) * 2);
                mma_ts_f16(acc, abuf + a * G::kAColsAtom + j * 8, bdesc, idesc, (it | a | j) != 0);
              }
            umma_commit(smem_u32(&hdr->a_empty[g & 1]));
          } else {
            const uint32_t sfc = tmem + kSfCol + (g & 1u) * G::kSfColsStage;
            if constexpr (G::kNvf4) {
              // every block-scale copy of the stage first (distinct columns), so the copies pipeline instead of each
              // pair sitting directly in front of the MMA that needs it
#pragma unroll
              for (int i = 0; i < ATOMS * 4; ++i) {
                const uint64_t sfo = (uint64_t)((s * G::kStageBytes + i * 512) >> 4);
                tmem_cp_32x128b_x4(sfc + (uint32_t)i * 8, sfa0 + sfo);
                tmem_cp_32x128b_x4(sfc + (uint32_t)i * 8 + 4, sfb0 + sfo);
              }
            }
#pragma unroll
            for (int a = 0; a < ATOMS; ++a) {
              const uint64_t adesc = adesc0 + (uint64_t)((s * G::kStageBytes + a * kAAtomTile) >> 4);
              const uint64_t bdesc = bdesc0 + (uint64_t)((s * G::kStageBytes + a * G::kBAtomTile) >> 4);
#pragma unroll
              for (int j = 0; j < 4; ++j) {  // 32 bytes of K per MMA for every kind
                const uint32_t acc_on = (it | a | j) != 0;
                if constexpr (FAM == FAM_F16) mma_ss_f16(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
                else if constexpr (FAM == FAM_F8) mma_ss_f8f6f4(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
                else if constexpr (FAM == FAM_I8) mma_ss_i8(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
                else {
                  const uint32_t sfa_t = sfc + (uint32_t)(a * 4 + j) * 8, sfb_t = sfa_t + 4;
                  mma_ss_nvf4(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on, sfa_t, sfb_t);
                }
              }
            }
          }
          umma_commit(smem_u32(&hdr->empty[s]));
          }
        }
        if (ok && leader) umma_commit(smem_u32(&hdr->acc_full[ab]));
        ++n_acc;
      }
    }
    __syncwarp();
    if (!prm.pdl_early) pdl_trigger();
  } else if (warp >= 6) {
    // ================================ helpers: block-scale feeder / weight converter ================================
    if constexpr (G::kHelpers) {
      const int ht = tid - 192;                // 0..kHelperThreads-1
      const int quarter = warp & 3;            // tensor-memory lanes this warp may touch: [32*quarter, +32)
      const int r = quarter * 32 + lane;       // row of the tile this thread works on
      const int group = ((warp - 6) >> 2) % G::kGroups;  // mixed kinds: stages g with g % 2 == group are this thread's
      const int part = ((warp - 6) >> 2) / G::kGroups;   // which share of the row's 16-byte chunks within the group
      const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
      bool ok = true;
      uint32_t g = 0;
      if (FAM == FAM_W4A16 && prm.sf_tma) {
        // ---- W4A16, scales delivered by TMA with the tile: widen each stage into tensor memory ----
        if constexpr (FAM == FAM_W4A16) {
          const bool bf16 = prm.bf16_act != 0;
          for (int item = item0; item < n_items && ok; item += item_step) {
            const Item w = decode_item<BQ, ATOMS>(prm, item);
            for (int it = 0; it < w.ntiles && ok; ++it, ++g) {
              if ((int)(g & 1u) != group) continue;
              const uint32_t s = g % S, st = stage0 + s * G::kStageBytes;
              ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word);
              if (ok && g >= 2) ok = mbar_wait(smem_u32(&hdr->a_empty[g & 1]), ((g >> 1) & 1) ^ 1, abort_word);
              if (!ok) { give_up(prm, ST_CONVERT_WAIT); break; }
              tc_fence_after();
              const uint32_t abuf = tmem + lane_addr + kABufCol + (g & 1u) * ATOMS * G::kAColsAtom;
              if (bf16) w4_widen_stage<G, ATOMS, true>(st, abuf, r, part);
              else w4_widen_stage<G, ATOMS, false>(st, abuf, r, part);
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(smem_u32(&hdr->a_full[g & 1]));
            }
          }
        }
      } else if (G::kNvf4 && prm.sf_tma) {
        // ---- NVFP4, scales delivered by TMA as [row][16 bytes]: reorder them in place into the layout the MMA's
        // scale copy reads - per MMA j a 512-byte block with row r at (r % 32) * 16 + (r / 32) * 4 ----
        if constexpr (G::kNvf4) {
          for (int item = item0; item < n_items && ok; item += item_step) {
            const Item w = decode_item<BQ, ATOMS>(prm, item);
            for (int it = 0; it < w.ntiles && ok; ++it, ++g) {
              const uint32_t s = g % S, st = stage0 + s * G::kStageBytes;
              ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word);
              if (!ok) give_up(prm, ST_CONVERT_WAIT);
              uint4 ra[ATOMS], rb[ATOMS];
#pragma unroll
              for (int a = 0; a < ATOMS; ++a) {
                ra[a] = lds128(st + G::kSfAOff + a * 2048 + r * 16);
                rb[a] = r < BQ ? lds128(st + G::kSfBOff + a * 2048 + r * 16) : make_uint4(0u, 0u, 0u, 0u);
              }
              // every row is read before any is overwritten; the barrier also makes the verdict of the wait common
              // to the 128 helper threads, so they leave the loop together
              {
                uint32_t all_ok;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 2, 128, p;\n\t"
                    "selp.u32 %0, 1, 0, q;\n\t}\n"
                    : "=r"(all_ok)
                    : "r"((uint32_t)ok)
                    : "memory");
                ok = all_ok != 0;
              }
              const uint32_t at = (uint32_t)((r & 31) * 16 + (r >> 5) * 4);
#pragma unroll
              for (int a = 0; a < ATOMS; ++a) {
                const uint32_t da = st + G::kSfAOff + a * 2048 + at, db = st + G::kSfBOff + a * 2048 + at;
                const uint32_t va[4] = {ra[a].x, ra[a].y, ra[a].z, ra[a].w}, vb[4] = {rb[a].x, rb[a].y, rb[a].z, rb[a].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  asm volatile("st.shared.u32 [%0], %1;" ::"r"(da + j * 512), "r"(va[j]) : "memory");
                  asm volatile("st.shared.u32 [%0], %1;" ::"r"(db + j * 512), "r"(vb[j]) : "memory");
                }
              }
              fence_async_shared();
              mbar_arrive(smem_u32(&hdr->sf_full[s]));
            }
          }
        }
      } else if constexpr (G::kNvf4 || FAM == FAM_W4A16) {
        // Block scales travel by 4-byte cp.async (their rows are only 4-byte aligned); each thread moves the 16 scale
        // bytes per atom of "its" row and keeps up to kSfLag stages in flight.
        pdl_wait();
        if constexpr (G::kNvf4) {
          // rows of the B scale blocks that no thread fills must not hold stale bytes
          for (int s = 0; s < S; ++s)
            for (int i = ht; i < G::kSfB / 4; i += 128)
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(stage0 + (uint32_t)s * G::kStageBytes + G::kSfBOff + i * 4), "r"(0u));
          asm volatile("bar.sync 2, 128;" ::: "memory");
        }
        // a slot is refilled only after the MMAs that read it have completed, and those need this thread's part of
        // the stage: the lag must stay below the ring depth
        const int lag = S - 1 < kSfLag ? S - 1 : kSfLag;
        const int sfk_total = prm.K >> 4;
        for (int item = item0; item < n_items && ok; item += item_step) {
          const Item w = decode_item<BQ, ATOMS>(prm, item);
          for (int it = 0; it < w.ntiles + lag && ok; ++it) {
            // W4A16: only the stages of this thread's group (an empty copy group keeps the count per iteration)
            if (it < w.ntiles && (!G::kMixed || (int)((g + (uint32_t)it) & 1u) == group)) {
              const uint32_t gi = g + (uint32_t)it, s = gi % S, st = stage0 + s * G::kStageBytes;
              if (gi >= (uint32_t)S) ok = mbar_wait(smem_u32(&hdr->empty[s]), ((gi / S) & 1) ^ 1, abort_word);
              if (!ok) { give_up(prm, ST_CONVERT_WAIT); break; }
#pragma unroll
              for (int a = 0; a < ATOMS; ++a) {
                const int sfk0 = ((w.kt_beg + it) * ATOMS + a) * 16;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int sfk = sfk0 + j * 4;
                  if (FAM == FAM_W4A16 && (j * G::kSubParts) / 4 != part) continue;  // another thread of this row owns the piece
                  {
                    const bool v = w.p0 + r < prm.P && sfk < sfk_total;
                    const unsigned char* src = v ? prm.a_sf + (int64_t)(w.p0 + r) * prm.lda_sf + sfk : prm.a_sf;
                    const uint32_t dst = G::kNvf4 ? st + G::kSfAOff + (a * 4 + j) * 512 + (r & 31) * 16 + (r >> 5) * 4
                                                  : st + G::kSfAOff + a * 2048 + r * 16 + j * 4;
                    cp_async4_zfill(dst, src, v);
                  }
                  if constexpr (G::kNvf4) {
                    if (r < BQ) {
                      const bool v = w.q0 + r < prm.Q && sfk < sfk_total;
                      const unsigned char* src = v ? prm.b_sf + (int64_t)(w.q0 + r) * prm.ldb_sf + sfk : prm.b_sf;
                      cp_async4_zfill(st + G::kSfBOff + (a * 4 + j) * 512 + (r & 31) * 16 + (r >> 5) * 4, src, v);
                    }
                  }
                }
              }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            const int done = it - lag;
            if (done < 0) continue;
            if (lag == 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
            else if (lag == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else asm volatile("cp.async.wait_group 1;" ::: "memory");
            const uint32_t gd = g + (uint32_t)done, s = gd % S;
            if (G::kMixed && (int)(gd & 1u) != group) continue;
            if constexpr (G::kNvf4) {
              fence_async_shared();
              mbar_arrive(smem_u32(&hdr->sf_full[s]));
            } else {
              // ---- W4A16: widen stage `done` (weight nibbles x block scale) into tensor memory ----
              const uint32_t st = stage0 + s * G::kStageBytes;
              const bool bf16 = prm.bf16_act != 0;
              ok = mbar_wait(smem_u32(&hdr->full[s]), (gd / S) & 1, abort_word);
              if (ok && gd >= 2) ok = mbar_wait(smem_u32(&hdr->a_empty[gd & 1]), ((gd >> 1) & 1) ^ 1, abort_word);
              if (!ok) { give_up(prm, ST_CONVERT_WAIT); break; }
              tc_fence_after();
              const uint32_t abuf = tmem + lane_addr + kABufCol + (gd & 1u) * ATOMS * G::kAColsAtom;
              if (bf16) w4_widen_stage<G, ATOMS, true>(st, abuf, r, part);
              else w4_widen_stage<G, ATOMS, false>(st, abuf, r, part);
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(smem_u32(&hdr->a_full[gd & 1]));
            }
          }
          g += (uint32_t)w.ntiles;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      } else {
        // ---- W8A16: widen each stage's weight bytes into tensor memory ----
        const bool bf16 = prm.bf16_act != 0;
        for (int item = item0; item < n_items && ok; item += item_step) {
          const Item w = decode_item<BQ, ATOMS>(prm, item);
          for (int it = 0; it < w.ntiles && ok; ++it, ++g) {
            if ((int)(g & 1u) != group) continue;
            const uint32_t s = g % S, st = stage0 + s * G::kStageBytes;
            ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word);
            if (ok && g >= 2) ok = mbar_wait(smem_u32(&hdr->a_empty[g & 1]), ((g >> 1) & 1) ^ 1, abort_word);
            if (!ok) { give_up(prm, ST_CONVERT_WAIT); break; }
            tc_fence_after();
            const uint32_t abuf = tmem + lane_addr + kABufCol + (g & 1u) * ATOMS * G::kAColsAtom;
            if (bf16) w8_widen_stage<G, ATOMS, true>(st, abuf, r, part);
            else w8_widen_stage<G, ATOMS, false>(st, abuf, r, part);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&hdr->a_full[g & 1]));
          }
        }
      }
    }
  } else {
    // ================================ epilogue (warps 2-5) ================================
    const int et = tid - 64;                 // 0..127
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t parked = stage0;          // cluster split-K: [BQ][128] 4-byte partials, q-major
    bool ok = true;
    uint32_t n_acc = 0;
    if (prm.pf_pace > 0 && warp == 2 && a_first && item0 < n_items) {
      // While the epilogue has nothing to do, one lane walks ahead of the producer and asks for the weight tiles of
      // the first item's later stages to be brought into L2, one stage per pf_pace cycles. A CTA that is resident
      // before the previous kernel has finished thus keeps the memory system busy through the hand-over, and its
      // producer later finds the tiles in L2. Every wait here is on the clock, so the loop is bounded.
      if (elect_one()) {
        const Item w = decode_item<BQ, ATOMS>(prm, item0);
        const long long t0 = clock64(), pace = prm.pf_pace;
        int k = S;
        while (k < w.ntiles) {
          const int prod = (int)*reinterpret_cast<volatile uint32_t*>(&hdr->prod_stage);
          if (prod + 1 >= w.ntiles) break;
          if (k <= prod + 1) k = prod + 2;  // the producer has caught up: stay a little ahead of it
          if (k >= w.ntiles || clock64() - t0 > kWaitCycles) break;
          // not further ahead of the producer than the L2 share this CTA may fill, and not faster than the pace
          if (k > (prod > S ? prod : S) + prm.pf_ahead || clock64() - t0 < (long long)(k - S + 1) * pace) {
            __nanosleep(64);
            continue;
          }
#pragma unroll
          for (int a = 0; a < ATOMS; ++a) {
            tma_prefetch_2d(&tmA, ((w.kt_beg + k) * ATOMS + a) * kAtomBytes, w.p0);
            if constexpr (FAM == FAM_W4A16 || G::kNvf4) {
              if (prm.sf_tma) tma_prefetch_2d(&tmS, ((w.kt_beg + k) * ATOMS + a) * 16, w.p0);
            }
          }
          ++k;
        }
      }
      __syncwarp();
    }
    pdl_wait();
    const float alpha = prm.alpha_ptr ? prm.alpha * __ldg(prm.alpha_ptr) : prm.alpha;
    for (int item = item0; item < n_items; item += item_step) {
      const Item w = decode_item<BQ, ATOMS>(prm, item);
      const uint32_t ab = n_acc % G::kAccBufs;
      bool have_acc = false;
      const int p = w.p0 + r;
      const int nq = min(BQ, prm.Q - w.q0);
      const int q0 = w.q0;
      // row-side epilogue operands are fetched while the MMAs still run
      const bool row_ok = p < prm.P && r < prm.p_rows;  // rows past the pitch belong to the next tile
      float rs = 1.f, bias_p = 0.f;
      if (ksplit == 1 && row_ok) {
        rs = tc_vec(prm.row_scale, prm.row_scale_len, p);
        if (prm.bias_dtype != LLG_DT_NONE && prm.bias_on_p) bias_p = tc_bias(prm, p);
      }
      // ... and so are the column-side factors of the first 16 columns (all of them for decode-sized tiles)
      const bool has_bias = prm.bias_dtype != LLG_DT_NONE, bias_on_p = prm.bias_on_p != 0;
      // Column factors. Tiles up to 64 columns wide: the epilogue threads fetch the whole tile's factors into shared
      // memory now (one column each) and every chunk reads them from there. Wider tiles: registers, one chunk ahead.
      float csn[16], cbn[16];
      float* const cs_s = hdr->colf[n_acc & 1u][0];
      float* const cb_s = hdr->colf[n_acc & 1u][1];
      if constexpr (BQ <= 64) {
        if (ksplit == 1) {
          if (et < BQ) {
            const float2 f = tc_col_factor(prm, q0 + et < prm.Q ? q0 + et : prm.Q - 1);
            cs_s[et] = f.x;
            cb_s[et] = f.y;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
        if (ksplit == 1 && row_ok) tc_col_factors(prm, q0, csn, cbn);
      }
      if (w.ntiles > 0) {
        if (ok) {
          ok = mbar_wait(smem_u32(&hdr->acc_full[ab]), (n_acc / G::kAccBufs) & 1, abort_word);
          if (!ok) give_up(prm, ST_EPILOGUE_WAIT);
        }
        tc_fence_after();
        have_acc = ok;
#ifdef LLG_TRACE
        if (et == 0) LLG_STAMP(hdr->trace_slot, 4);
#endif
      }
      for (int c0 = 0; c0 < BQ; c0 += 16) {
        if (c0 >= nq) break;
        uint32_t v[16];
        if (have_acc) {
          tmem_ld16(tmem + lane_addr + ab * G::kAccCols + c0, v);
          tmem_wait_ld();
          if constexpr (FAM == FAM_W4A16) {
            // bf16 activations: the widened weights carry a factor 2^-8 (see widen_e2m1x8); undone exactly here
            if (prm.bf16_act) {
#pragma unroll
              for (int c = 0; c < 16; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * 256.f);
            }
          }
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) v[c] = 0u;
        }
        if (ksplit == 1) {
          if (row_ok) {
            if constexpr (BQ <= 64) {
#pragma unroll
              for (int c = 0; c < 16; c += 4) {
                const float4 a = *reinterpret_cast<const float4*>(cs_s + c0 + c), b = *reinterpret_cast<const float4*>(cb_s + c0 + c);
                csn[c] = a.x; csn[c + 1] = a.y; csn[c + 2] = a.z; csn[c + 3] = a.w;
                cbn[c] = b.x; cbn[c + 1] = b.y; cbn[c + 2] = b.z; cbn[c + 3] = b.w;
              }
            }
            float o[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const float acc = G::kIntAcc ? (float)(int32_t)v[c] : __uint_as_float(v[c]);
              const float t = __fmul_rn(__fmul_rn(__fmul_rn(acc, alpha), rs), csn[c]);
              o[c] = has_bias ? __fadd_rn(t, bias_on_p ? bias_p : cbn[c]) : t;
            }
            // the next chunk's factors travel while this chunk is stored
            if constexpr (BQ > 64) {
              if (c0 + 16 < nq) tc_col_factors(prm, q0 + c0 + 16, csn, cbn);
            }
            const int nvalid = min(16, nq - c0);
            if (prm.swap) {
              if (prm.push_n == 0) {
                tc_emit_transposed_any(prm.y, prm.out_dtype, prm.ldy, p, q0 + c0, nvalid, o);
              } else {
                // push mode: to every rank's copy of this rank's partial (plain stores into peer-mapped memory)
#pragma unroll
                for (int d = 0; d < 8; ++d)
                  if (d < prm.push_n) tc_emit_transposed_any(prm.push_y[d], prm.out_dtype, prm.ldy, p, q0 + c0, nvalid, o);
              }
            } else {
              bool done = false;
              if (nvalid == 16 && prm.push_n == 0) {
                // 16 consecutive outputs of one row: vector stores when the run is 16-byte aligned
                if (prm.out_dtype == LLG_DT_F32) {
                  float* dst = static_cast<float*>(prm.y) + (int64_t)p * prm.ldy + q0 + c0;
                  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                    for (int c = 0; c < 16; c += 4)
                      *reinterpret_cast<float4*>(dst + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
                    done = true;
                  }
                } else {
                  uint16_t* dst = static_cast<uint16_t*>(prm.y) + (int64_t)p * prm.ldy + q0 + c0;
                  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    uint32_t w2[8];
#pragma unroll
                    for (int c = 0; c < 16; c += 2) {
                      if (prm.out_dtype == LLG_DT_BF16) {
                        const __nv_bfloat162 t = __halves2bfloat162(__float2bfloat16_rn(o[c]), __float2bfloat16_rn(o[c + 1]));
                        w2[c / 2] = *reinterpret_cast<const uint32_t*>(&t);
                      } else {
                        const __half2 t = __halves2half2(__float2half_rn(o[c]), __float2half_rn(o[c + 1]));
                        w2[c / 2] = *reinterpret_cast<const uint32_t*>(&t);
                      }
                    }
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w2[0], w2[1], w2[2], w2[3]);
                    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w2[4], w2[5], w2[6], w2[7]);
                    done = true;
                  }
                }
              }
              if (!done) {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                  if (c < nvalid) tc_store(prm, p, q0 + c0 + c, o[c]);
              }
            }
          }
        } else if (prm.cluster) {
#pragma unroll
          for (int c = 0; c < 16; ++c)
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(parked + (uint32_t)((c0 + c) * kBP + r) * 4u), "r"(v[c]) : "memory");
        } else {
          // partial plane in the output's own element order, so both this write and the later read are coalesced
          uint32_t* const ws = static_cast<uint32_t*>(prm.ws) + (int64_t)w.split * prm.P * prm.Q;
          if (p < prm.P) {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (c0 + c < nq) {
                const int q = q0 + c0 + c;
                ws[prm.swap ? (int64_t)q * prm.P + p : (int64_t)p * prm.Q + q] = v[c];
              }
          }
        }
      }
#ifdef LLG_TRACE
      if (et == 0) LLG_STAMP(hdr->trace_slot, 6);
#endif
      if (w.ntiles > 0) {
        // the accumulator buffer may be overwritten by the MMAs of a later item from here on
        tc_fence_before();
        mbar_arrive(smem_u32(&hdr->acc_empty[ab]));
        ++n_acc;
      }

      if (ksplit > 1 && !prm.cluster) {
        // Publish: the CTA barrier orders every thread's partial stores before thread 0's gpu-scope fence, which is
        // cumulative, so whoever observes the counter increment also observes the whole tile of partials.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          __threadfence();
          hdr->last = atomicAdd(&prm.counters[w.tile], 1u) == (unsigned)(ksplit - 1) ? 1u : 0u;
          __threadfence();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (hdr->last) {
          const int np = min(kBP, prm.P - w.p0);
          const int64_t plane = (int64_t)prm.P * prm.Q;
          const uint32_t* const ws = static_cast<const uint32_t*>(prm.ws);
          // four output elements per thread at a time, every partial of all four in flight before the first add
          for (int i0 = et; i0 < np * nq; i0 += 4 * 128) {
            uint32_t part[4][8];
            int pp[4], qq[4];
            const uint32_t* src[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = i0 + e * 128;
              const int ii = i < np * nq ? i : 0;
              const int pl = prm.swap ? ii % np : ii / nq, ql = prm.swap ? ii / np : ii % nq;
              pp[e] = w.p0 + pl;
              qq[e] = q0 + ql;
              src[e] = ws + (prm.swap ? (int64_t)qq[e] * prm.P + pp[e] : (int64_t)pp[e] * prm.Q + qq[e]);
            }
            uint32_t total[4] = {0u, 0u, 0u, 0u};
            for (int k0 = 0; k0 < ksplit; k0 += 8) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (k0 + j < ksplit) part[e][j] = __ldcg(src[e] + (int64_t)(k0 + j) * plane);
#pragma unroll
              for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  if (k0 + j < ksplit) {  // added in split order
                    if (k0 + j == 0) total[e] = part[e][j];
                    else if constexpr (G::kIntAcc) total[e] = (uint32_t)((int32_t)total[e] + (int32_t)part[e][j]);
                    else total[e] = __float_as_uint(__uint_as_float(total[e]) + __uint_as_float(part[e][j]));
                  }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (i0 + e * 128 < np * nq)
                tc_store(prm, pp[e], qq[e], tc_finish<G::kIntAcc>(prm, alpha, pp[e], qq[e], total[e]));
          }
          if (et == 0) prm.counters[w.tile] = 0u;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // hdr->last is rewritten by the next item
      }
    }
  }

  if (prm.cluster && ksplit > 1) {
    // every thread of every CTA of the cluster passes both barriers, whatever happened above
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && warp < 6) {
      const Item w = decode_item<BQ, ATOMS>(prm, 0);
      const int et = tid - 64;
      const float alpha = prm.alpha_ptr ? prm.alpha * __ldg(prm.alpha_ptr) : prm.alpha;
      const int np = min(kBP, prm.P - w.p0), nq = min(BQ, prm.Q - w.q0);
      const int total = kBP * nq, share = (total + ksplit - 1) / ksplit;
      const int lo = (int)cluster_ctarank() * share, hi = min(total, lo + share);
      const bool has_bias = prm.bias_dtype != LLG_DT_NONE;
      for (int i0 = lo + et; i0 < hi; i0 += 4 * 128) {
        // four elements per thread at a time: every partial and every epilogue factor of the batch is requested before
        // the first sum, so the distributed-shared-memory and global latencies overlap instead of adding up
        uint32_t part[4][8];
        float rs[4], cs[4], bv[4];
        int pp[4], qq[4];
        bool live[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + e * 128;
          const int pl = i % kBP, ql = i / kBP;
          live[e] = i < hi && pl < np;
          pp[e] = w.p0 + (live[e] ? pl : 0);
          qq[e] = w.q0 + (live[e] ? ql : 0);
          const uint32_t addr = stage0 + (uint32_t)(live[e] ? i : lo) * 4u;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (k < ksplit) part[e][k] = ld_cluster_u32(cluster_map_shared(addr, (uint32_t)k));
          rs[e] = tc_vec(prm.row_scale, prm.row_scale_len, pp[e]);
          cs[e] = tc_vec(prm.col_scale, prm.col_scale_len, qq[e]);
          bv[e] = has_bias ? tc_bias(prm, prm.bias_on_p ? pp[e] : qq[e]) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          uint32_t sum = part[e][0];
#pragma unroll
          for (int k = 1; k < 8; ++k)
            if (k < ksplit) {  // added in split order
              if constexpr (G::kIntAcc) sum = (uint32_t)((int32_t)sum + (int32_t)part[e][k]);
              else sum = __float_as_uint(__uint_as_float(sum) + __uint_as_float(part[e][k]));
            }
          const float acc = G::kIntAcc ? (float)(int32_t)sum : __uint_as_float(sum);
          const float t = __fmul_rn(__fmul_rn(__fmul_rn(acc, alpha), rs[e]), cs[e]);
          const float v = has_bias ? __fadd_rn(t, bv[e]) : t;
          if (live[e]) tc_store(prm, pp[e], qq[e], v);
        }
      }
    }
    cluster_arrive();  // partials stay readable until every CTA of the cluster is done with them
    cluster_wait();
  }

  tc_fence_before();
  __syncthreads();
#ifdef LLG_TRACE
  if (tid == 0) LLG_STAMP(hdr->trace_slot, 5);
#endif
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, G::kTmemCols);
  }
  if (prm.push_n > 0 && warp == 0) {
    // Every output store of this CTA precedes the barrier above. Lane 0 orders them device-wide (a cumulative fence
    // after the CTA barrier) and counts the CTA in; the CTA that completes the count has thereby observed every other
    // CTA's stores, resets the counter for the next launch, issues the ONE system-scope fence of the launch - cumulative
    // too, so it covers what the other CTAs stored - and tells each rank, once per token row, that this rank's partial
    // has arrived. (A system-scope fence in every CTA measured 9 us per GEMM of 256 CTAs.) Signals are one-way adds;
    // nothing here waits.
    unsigned last = 0u;
    if (lane == 0) {
      __threadfence();
      const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
      last = atomicAdd(prm.push_done, 1u) == ctas - 1u ? 1u : 0u;
      if (last) atomicExch(prm.push_done, 0u);
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      __threadfence_system();
      for (int i = lane; i < prm.push_rows * prm.push_n; i += 32) {
        const int row = i / prm.push_n, d = i - row * prm.push_n;
        atomicAdd_system(prm.push_flag[d] + (int64_t)row * prm.push_n + prm.push_rank, 1u);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host side

template <int FAM, int BQ, int ATOMS>
cudaError_t umma_launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& prm, bool pdl, cudaStream_t stream) {
  using G = Geo<FAM, BQ, ATOMS>;
  if constexpr (!G::kValid) {
    return cudaErrorInvalidConfiguration;
  } else {
    TcDev p = prm;
    const int cap = kSmemBudget / G::kStageBytes < LLG_MAX_STAGES ? kSmemBudget / G::kStageBytes : LLG_MAX_STAGES;
    p.stages = prm.stages < 2 ? 2 : (prm.stages > cap ? cap : prm.stages);
    size_t smem = 1024 + kHeaderBytes + (size_t)p.stages * G::kStageBytes;
    if (p.ksplit == 1) p.cluster = 0;
    if (p.cluster) {
      if (p.ksplit > 8) return cudaErrorInvalidConfiguration;
      const size_t need = 1024 + kHeaderBytes + (size_t)kBP * BQ * 4;
      if (need > 227 * 1024) return cudaErrorInvalidConfiguration;
      if (smem < need) smem = need;
    }
    static std::atomic<uint64_t> attr_done{0};  // one bit per device
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
      e = cudaFuncSetAttribute(umma_gemm_kernel<FAM, BQ, ATOMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
    }
    if (p.cluster || p.ksplit > 1 || p.p_rows < 8 || p.p_rows > kBP) p.p_rows = kBP;  // ragged rows only without split-K
    const int64_t tiles = (int64_t)((p.P + p.p_rows - 1) / p.p_rows) * ((p.Q + BQ - 1) / BQ);
    dim3 grid;
    if (p.cluster) {
      if (tiles > INT32_MAX) return cudaErrorInvalidValue;
      p.n_items = 1;
      p.pf_pace = 0;
      grid = dim3((unsigned)tiles, 1, p.ksplit);
      p.pdl_early = tiles * p.ksplit <= sm_count();
    } else {
      const int64_t items = tiles * p.ksplit;
      if (items > INT32_MAX) return cudaErrorInvalidValue;
      p.n_items = (int)items;
      // CTAs that fit on one SM at once: shared memory (228 KB per SM, 1 KB reserved per CTA) and tensor memory
      int occ = (int)((228 * 1024) / (smem + 1024));
      if (occ > 512 / G::kTmemCols) occ = 512 / G::kTmemCols;
      occ = occ < 1 ? 1 : occ > 4 ? 4 : occ;
      const int64_t resident = (int64_t)sm_count() * occ;
      grid = dim3((unsigned)(items < resident ? items : resident), 1, 1);
      p.pdl_early = 1;  // one wave by construction: let the next kernel's CTAs take the SMs as they free up
      // Self-prefetch pace (see the kernel's epilogue warps): one stage of weights per CTA every so many cycles that
      // all CTAs together ask for about what the memory delivers, kHbmBytesPerCycle (about 5 TB/s at 1.9 GHz; asking faster measured slower).
      // Only in a chain of dependent launches, with the weights on the streamed side and one item per CTA.
      // Only when everything beyond the ring fits the part of L2 that the running kernel's own stream can spare
      // (0.4 of it): a larger weight would be fetched half by request and half ahead, and that measured slower than
      // no prefetch at all.
      constexpr int64_t kHbmBytesPerCycle = 2600;
      const int64_t stage_w = (int64_t)ATOMS * 128 * p.p_rows, nk = (p.k_atoms + ATOMS - 1) / ATOMS;
      const int64_t ahead = nk > p.stages ? nk - p.stages : 0;
      const bool fits = ahead * stage_w * grid.x <= l2_bytes() * 2 / 5;
      p.pf_pace = (pdl && p.a_is_weight && p.ksplit == 1 && items <= resident && ahead > 0 && fits)
                      ? (int)(stage_w * grid.x / kHbmBytesPerCycle) : 0;
      p.pf_ahead = (int)ahead;
    }
    return launch_ex(umma_gemm_kernel<FAM, BQ, ATOMS>, grid, dim3(G::kThreads), smem, stream, pdl,
                     dim3(1, 1, p.cluster ? p.ksplit : 1), ta, tb, ts, tt, p);
  }
}

template <int FAM>
cudaError_t umma_launch_family(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl,
                               cudaStream_t s) {
  switch (cfg) {
    case 0: return umma_launch_one<FAM, 16, 1>(ta, tb, ts, tt, p, pdl, s);
    case 1: return umma_launch_one<FAM, 32, 1>(ta, tb, ts, tt, p, pdl, s);
    case 2: return umma_launch_one<FAM, 64, 1>(ta, tb, ts, tt, p, pdl, s);
    case 3: return umma_launch_one<FAM, 128, 1>(ta, tb, ts, tt, p, pdl, s);
    case 4: return umma_launch_one<FAM, 256, 1>(ta, tb, ts, tt, p, pdl, s);
    case 5: return umma_launch_one<FAM, 16, 2>(ta, tb, ts, tt, p, pdl, s);
    case 6: return umma_launch_one<FAM, 32, 2>(ta, tb, ts, tt, p, pdl, s);
    case 7: return umma_launch_one<FAM, 64, 2>(ta, tb, ts, tt, p, pdl, s);
    case 8: return umma_launch_one<FAM, 128, 2>(ta, tb, ts, tt, p, pdl, s);
    case 9: return umma_launch_one<FAM, 256, 2>(ta, tb, ts, tt, p, pdl, s);
    default: return cudaErrorInvalidValue;
  }
}

template <int FAM>
constexpr int umma_stage_bytes(int cfg) {
  switch (cfg) {
    case 0: return Geo<FAM, 16, 1>::kValid ? Geo<FAM, 16, 1>::kStageBytes : 0;
    case 1: return Geo<FAM, 32, 1>::kValid ? Geo<FAM, 32, 1>::kStageBytes : 0;
    case 2: return Geo<FAM, 64, 1>::kValid ? Geo<FAM, 64, 1>::kStageBytes : 0;
    case 3: return Geo<FAM, 128, 1>::kValid ? Geo<FAM, 128, 1>::kStageBytes : 0;
    case 4: return Geo<FAM, 256, 1>::kValid ? Geo<FAM, 256, 1>::kStageBytes : 0;
    case 5: return Geo<FAM, 16, 2>::kValid ? Geo<FAM, 16, 2>::kStageBytes : 0;
    case 6: return Geo<FAM, 32, 2>::kValid ? Geo<FAM, 32, 2>::kStageBytes : 0;
    case 7: return Geo<FAM, 64, 2>::kValid ? Geo<FAM, 64, 2>::kStageBytes : 0;
    case 8: return Geo<FAM, 128, 2>::kValid ? Geo<FAM, 128, 2>::kStageBytes : 0;
    case 9: return Geo<FAM, 256, 2>::kValid ? Geo<FAM, 256, 2>::kStageBytes : 0;
    default: return 0;
  }
}

}  // namespace llg
