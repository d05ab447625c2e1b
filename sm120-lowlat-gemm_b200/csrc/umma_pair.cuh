// Tensor-core GEMM on CTA pairs for large problems: C[p,q] = sum_k A[p,k] B[q,k], 256 x BQ output tiles.
//
// Two CTAs on neighbouring SMs (a cluster of two) compute one tile with tcgen05.mma.cta_group::2: CTA r of the pair
// holds rows [128 r, 128 r + 128) of the A tile and rows [BQ/2 r, BQ/2 (r+1)) of the B tile in its own shared memory
// and lanes 0..127 x BQ columns of the accumulator in its own tensor memory. Per output element each SM so fetches
// half of the B bytes a single-CTA 128 x BQ tile needs - at hundreds of tokens the limit is the L2 -> shared-memory
// traffic, not HBM and not the tensor pipe. No load uses multicast: every CTA brings its own operands by plain tiled
// TMA and has the bytes counted on the barrier of the CTA that issues the MMAs.
//
//   warp 0      TMA producer of its CTA
//   warp 1      allocates tensor memory (both CTAs); in the CTA of cluster rank 0 it issues the MMAs of the pair and the
//               commits that release a stage / publish an accumulator in BOTH CTAs (a barrier signal fanned out to the
//               pair; no data is multicast)
//   warps 2-5   epilogue of the CTA's 128 rows; two accumulator buffers, so a tile's epilogue overlaps the next
//               tile's MMAs
// Persistent: pair c walks tiles c, c + pairs, ... with the A-side index fastest, so the pairs running at one time
// share B tiles through L2. No split-K (K is never the scarce dimension here). Epilogue arithmetic and bounded waits
// are those of the single-CTA kernel. Large-tile counterpart of the reference's 256 x 128 and 128 x 128 configurations
// (csrc/tc_gemm.cuh:92-101).
#pragma once

#include "umma_gemm.cuh"

namespace llg {

template <int BQ>
struct PairGeo {
  static_assert(BQ == 128 || BQ == 256, "pair tiles are 256 x 128 or 256 x 256");
  static constexpr int kThreads = 192;
  static constexpr int kABytes = 128 * kAtomBytes;       // this CTA's rows of the A tile, one K atom
  static constexpr int kBBytes = (BQ / 2) * kAtomBytes;  // this CTA's half of the B tile
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTxBytes = 2u * kStageBytes;  // both CTAs report to one barrier
  static constexpr int kAccBufs = 2;
  static constexpr int kTmemCols = kAccBufs * BQ;
  // epilogue scratch behind the ring: per epilogue warp a 32 rows x 128 bytes transposition buffer, then the tile's
  // column-side factors (scale and bias as fp32) for two tiles in flight
  static constexpr int kOutBuf = 4 * 32 * 128;
  static constexpr int kColVec = 2 * 2 * BQ * 4;
  static constexpr int kEpiBytes = kOutBuf + kColVec;
};

struct PairHeader {
  uint64_t full[LLG_MAX_STAGES];   // rank 0's are used: the stage's bytes of both CTAs have landed
  uint64_t empty[LLG_MAX_STAGES];  // own: the MMAs that read this CTA's stage have completed
  uint64_t acc_full[2];            // own: every MMA of the tile in this accumulator buffer has completed
  uint64_t acc_empty[2];           // rank 0's are used: all 8 epilogue warps of the pair have read the buffer out
  uint32_t tmem_base;
  uint32_t abort;
};
static_assert(sizeof(PairHeader) <= kHeaderBytes, "header too large");

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// v = ((acc * alpha) * row_scale[p]) * col_scale[q] (+ bias), each operation rounded: the arithmetic of tc_finish_row
// with the column-side factors taken from the tile's vectors in shared memory.
template <bool INT_ACC>
__device__ __forceinline__ float pair_finish(float alpha, float rs, float bias_p, bool has_bias, bool bias_on_p, float cs,
                                             float cb, uint32_t bits) {
  const float acc = INT_ACC ? (float)(int32_t)bits : __uint_as_float(bits);
  float v = __fmul_rn(__fmul_rn(__fmul_rn(acc, alpha), rs), cs);
  if (has_bias) v = __fadd_rn(v, bias_on_p ? bias_p : cb);
  return v;
}

template <int FAM, int BQ>
__global__ void __launch_bounds__(PairGeo<BQ>::kThreads, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcDev prm) {
  using G = PairGeo<BQ>;
  constexpr bool kIntAcc = FAM == FAM_I8;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_base = smem_u32(smem_raw);
  const uint32_t base = (raw_base + 1023u) & ~1023u;  // the same offset in both CTAs: descriptors and commits rely on it
  PairHeader* const hdr = reinterpret_cast<PairHeader*>(smem_raw + (base - raw_base));
  const uint32_t stage0 = base + kHeaderBytes;
  volatile uint32_t* const abort_word = &hdr->abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs of the pair
  const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
  const int S = prm.stages, nk = prm.k_atoms;
  const int tiles_p = (prm.P + 255) / 256, ntile = prm.n_items;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&hdr->full[s]), 1);
      mbar_init(smem_u32(&hdr->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&hdr->acc_full[b]), 1);
      mbar_init(smem_u32(&hdr->acc_empty[b]), 8);
    }
    hdr->abort = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  pdl_trigger();  // one wave by construction
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(&hdr->tmem_base), G::kTmemCols);
    tmem_relinquish_pair();
  }
  // barriers initialised and tensor memory allocated in BOTH CTAs before either one signals the other
  tc_fence_before();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem = hdr->tmem_base;

  if (warp == 0) {
    // ================================ TMA producer (both CTAs) ================================
    pdl_wait();
    const bool issuer = elect_one();
    const uint32_t full_r0 = cluster_map_shared(smem_u32(&hdr->full[0]), 0);
    // the streamed side is the weight; it is read again (by the pairs on the other tile rows) only when the
    // activation side spans several tiles
    const bool a_w = prm.a_is_weight != 0;
    const int tiles_act = a_w ? (prm.Q + BQ - 1) / BQ : tiles_p;
    const uint64_t pol_w = tiles_act > 1 ? policy_evict_normal() : policy_evict_first(), pol_x = policy_evict_last();
    uint32_t g = 0;
    bool ok = true;
    for (int t = pair; t < ntile && ok; t += npairs) {
      const int p0 = (t % tiles_p) * 256 + (int)rank * 128, q0 = (t / tiles_p) * BQ + (int)rank * (BQ / 2);
      for (int it = 0; it < nk; ++it, ++g) {
        const uint32_t s = g % (uint32_t)S, st = stage0 + s * G::kStageBytes;
        if (g >= (uint32_t)S) {
          ok = mbar_wait(smem_u32(&hdr->empty[s]), ((g / S) & 1) ^ 1, abort_word);
          if (!ok) { give_up(prm, ST_PRODUCER_EMPTY_WAIT); break; }
        }
        if (issuer) {
          if (rank == 0) mbar_expect_tx(smem_u32(&hdr->full[s]), G::kTxBytes);
          tma_load_2d_pair(st, &tmA, full_r0 + s * 8u, it * kAtomBytes, p0, a_w ? pol_w : pol_x);
          tma_load_2d_pair(st + G::kABytes, &tmB, full_r0 + s * 8u, it * kAtomBytes, q0, a_w ? pol_x : pol_w);
        }
      }
    }
    if (!ok) {
      // copies already issued land within microseconds; stay resident for a bounded while so that none of them
      // writes shared memory of a CTA that has gone
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000ll) __nanosleep(256);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ================================ MMA issuer (rank 0 only) ================================
    if (rank == 0) {
      const bool issuer = elect_one();
      const uint32_t idesc = prm.idesc;
      const uint64_t adesc0 = umma_desc_sw128(stage0), bdesc0 = umma_desc_sw128(stage0 + G::kABytes);
      uint32_t g = 0, n_acc = 0;
      bool ok = true;
      for (int t = pair; t < ntile && ok; t += npairs) {
        const uint32_t ab = n_acc & 1u, acc = tmem + ab * BQ;
        if (n_acc >= 2u) {  // the epilogue warps of both CTAs must have drained this buffer
          ok = mbar_wait(smem_u32(&hdr->acc_empty[ab]), ((n_acc >> 1) & 1u) ^ 1u, abort_word);
          if (!ok) { give_up(prm, ST_MMA_FULL_WAIT); break; }
          tc_fence_after();
        }
        for (int it = 0; it < nk; ++it, ++g) {
          const uint32_t s = g % (uint32_t)S;
          ok = mbar_wait(smem_u32(&hdr->full[s]), (g / S) & 1, abort_word);
          if (!ok) { give_up(prm, ST_MMA_FULL_WAIT); break; }
          tc_fence_after();
          if (issuer) {
            const uint64_t adesc = adesc0 + (uint64_t)((s * G::kStageBytes) >> 4);
            const uint64_t bdesc = bdesc0 + (uint64_t)((s * G::kStageBytes) >> 4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 32 bytes of K per MMA
              const uint32_t acc_on = (it | j) != 0;
              if constexpr (FAM == FAM_F16) mma_pair_f16(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
              else if constexpr (FAM == FAM_F8) mma_pair_f8f6f4(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
              else mma_pair_i8(acc, adesc + 2 * j, bdesc + 2 * j, idesc, acc_on);
            }
            umma_commit_pair(smem_u32(&hdr->empty[s]), (uint16_t)3);
          }
        }
        if (ok && issuer) umma_commit_pair(smem_u32(&hdr->acc_full[ab]), (uint16_t)3);
        ++n_acc;
      }
    }
    __syncwarp();
  } else {
    // ================================ epilogue (both CTAs, 128 rows each) ================================
    // A thread owns one accumulator row (a tensor-memory lane). Storing its 16-column pieces straight to y would make
    // every store instruction touch 32 output rows; instead each warp turns 128 output bytes per row of its 32 rows
    // around in shared memory and writes them out as whole 128-byte lines, four rows per instruction. The transposed
    // (swap) orientation and outputs whose rows are not 16-byte aligned keep element stores.
    const int quarter = warp & 3;  // tensor-memory lanes this warp may read: [32 * quarter, +32)
    const int r = quarter * 32 + lane;
    const int et = tid - 64;       // 0..127 over the epilogue threads
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t acc_empty_r0 = cluster_map_shared(smem_u32(&hdr->acc_empty[0]), 0);
    const uint32_t obuf = stage0 + (uint32_t)S * G::kStageBytes + (uint32_t)quarter * 4096u;
    float* const colvec = reinterpret_cast<float*>(smem_raw + (stage0 - raw_base) + (size_t)S * G::kStageBytes + G::kOutBuf);
    pdl_wait();
    const float alpha = prm.alpha_ptr ? prm.alpha * __ldg(prm.alpha_ptr) : prm.alpha;
    const bool has_bias = prm.bias_dtype != LLG_DT_NONE, bias_on_p = prm.bias_on_p != 0;
    const int esz = prm.out_dtype == LLG_DT_F32 ? 4 : 2;
    const bool lines = !prm.swap && prm.push_n == 0 && (((uintptr_t)prm.y | (uintptr_t)(prm.ldy * esz)) & 15) == 0;
    uint32_t n_acc = 0;
    bool ok = true;
    for (int t = pair; t < ntile; t += npairs) {
      const uint32_t ab = n_acc & 1u;
      const int prow0 = (t % tiles_p) * 256 + (int)rank * 128, q0 = (t / tiles_p) * BQ;
      const int p = prow0 + r;
      const int nq = min(BQ, prm.Q - q0);
      const bool row_ok = p < prm.P;
      // column-side factors of the tile, fetched once per CTA while the MMAs still run
      float* const cs = colvec + ab * 2 * BQ;
      float* const cb = cs + BQ;
      for (int c = et; c < BQ; c += 128) {
        const int q = q0 + c < prm.Q ? q0 + c : prm.Q - 1;
        cs[c] = tc_vec(prm.col_scale, prm.col_scale_len, q);
        cb[c] = has_bias && !bias_on_p ? tc_bias(prm, q) : 0.f;
      }
      float rs = 1.f, bias_p = 0.f;
      if (row_ok) {
        rs = tc_vec(prm.row_scale, prm.row_scale_len, p);
        if (has_bias && bias_on_p) bias_p = tc_bias(prm, p);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the vectors are complete (the other buffer belongs to the previous tile)
      if (ok) {
        ok = mbar_wait(smem_u32(&hdr->acc_full[ab]), (n_acc >> 1) & 1u, abort_word);
        if (!ok) give_up(prm, ST_EPILOGUE_WAIT);
      }
      tc_fence_after();
      if (ok && lines) {
        const int blk = 128 / esz;  // columns per 128 output bytes: 64 (16-bit) or 32 (fp32)
        for (int b0 = 0; b0 < nq; b0 += blk) {
          uint32_t v[4][16];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j * 16 < blk && b0 + j * 16 < nq) tmem_ld16(tmem + lane_addr + ab * BQ + b0 + j * 16, v[j]);
          tmem_wait_ld();
          __syncwarp();  // the warp has read the previous block out of its buffer
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (j * 16 < blk && b0 + j * 16 < nq) {
              float o[16];
#pragma unroll
              for (int c = 0; c < 16; ++c)
                o[c] = pair_finish<kIntAcc>(alpha, rs, bias_p, has_bias, bias_on_p, cs[b0 + j * 16 + c], cb[b0 + j * 16 + c], v[j][c]);
              // 16-byte pieces of the row, XOR-swizzled by the row so that neither the writes (one row per lane) nor the
              // reads (eight lanes per row) collide on banks
              if (esz == 4) {
#pragma unroll
                for (int h = 0; h < 4; ++h)
                  sts128(obuf + lane * 128 + (((j * 4 + h) ^ (lane & 7)) << 4),
                         make_uint4(__float_as_uint(o[4 * h]), __float_as_uint(o[4 * h + 1]), __float_as_uint(o[4 * h + 2]),
                                    __float_as_uint(o[4 * h + 3])));
              } else {
                uint32_t w2[8];
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                  if (prm.out_dtype == LLG_DT_BF16) {
                    const __nv_bfloat162 h2 = __halves2bfloat162(__float2bfloat16_rn(o[c]), __float2bfloat16_rn(o[c + 1]));
                    w2[c / 2] = *reinterpret_cast<const uint32_t*>(&h2);
                  } else {
                    const __half2 h2 = __halves2half2(__float2half_rn(o[c]), __float2half_rn(o[c + 1]));
                    w2[c / 2] = *reinterpret_cast<const uint32_t*>(&h2);
                  }
                }
                sts128(obuf + lane * 128 + (((j * 2) ^ (lane & 7)) << 4), make_uint4(w2[0], w2[1], w2[2], w2[3]));
                sts128(obuf + lane * 128 + (((j * 2 + 1) ^ (lane & 7)) << 4), make_uint4(w2[4], w2[5], w2[6], w2[7]));
              }
            }
          }
          __syncwarp();
          const int piece = lane & 7, per = 16 / esz;  // this lane's 16-byte piece of a row; elements in it
          const int col = b0 + piece * per;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rl = i * 4 + (lane >> 3), pr = prow0 + quarter * 32 + rl;
            if (pr < prm.P && col < nq) {
              const uint4 d = lds128(obuf + rl * 128 + ((piece ^ (rl & 7)) << 4));
              unsigned char* const dst = static_cast<unsigned char*>(prm.y) + ((int64_t)pr * prm.ldy + q0 + col) * esz;
              if (col + per <= nq) {
                *reinterpret_cast<uint4*>(dst) = d;
              } else {  // the ragged right edge: element by element
                const uint32_t w4[4] = {d.x, d.y, d.z, d.w};
                for (int e = 0; col + e < nq; ++e) {
                  if (esz == 4) reinterpret_cast<uint32_t*>(dst)[e] = w4[e];
                  else reinterpret_cast<uint16_t*>(dst)[e] = (uint16_t)(w4[e >> 1] >> ((e & 1) * 16));
                }
              }
            }
          }
        }
      } else if (ok) {
        for (int c0 = 0; c0 < BQ; c0 += 16) {
          if (c0 >= nq) break;
          uint32_t v[16];
          tmem_ld16(tmem + lane_addr + ab * BQ + c0, v);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (c0 + c < nq)
                tc_store(prm, p, q0 + c0 + c,
                         pair_finish<kIntAcc>(alpha, rs, bias_p, has_bias, bias_on_p, cs[c0 + c], cb[c0 + c], v[c]));
          }
        }
      }
      // the buffer may be overwritten by the MMAs of a later tile from here on
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_r0 + ab * 8u);
      ++n_acc;
    }
  }

  // Nobody leaves while the other CTA may still signal its barriers, read its shared memory or write its tensor memory.
  tc_fence_before();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem, G::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// host side

template <int FAM, int BQ>
cudaError_t pair_launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const TcDev& prm, bool pdl, cudaStream_t stream) {
  using G = PairGeo<BQ>;
  TcDev p = prm;
  constexpr int kRing = (kSmemBudget - G::kEpiBytes) / G::kStageBytes;
  const int cap = kRing < LLG_MAX_STAGES ? kRing : LLG_MAX_STAGES;
  p.stages = prm.stages < 2 ? 2 : (prm.stages > cap ? cap : prm.stages);
  // at least half of an SM's shared memory, so that an SM never holds two CTAs of one launch (the second would sit in
  // its tensor-memory allocation until the first has walked all its tiles)
  size_t smem = 1024 + kHeaderBytes + (size_t)p.stages * G::kStageBytes + G::kEpiBytes;
  if (smem < 116 * 1024) smem = 116 * 1024;
  static std::atomic<uint64_t> attr_done{0};  // one bit per device
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !((attr_done.load(std::memory_order_acquire) >> dev) & 1ull)) {
    e = cudaFuncSetAttribute(umma_pair_kernel<FAM, BQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_done.fetch_or(1ull << dev, std::memory_order_release);
  }
  const int64_t tiles = (int64_t)((p.P + 255) / 256) * ((p.Q + BQ - 1) / BQ);
  if (tiles > INT32_MAX) return cudaErrorInvalidValue;
  p.n_items = (int)tiles;
  p.ksplit = 1;
  p.cluster = 0;
  // One wave of pairs: as many clusters of two as the device can hold at once with this much shared memory (asked of
  // the runtime once per device and ring depth; a pair needs two SMs of one TPC, so it may be fewer than SMs / 2).
  static std::atomic<int> slots_of[64][LLG_MAX_STAGES + 1] = {};
  int slots = (dev >= 0 && dev < 64) ? slots_of[dev][p.stages].load(std::memory_order_acquire) : 0;
  if (slots <= 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)(sm_count() > 1 ? sm_count() / 2 : 1), 1, 1);
    cfg.blockDim = dim3(G::kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, umma_pair_kernel<FAM, BQ>, &cfg);
    if (e != cudaSuccess) return e;
    slots = n > 0 ? n : 1;
    if (slots > sm_count() / 2 && sm_count() >= 2) slots = sm_count() / 2;
    if (dev >= 0 && dev < 64) slots_of[dev][p.stages].store(slots, std::memory_order_release);
  }
  const unsigned pairs = (unsigned)(tiles < slots ? tiles : slots);
  return launch_ex(umma_pair_kernel<FAM, BQ>, dim3(2 * pairs, 1, 1), dim3(G::kThreads), smem, stream, pdl, dim3(2, 1, 1), ta, tb, p);
}

template <int FAM>
cudaError_t pair_launch_family(const CUtensorMap& ta, const CUtensorMap& tb, const TcDev& p, int bq, bool pdl, cudaStream_t s) {
  switch (bq) {
    case 128: return pair_launch_one<FAM, 128>(ta, tb, p, pdl, s);
    case 256: return pair_launch_one<FAM, 256>(ta, tb, p, pdl, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace llg
