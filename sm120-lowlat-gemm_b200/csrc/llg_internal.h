// Internal launch interfaces between the C-ABI layer (api.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/llg_core.h"

namespace llg {

// ---- status word ------------------------------------------------------------------------------------------------
// One word per device, set by a kernel whose bounded wait expired (first code wins). Codes:
enum : uint32_t {
  ST_OK = 0,
  ST_PRODUCER_EMPTY_WAIT = 1,  // TMA producer waited for a free pipeline slot
  ST_MMA_FULL_WAIT = 2,        // MMA issuer waited for operands
  ST_EPILOGUE_WAIT = 3,        // epilogue waited for the accumulator
  ST_CONVERT_WAIT = 4,         // converter / scale warps waited for a buffer
  ST_DRAIN_WAIT = 5,           // producer waited for its own copies while leaving early
  ST_SKINNY_PRODUCER_WAIT = 6, // skinny GEMV: producer waited for a free stage
  ST_SKINNY_CONVERT_WAIT = 7,  // skinny GEMV: activation converters waited for a stage to land
  ST_SKINNY_COMPUTE_WAIT = 8,  // skinny GEMV: compute warps waited for a full stage
  ST_ALLREDUCE_WAIT = 16,      // all-reduce: a peer's signal did not arrive
};
unsigned int* status_word_device_ptr();  // device address of the status word of the current device (cached)

// ---- process-wide switches / caches --------------------------------------------------------------------------
bool pdl_on();
int sm_count();
int64_t l2_bytes();  // L2 cache size of the current device

// Launch with optional PDL attribute and cluster shape.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             bool pdl, dim3 cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Tiled map over a row-major byte matrix seen as four-byte elements: box = box_bytes x box_rows, no swizzle (rows of a
// box are dense in shared memory), zero fill outside the tensor. row_bytes, ld_bytes and box_bytes are multiples of 16.
bool make_dense_map(CUtensorMap* m, const void* ptr, int64_t row_bytes, int64_t rows, int64_t ld_bytes, int box_bytes,
                    int box_rows, bool streamed);

// ---- skinny GEMV -------------------------------------------------------------------------------------------------
struct SkinnyDev {
  const void* x;
  const void* w;
  void* y;
  int64_t ldx, ldw, ldy;  // elements
  int M, N, K, ksplit;
  float* ws;
  unsigned* counters;
  int max_ranges;         // workspace split-K: counters available, one per row range (= gridDim.x)
  const void* pf;
  int64_t pf_bytes;
  unsigned* status;
  // geometry, filled in by the launcher
  int rounds;             // rounds of LPR vectors per pipeline stage
  int stages;             // ring depth
  int rows_pass;          // rows one pass over K covers
  int pitch;              // bytes between the rows of a weight stage
  int xraw_off;           // offset of the activation box inside a stage
  int xraw_pitch;         // bytes between its token rows
  int xslot_off;          // offset of the activations widened to fp32 inside a stage
  int stage_bytes;
  int w_box_bytes, x_box_bytes;  // bytes the two TMA boxes of a stage deliver
  unsigned char out_fp32, cluster;
};
// One translation unit per lanes-per-row. rows / unroll / warps are tile knobs that never change a result bit.
cudaError_t skinny_launch_l8(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s);
cudaError_t skinny_launch_l16(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s);
cudaError_t skinny_launch_l32(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s);

// ---- one-shot all-reduce over peer memory ------------------------------------------------------------------------
// Bound of every spin on a peer's signal, in clock cycles (about one second unless llg_set_wait_limit changed it).
long long ar_spin_cycles();
void set_ar_spin_cycles(long long cycles);
// Consumer of the pushed partials: recv holds `world` regions (index = source rank) of [rows, cols] 16-bit values.
cudaError_t reduce_local_launch(const void* recv, int64_t region_bytes, uint32_t* flags, void* out, const void* residual,
                                void* q, int64_t ldq, float* scale_out, int rows, int cols, int dtype, float min_scale,
                                int world, unsigned* status, cudaStream_t s);
cudaError_t allreduce_launch(const void* const* buffers, uint32_t* const* flags, void* out, int64_t vecs, int rank,
                             int world, int dtype, int ctas, unsigned* status, cudaStream_t s);
cudaError_t allreduce_quant_fp8_launch(const void* const* buffers, uint32_t* const* flags, void* out, void* q, int64_t ldq,
                                       float* scale_out, int rows, int cols, int dtype, float min_scale, int rank,
                                       int world, unsigned* status, cudaStream_t s);

// ---- quantizers --------------------------------------------------------------------------------------------------
struct GatedExtra {
  const void* up;  // non-null: the input row is silu(x) * up
  int64_t ldup;
  void* act;       // optional copy of the activation in the input type
  int64_t ldact;
};
cudaError_t quant_launch(const llg_quant_args& a, const GatedExtra& g, cudaStream_t s);

// ---- block-scale layouts (relayout.cu) ---------------------------------------------------------------------------
// Row-major [rows, cols] bytes (row pitch ld) <-> tiles of 128 rows x 4 columns, 512 bytes each, padded to whole tiles.
cudaError_t sf_relayout_launch(const void* src, void* dst, int rows, int cols, int64_t ld, bool to_tiled, cudaStream_t s);

// ---- tensor-core GEMM --------------------------------------------------------------------------------------------
// Kernel families (one template instantiation set each).
enum TcFamily : int { FAM_F16 = 0, FAM_F8 = 1, FAM_I8 = 2, FAM_NVF4 = 3, FAM_W8A16 = 4, FAM_W4A16 = 5, FAM_COUNT = 6 };

struct TcDev {
  // epilogue
  const float* row_scale;
  const float* col_scale;
  const void* bias;
  const float* alpha_ptr;
  void* y;
  int64_t ldy;
  float alpha;
  int row_scale_len, col_scale_len;
  int bias_dtype, out_dtype;
  // block scales (row-major [rows, K/16] bytes)
  const unsigned char* a_sf;
  const unsigned char* b_sf;
  int64_t lda_sf, ldb_sf;
  // problem
  int P, Q, K;          // K in elements
  int k_atoms;          // ceil(K bytes of the streamed (narrower) operand per row / 128)
  int ksplit, stages;
  int p_rows;           // rows of A one tile owns (128, or fewer to spread a few tiles over all SMs when ksplit == 1)
  int n_items;          // (tile, K partition) pairs a persistent grid walks; 1 per CTA in cluster mode
  uint32_t idesc;
  // split-K
  void* ws;
  unsigned* counters;
  // misc
  const void* pf;
  int64_t pf_bytes;
  unsigned* status;
  unsigned char swap, bias_on_p, cluster, pdl_early, a_is_weight, bf16_act;
  int pf_pace;          // > 0: self-prefetch of later weight stages into L2, one stage per pf_pace cycles
  int pf_ahead;         // ... at most this many stages ahead of the producer
  unsigned char sf_tma;  // W4A16 / NVFP4: block scales come by TMA (third and fourth tensor map), not per-thread copies
  // Push mode (row-parallel GEMM of a tensor-parallel layer): every finished output element is stored to push_y[d] for
  // each of the push_n ranks d instead of to y, and the last CTA of the grid to finish signals row slot r of every
  // rank: one add to push_flag[d][r * push_n + push_rank].
  int push_n, push_rank, push_rows;
  void* push_y[8];
  uint32_t* push_flag[8];
  unsigned* push_done;   // local counter of finished CTAs, zero between launches
};

struct TcTile {
  int bq;      // 16, 32, 64, 128, 256
  int atoms;   // 128-byte K atoms of the A operand per pipeline stage (1 or 2)
  int pair;    // 1: a 256 x bq tile computed by a pair of CTAs (tcgen05 cta_group::2); 0: 128 x bq on one CTA
};
TcTile tc_tile_of(int cfg);
int tc_family_of(int kind);
// bytes per stage of (family, cfg); 0 if invalid
int tc_stage_bytes_of(int kind, int cfg);
int tc_threads_of(int kind);  // 192; 320 with NVFP4's block-scale feeders; 448 with the mixed kinds' converter warps
constexpr int kSmemBudget = 227 * 1024 - 3072;  // dynamic shared memory for stages; the rest holds the header (barriers, epilogue factors) and alignment slack

// 256-row tiles on CTA pairs (umma_pair.cu): families F16, F8 and I8, bq 128 or 256, no split-K.
cudaError_t tc_launch_pair(int family, const CUtensorMap& ta, const CUtensorMap& tb, const TcDev& p, int bq, bool pdl, cudaStream_t s);
int tc_pair_stage_bytes(int family, int bq);  // 0 when the family has no pair kernel

// Defined per family in umma_<family>.cu.
cudaError_t tc_launch_f16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);
cudaError_t tc_launch_f8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);
cudaError_t tc_launch_i8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);
cudaError_t tc_launch_nvf4(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);
cudaError_t tc_launch_w8a16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);
cudaError_t tc_launch_w4a16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s);

}  // namespace llg
