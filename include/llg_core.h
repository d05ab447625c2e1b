/* libllg_core: C ABI of the B200 (sm_100a) low-latency GEMM core.
 *
 * Plain pointers, sizes and strides only - no torch types. Every pointer is a DEVICE pointer unless a comment
 * says otherwise. The caller owns all buffers; the library allocates nothing, keeps no pointer after a call
 * returns, and launches on the CUDA stream it is given (a cudaStream_t passed as void*; NULL = default stream) on
 * the device that is current in the calling thread. Launch descriptors (including TMA tensor maps) are passed to
 * the kernels by value, so calls are legal during CUDA-graph capture.
 *
 * Return value of the int functions: 0 on success, a negative LLG_E_* code on failure; llg_last_error() then
 * returns a message prefixed "lowlat_gemm: " (thread-local, valid until the next failing call of that thread).
 *
 * Each entry point states which interface of the reference (Cerynitius/sm120-lowlat-gemm) it stands in for.
 */
#ifndef LLG_CORE_H_
#define LLG_CORE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLG_ABI_VERSION 2

#if defined(__GNUC__)
#define LLG_API __attribute__((visibility("default")))
#else
#define LLG_API
#endif

enum {
  LLG_OK = 0,
  LLG_E_INVALID = -1,   /* argument validation failed (reference: TORCH_CHECK in csrc/ops.cpp) */
  LLG_E_CONFIG = -2,    /* tile config cannot be launched for this kind (reference: csrc/ops.cpp:294-298) */
  LLG_E_CUDA = -3,      /* a CUDA runtime / driver call failed */
  LLG_E_UNAVAILABLE = -4 /* the library was built without this kernel */
};

/* Precision kinds; ids equal the reference's enum TcKind (csrc/tc_params.h:10-21) and KINDS table
 * (lowlat_gemm/__init__.py:64-74). */
enum {
  LLG_KIND_BF16 = 0,
  LLG_KIND_F16 = 1,
  LLG_KIND_FP8 = 2,
  LLG_KIND_INT8 = 3,
  LLG_KIND_NVFP4 = 4,
  LLG_KIND_W8A16_BF16 = 5,
  LLG_KIND_W8A16_F16 = 6,
  LLG_KIND_W4A16_BF16 = 7,
  LLG_KIND_W4A16_F16 = 8,
  LLG_KIND_COUNT = 9
};

/* Element types of 16/32-bit tensors; values equal the reference's enum DType (csrc/tc_params.h:23). */
enum { LLG_DT_NONE = 0, LLG_DT_BF16 = 1, LLG_DT_F16 = 2, LLG_DT_F32 = 3 };

/* Quantizer modes; values equal the reference's enum QuantMode (csrc/quant.h:9-14). */
enum { LLG_QUANT_FP8_STATIC = 0, LLG_QUANT_FP8_PER_TOKEN = 1, LLG_QUANT_INT8_PER_TOKEN = 2, LLG_QUANT_NVFP4 = 3 };

#define LLG_NUM_CFGS 12
#define LLG_MAX_STAGES 16
#define LLG_SKINNY_MAX_TOKENS 16

/* ---------------------------------------------------------------------------------------------------------------
 * Skinny streaming GEMV: y[M,N] = x[M,K] @ w[N,K]^T for bf16/f16 with M <= 16, fp32 accumulation in an order that
 * depends on (K, lanes_per_row, ksplit) only, so a row of the result is bit-identical for every M and tile.
 * Stands in for torch.ops.lowlat_gemm.skinny_out (reference csrc/ops.cpp:59-129, 381-385; launch descriptor
 * csrc/params.h:10-34; kernel csrc/gemv.cuh:74-234, whose summation order csrc/gemv.cuh:6-12 is kept bit for bit).
 * The kernel is a persistent one-wave grid: each CTA owns a contiguous range of rows. rows / unroll / warps are tile
 * knobs with the reference's ranges; here they set the row groups a warp carries (rows), the K depth of a pipeline
 * stage (unroll) and the compute warps per CTA (2 * warps). */
typedef struct llg_skinny_args {
  const void* x;  int64_t ldx;   /* [M,K], row stride in elements, 16-byte aligned, ldx % 8 == 0 */
  const void* w;  int64_t ldw;   /* [N,K], same element type as x */
  void* y;        int64_t ldy;   /* [M,N], element type of x, or fp32 when out_fp32 */
  int32_t M, N, K;               /* 1 <= M <= 16, K % 8 == 0 */
  int32_t f16;                   /* 0: bf16, 1: f16 */
  int32_t out_fp32;
  int32_t rows, unroll, lanes_per_row, warps, ksplit; /* tile: (rows,unroll) in {(1,2),(1,4),(1,8),(2,2),(2,4),(4,2)} */
  int32_t cluster;               /* split-K reduced through cluster shared memory (ksplit <= 8) */
  float* ws;      int64_t ws_elems;        /* split-K partials, >= ksplit*M*N floats (workspace mode) */
  int32_t* counters; int64_t counters_elems; /* workspace mode: one per row range, zero between launches; at least 1,
                                                llg_skinny_ranges(N, ksplit) for full speed */
  const void* prefetch; int64_t prefetch_bytes; /* optional L2 prefetch range (16-byte aligned), NULL = none */
} llg_skinny_args;

LLG_API int llg_skinny(const llg_skinny_args* args, void* stream);

/* Row ranges (= CTAs along N, = split-K counters) llg_skinny uses on the current device for this N and ksplit when
 * enough counters are passed. No counterpart in the reference, whose grid follows from the tile. */
LLG_API int32_t llg_skinny_ranges(int32_t N, int32_t ksplit);

/* ---------------------------------------------------------------------------------------------------------------
 * Tensor-core GEMM (tcgen05): C[p,q] = sum_k A[p,k] B[q,k], then
 *   v = ((acc * alpha * (*alpha_ptr)) * row_scale[p]) * col_scale[q]   (fp32, each product rounded)
 *   v = v + bias[p or q]                                               (rounded add, no fused multiply-add)
 * stored as y[q,p] when swap else y[p,q]. INT8 accumulates in int32 (exact) and converts once.
 * Stands in for torch.ops.lowlat_gemm.tc_gemm (reference csrc/ops.cpp:201-300, 393-401; descriptor
 * csrc/tc_params.h:28-60; kernel csrc/tc_gemm.cuh:179-501).
 * Tile configs: 0-4 = 128 x {16,32,64,128,256} with one 128-byte K atom per pipeline stage, 5-9 = the same with two;
 * 10, 11 = 256 x {128,256} computed by a pair of CTAs (the large tiles, reference csrc/tc_gemm.cuh:92-101): bf16, f16,
 * fp8 and int8 only, ksplit must be 1. */
typedef struct llg_tc_args {
  int32_t kind;                  /* LLG_KIND_* */
  int32_t cfg, stages, ksplit;   /* tile config [0, LLG_NUM_CFGS), pipeline depth (clamped), K partitions [1,64] */
  int32_t cluster;               /* split-K through cluster shared memory (ksplit <= 8) instead of the workspace */
  int32_t swap;                  /* y stored transposed: A is the weight */
  const void* a;  int64_t a_rows, a_row_bytes, lda_bytes;  /* A [P, K] as bytes, rows 16-byte aligned */
  const void* b;  int64_t b_rows, b_row_bytes, ldb_bytes;  /* B [Q, K] */
  const void* a_sf; int64_t lda_sf;  /* block scales of A: [P, K/16] e4m3 bytes, row stride % 4 == 0 (NVFP4, W4A16) */
  const void* b_sf; int64_t ldb_sf;  /* block scales of B (NVFP4) */
  const float* row_scale; int32_t row_scale_len;  /* 0 none, 1 scalar, else P */
  const float* col_scale; int32_t col_scale_len;  /* 0 none, 1 scalar, else Q */
  const void* bias; int32_t bias_dtype; int32_t bias_on_p;  /* LLG_DT_*; indexed by p or by q */
  const float* alpha_ptr; float alpha;
  void* y; int64_t ldy; int32_t out_dtype;        /* row stride in elements; LLG_DT_* */
  void* ws; int64_t ws_elems;                     /* split-K partials (4-byte), >= ksplit*P*Q */
  int32_t* counters; int64_t counters_elems;      /* >= number of output tiles, zero between launches */
  const void* prefetch; int64_t prefetch_bytes;
} llg_tc_args;

LLG_API int llg_tc_gemm(const llg_tc_args* args, void* stream);

/* (BP, BQ, threads, shared bytes per pipeline stage) of a tile config; stands in for
 * torch.ops.lowlat_gemm.tc_info (reference csrc/ops.cpp:412-416, csrc/tc_info.cu:8-61). Returns 0 or LLG_E_INVALID. */
LLG_API int llg_tc_info(int32_t kind, int32_t cfg, int32_t out[4]);

/* Dynamic shared memory a CTA may use for pipeline stages on this build (bytes); the Python planner divides it by
 * the stage size where the reference hard-codes 99 KB (lowlat_gemm/__init__.py:208, csrc/tc_gemm.cuh:141). */
LLG_API int32_t llg_smem_budget(void);

/* ---------------------------------------------------------------------------------------------------------------
 * Activation quantizers, one call per [M,K] matrix. Stands in for torch.ops.lowlat_gemm.quant (reference
 * csrc/ops.cpp:305-367; descriptor csrc/quant.h:16-29; kernels csrc/quant.cu:43-114). Bit-exact with them. */
typedef struct llg_quant_args {
  int32_t mode;          /* LLG_QUANT_* */
  int32_t in_dtype;      /* LLG_DT_BF16 / F16 / F32 */
  const void* x; int64_t ldx;   /* [M,K], row stride in elements */
  void* q; int64_t ldq;         /* [M,K] bytes, or [M,K/2] packed fp4 (low nibble = even element); stride in bytes */
  void* sf_out; int64_t ldsf;   /* nvfp4: [M,K/16] e4m3 bytes */
  const float* scale_in;        /* fp8 static: the scale; nvfp4: the global scale g (1 float, device) */
  float* scale_out;             /* per-token modes: [M] */
  float min_scale;
  int32_t M, K;
} llg_quant_args;

LLG_API int llg_quant(const llg_quant_args* args, void* stream);

/* Gated activation fused with the quantizer: per row act = round_to_input_type(silu(gate) * up) (fp32 arithmetic, one
 * rounding - the tensor a separate SiLU-and-multiply kernel would have stored), then the quantizer of q.mode on act
 * (LLG_QUANT_FP8_PER_TOKEN, LLG_QUANT_NVFP4) or no quantizer at all (LLG_QUANT_NONE: only `act` is written). q.x is the
 * gate, `up` the other half; `act` (optional unless mode is NONE) receives the activation in the input type. The step
 * on the input side of the down projection (reference: the "act" stand-ins of tools/decode_step.py:27-40, which it
 * leaves to the framework); it removes two elementwise launches per decode layer. */
#define LLG_QUANT_NONE 4
typedef struct llg_gated_quant_args {
  llg_quant_args q;
  const void* up; int64_t ldup;     /* [M,K], row stride in elements */
  void* act; int64_t ldact;         /* [M,K] in the input type, or NULL */
} llg_gated_quant_args;

LLG_API int llg_gated_quant(const llg_gated_quant_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Process-wide programmatic-dependent-launch switch; stands in for torch.ops.lowlat_gemm.set_pdl / pdl_enabled
 * (reference csrc/ops.cpp:409-410, csrc/tc_info.cu:67-70). */
LLG_API void llg_set_pdl(int32_t on);
LLG_API int32_t llg_pdl_enabled(void);

/* Load-time conversion of a block-scale matrix (one e4m3 byte per 16 K elements) between the row-major form the
 * entry points above take - [rows, cols] bytes, row pitch ld - and the tiled form of checkpoints prepared for
 * block-scaled tensor-core GEMMs: tiles of 128 rows x 4 columns, 512 contiguous bytes each, byte (r, c) of a tile at
 * (r % 32) * 16 + (r / 32) * 4 + c, row-tile major, rows and columns padded to whole tiles (padding written as zero).
 * to_tiled = 0 reads the tiled buffer `src` and writes row-major `dst`; 1 the other way. The tiled buffer holds
 * ceil(rows / 128) * ceil(cols / 4) * 512 bytes and must be 16-byte aligned. The reference takes row-major scales only
 * (lowlat_gemm/__init__.py:10-16) and has no converter. */
LLG_API int llg_sf_relayout(const void* src, void* dst, int32_t rows, int32_t cols, int64_t ld, int32_t to_tiled, void* stream);

/* Host-buffer convenience used for end-to-end timing: copies x (HOST, pinned or pageable) to x_dev, runs the GEMM
 * described by `args` (whose activation operand must already point at x_dev), copies y back to y_host, all on
 * `stream`, without synchronising. No counterpart in the reference (its callers hold device tensors). */
LLG_API int llg_tc_gemm_host(const llg_tc_args* args, const void* x_host, void* x_dev, int64_t x_bytes, void* y_host,
                     int64_t y_bytes, void* stream);

/* Reads and clears the device status word of the current device (synchronises the device). 0 = no kernel ever gave
 * up a bounded wait; otherwise the code of the first wait that expired. No counterpart in the reference. */
LLG_API int llg_device_status(uint32_t* status);

/* ---------------------------------------------------------------------------------------------------------------
 * One-shot all-reduce (sum) of a small tensor across the GPUs of one node over peer-mapped ("symmetric") buffers;
 * the low-latency replacement for an NCCL all_reduce at the row-parallel boundaries of a tensor-parallel decode
 * layer. buffers_dev / flags_dev are DEVICE arrays of `world` device pointers (index = rank) to every rank's data
 * buffer and flag words; each rank must have written its partial into buffers_dev[rank] on `stream` (or before)
 * and must use a different data buffer for consecutive calls (two alternating buffers are enough). The flag words
 * (2 * LLG_AR_MAX_CTAS * world uint32 per rank: arrival counters that the peers add to, then this rank's count of
 * consumed signals) must be zero before the first call and belong to the library afterwards: counters only grow, so a
 * captured launch replays, provided every rank issues the same sequence of all-reduce calls. Partials
 * are added in rank order in fp32, so all ranks get identical bits. bytes must be a multiple of 16, buffers 16-byte
 * aligned, world <= 8, 1 <= ctas <= LLG_AR_MAX_CTAS. Waits are bounded (~1 s): on expiry the device status word
 * is set (llg_device_status) and the result is undefined, but nothing hangs.
 * No counterpart in the reference (it has no multi-GPU code). */
#define LLG_AR_MAX_CTAS 64
LLG_API int llg_allreduce_oneshot(const void* const* buffers_dev, uint32_t* const* flags_dev, void* out, int64_t bytes,
                                  int32_t dtype, int32_t rank, int32_t world, int32_t ctas, void* stream);

/* The same all-reduce followed, in the same kernel, by the per-token FP8 activation quantizer
 * (lowlat_gemm/__init__.py:quantize_fp8, csrc/quant.cu:43-66 of the reference): the partials are [rows, cols] 16-bit
 * values, contiguous, at the start of every rank's buffer; one CTA and one flag set per row, so rows <= LLG_AR_MAX_CTAS
 * (same flag words as above); cols a multiple of 8, at most LLG_ARQ_MAX_COLS. Writes
 * q [rows, ldq] (e4m3 bytes) and scale_out [rows] = max(amax / 448, min_scale), bit-identical to quantize_fp8 applied
 * to the all-reduce's 16-bit result, and that result itself to `out` unless out is NULL. Same buffer alternation,
 * flag and bounded-wait rules as llg_allreduce_oneshot. No counterpart in the reference. */
#define LLG_ARQ_MAX_COLS 16384
LLG_API int llg_allreduce_quant_fp8(const void* const* buffers_dev, uint32_t* const* flags_dev, void* out, void* q,
                                    int64_t ldq, float* scale_out, int32_t rows, int32_t cols, int32_t dtype,
                                    float min_scale, int32_t rank, int32_t world, void* stream);

/* Row-parallel GEMM of a tensor-parallel layer with the all-reduce's transfer inside its epilogue ("push"): every
 * finished output element is stored, with plain stores into peer-mapped memory, to dst[d] for every rank d - the place
 * where rank d collects this rank's partial, laid out like y - instead of to args->y (which is ignored), so the bytes
 * cross NVLink while the remaining tiles are still being computed. When the whole grid has finished, its last CTA adds 1
 * to flags[d][row * world + rank] for every rank d and token row: the same arrival counters llg_allreduce_oneshot uses,
 * sent one way. The consumer on every rank is llg_reduce_local. `done` is a zero-initialised counter local to this
 * rank that the kernel returns to zero. rows = the GEMM's token count (<= LLG_AR_MAX_CTAS); world <= 8. Consecutive
 * pushes must alternate between two destination buffers, as with llg_allreduce_oneshot. No multicast, no TMA on peer
 * memory. No counterpart in the reference (it has no multi-GPU code); nearest analogue: the row-parallel projections
 * in the op sequence of tools/decode_step.py:27-40, followed by the framework's all-reduce. */
typedef struct llg_push_args {
  int32_t world, rank, rows, reserved;
  void* dst[8];
  uint32_t* flags[8];
  uint32_t* done;
} llg_push_args;

LLG_API int llg_tc_gemm_push(const llg_tc_args* args, const llg_push_args* push, void* stream);

/* Consumer of pushed partials, one CTA per token row: waits (bounded) until all `world` ranks have signalled the row,
 * adds the local copies recv + src * region_bytes in rank order in fp32 and rounds to the 16-bit type - bit for bit the
 * result of llg_allreduce_oneshot - then optionally adds `residual` (fp32 add, one rounding), stores the row to `out`
 * (may be NULL when q is given) and, when q is given, quantizes it per token to FP8 exactly as llg_quant does
 * (scale_out[rows], q [rows, ldq]). `flags` are THIS rank's flag words. No counterpart in the reference. */
LLG_API int llg_reduce_local(const void* recv, int64_t region_bytes, uint32_t* flags, void* out, const void* residual,
                             void* q, int64_t ldq, float* scale_out, int32_t rows, int32_t cols, int32_t dtype,
                             float min_scale, int32_t world, void* stream);

/* Bound, in GPU clock cycles, of every wait for a peer's signal in the all-reduce kernels (default about one second;
 * cycles <= 0 restores it). Process-wide, read at launch. Meant for failure tests and for deployments that want a
 * stalled peer reported sooner; after an expired wait llg_device_status() returns 16. No counterpart in the reference. */
LLG_API void llg_set_wait_limit(int64_t cycles);

/* Split-K tensor-core GEMM for callers that must not allocate device memory. Same arguments and result as
 * llg_tc_gemm, except that args->ws / args->counters are ignored: partial sums and arrival counters live in a fixed
 * scratch array inside the library (LLG_STATIC_WS_ELEMS 4-byte partials + LLG_STATIC_COUNTERS counters, about 4 MB,
 * held by every GPU that loads the library until the process exits). Meant for hosts that own all device memory
 * themselves - an inference server that carved the GPU into its own pools at start-up, a plugin sandbox or a
 * real-time loop where cudaMalloc is forbidden because it synchronises the device and may fail late - and so cannot
 * hand this library a workspace tensor. The call itself performs no cudaMalloc / cudaFree and calls no allocating
 * library routine.
 *   - A problem needing more than the fixed scratch (ksplit * P * Q partials, one counter per output tile) is
 *     rejected with LLG_E_INVALID and a message that names both numbers.
 *   - The first call on each device looks up the scratch address (one cudaGetSymbolAddress with that device current);
 *     make that first call outside any stream capture.
 *   - Every call on a device shares the one array: the counters the launch needs are cleared on the stream before the
 *     kernel, the partials are fully rewritten before they are read, and two calls that overlap on the GPU (different
 *     streams) race with each other - keep calls that use it on one stream.
 * This entry point has no counterpart in the reference, whose callers always pass workspace tensors. */
#define LLG_STATIC_WS_ELEMS (1 << 20)
#define LLG_STATIC_COUNTERS 4096
LLG_API int llg_tc_gemm_static_ws(const llg_tc_args* args, void* stream);

/* sizeof of llg_skinny_args, llg_tc_args, llg_quant_args, llg_gated_quant_args, llg_push_args as this library was
 * compiled: lets a foreign-function binding verify its struct layout before the first call. No counterpart in the
 * reference. */
LLG_API void llg_struct_sizes(int32_t out[5]);

LLG_API const char* llg_last_error(void);
LLG_API int32_t llg_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LLG_CORE_H_ */
