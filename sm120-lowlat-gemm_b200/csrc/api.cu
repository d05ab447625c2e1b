// C ABI of libllg_core (declared in include/llg_core.h): argument validation, TMA tensor maps, kernel dispatch.
//
// Validation rules and messages follow the reference's binding layer csrc/ops.cpp (skinny_run 59-129,
// tc_gemm_impl 201-300, quant_impl 305-367); checks that need tensor metadata (device, dtype object, contiguity)
// are done by the Python wrapper, everything that can be decided from pointers, sizes and strides is decided here.
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "llg_internal.h"

namespace llg {

int tc_stage_bytes_f16(int cfg);
int tc_stage_bytes_f8(int cfg);
int tc_stage_bytes_i8(int cfg);
int tc_stage_bytes_nvf4(int cfg);
int tc_stage_bytes_w8a16(int cfg);
int tc_stage_bytes_w4a16(int cfg);

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  int n = snprintf(g_err, sizeof(g_err), "lowlat_gemm: ");
  vsnprintf(g_err + n, sizeof(g_err) - n, fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(const char* what, cudaError_t e) {
  return fail(LLG_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool aligned(const void* p, uintptr_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

std::atomic<bool> g_pdl{false};

__device__ unsigned int g_status_word = 0;

// Fixed split-K scratch of llg_tc_gemm_static_ws: partials first, arrival counters behind them. In host code this
// name is only a handle for cudaGetSymbolAddress, never a device address.
constexpr size_t kStaticWsBytes = (size_t)LLG_STATIC_WS_ELEMS * 4, kStaticCntBytes = (size_t)LLG_STATIC_COUNTERS * 4;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticWsBytes + kStaticCntBytes];

struct KindSpec {
  int a_bits, b_bits;
  bool a_sf, b_sf;
  int k_align;
};

bool kind_spec(int kind, KindSpec* k) {
  switch (kind) {
    case LLG_KIND_BF16:
    case LLG_KIND_F16: *k = {16, 16, false, false, 8}; return true;
    case LLG_KIND_FP8:
    case LLG_KIND_INT8: *k = {8, 8, false, false, 16}; return true;
    case LLG_KIND_NVFP4: *k = {4, 4, true, true, 64}; return true;
    case LLG_KIND_W8A16_BF16:
    case LLG_KIND_W8A16_F16: *k = {8, 16, false, false, 16}; return true;
    case LLG_KIND_W4A16_BF16:
    case LLG_KIND_W4A16_F16: *k = {4, 16, true, false, 64}; return true;
    default: return false;
  }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// Byte-typed 2-D map over a row-major matrix: dim0 = bytes of one row, dim1 = rows; box = 128 bytes x box_rows with the
// 128-byte swizzle the MMA descriptors expect; out-of-range parts of a box read as zero.
bool make_map(CUtensorMap* m, const void* ptr, int64_t row_bytes, int64_t rows, int64_t ld_bytes, int box_rows,
              bool streamed) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        streamed ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Byte map over a block-scale matrix (one e4m3 byte per 16 K elements): box = 16 bytes x box_rows, no swizzle, so a
// box lands as [row][16 bytes]. Needs a 16-byte aligned base and row pitch.
bool make_sf_map(CUtensorMap* m, const void* ptr, int64_t row_bytes, int64_t rows, int64_t ld_bytes, int box_rows) {
  auto fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {16u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

bool make_dense_map(CUtensorMap* m, const void* ptr, int64_t row_bytes, int64_t rows, int64_t ld_bytes, int box_bytes,
                    int box_rows, bool streamed) {
  auto fn = encode_fn();
  if (!fn || box_bytes % 16 || box_bytes > 1024 || box_rows < 1 || box_rows > 256) return false;
  cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 4), (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 4), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        streamed ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool pdl_on() { return g_pdl.load(std::memory_order_relaxed); }

// Per-device facts, looked up once per device. Concurrent first use from several threads is harmless: every thread
// computes the same value and the slots are atomics.
static int cached_attr(std::atomic<int>* slots, cudaDeviceAttr attr) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int v = slots[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    cudaDeviceGetAttribute(&v, attr, dev);
    slots[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

int sm_count() {
  static std::atomic<int> counts[64];
  return cached_attr(counts, cudaDevAttrMultiProcessorCount);
}

int64_t l2_bytes() {
  static std::atomic<int> sizes[64];
  return cached_attr(sizes, cudaDevAttrL2CacheSize);
}

unsigned int* status_word_device_ptr() {
  static std::atomic<unsigned int*> ptrs[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  unsigned int* ptr = ptrs[dev].load(std::memory_order_acquire);
  if (!ptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptr = static_cast<unsigned int*>(p);
    ptrs[dev].store(ptr, std::memory_order_release);
  }
  return ptr;
}

TcTile tc_tile_of(int cfg) {
  static const int bq[5] = {16, 32, 64, 128, 256};
  if (cfg < 0 || cfg >= LLG_NUM_CFGS) return {0, 0, 0};
  if (cfg >= 10) return {cfg == 10 ? 128 : 256, 1, 1};  // 256-row tiles on CTA pairs
  return {bq[cfg % 5], 1 + cfg / 5, 0};
}

int tc_family_of(int kind) {
  switch (kind) {
    case LLG_KIND_BF16:
    case LLG_KIND_F16: return FAM_F16;
    case LLG_KIND_FP8: return FAM_F8;
    case LLG_KIND_INT8: return FAM_I8;
    case LLG_KIND_NVFP4: return FAM_NVF4;
    case LLG_KIND_W8A16_BF16:
    case LLG_KIND_W8A16_F16: return FAM_W8A16;
    case LLG_KIND_W4A16_BF16:
    case LLG_KIND_W4A16_F16: return FAM_W4A16;
    default: return -1;
  }
}

int tc_threads_of(int kind) {
  const int f = tc_family_of(kind);
  return f == FAM_W4A16 ? 192 + 256 : f == FAM_W8A16 ? 192 + 256 : f == FAM_NVF4 ? 320 : 192;
}

int tc_stage_bytes_of(int kind, int cfg) {
  const TcTile t = tc_tile_of(cfg);
  if (t.pair) return tc_pair_stage_bytes(tc_family_of(kind), t.bq);
  switch (tc_family_of(kind)) {
    case FAM_F16: return tc_stage_bytes_f16(cfg);
    case FAM_F8: return tc_stage_bytes_f8(cfg);
    case FAM_I8: return tc_stage_bytes_i8(cfg);
    case FAM_NVF4: return tc_stage_bytes_nvf4(cfg);
    case FAM_W8A16: return tc_stage_bytes_w8a16(cfg);
    case FAM_W4A16: return tc_stage_bytes_w4a16(cfg);
    default: return 0;
  }
}

#ifdef LLG_TRACE
__device__ unsigned long long g_trace[16384 * 8];
__device__ unsigned int g_trace_count = 0;
#endif

}  // namespace llg

using namespace llg;

#ifdef LLG_TRACE
extern "C" __attribute__((visibility("default"))) int llg_trace_dump(unsigned long long* host, unsigned int* count) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(count, llg::g_trace_count, sizeof(unsigned int));
  cudaMemcpyFromSymbol(host, llg::g_trace, sizeof(unsigned long long) * 16384 * 8);
  const unsigned int zero = 0;
  cudaMemcpyToSymbol(llg::g_trace_count, &zero, sizeof(zero));
  return 0;
}
#endif

extern "C" {

const char* llg_last_error(void) { return g_err; }
int32_t llg_abi_version(void) { return LLG_ABI_VERSION; }
void llg_set_pdl(int32_t on) { g_pdl.store(on != 0, std::memory_order_relaxed); }
int32_t llg_pdl_enabled(void) { return g_pdl.load(std::memory_order_relaxed) ? 1 : 0; }
int32_t llg_smem_budget(void) { return kSmemBudget; }
void llg_struct_sizes(int32_t out[5]) {
  out[0] = (int32_t)sizeof(llg_skinny_args);
  out[1] = (int32_t)sizeof(llg_tc_args);
  out[2] = (int32_t)sizeof(llg_quant_args);
  out[3] = (int32_t)sizeof(llg_gated_quant_args);
  out[4] = (int32_t)sizeof(llg_push_args);
}
void llg_set_wait_limit(int64_t cycles) { set_ar_spin_cycles(cycles > 0 ? cycles : 2000000000ll); }

int llg_device_status(uint32_t* status) {
  unsigned int* dptr = status_word_device_ptr();
  if (!dptr) return fail(LLG_E_CUDA, "no device status word");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail("device synchronize", e);
  unsigned int v = 0;
  e = cudaMemcpy(&v, dptr, sizeof(v), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail("status read", e);
  if (v != 0) {
    const unsigned int zero = 0;
    cudaMemcpy(dptr, &zero, sizeof(zero), cudaMemcpyHostToDevice);
  }
  if (status) *status = v;
  return LLG_OK;
}

int llg_tc_info(int32_t kind, int32_t cfg, int32_t out[4]) {
  const TcTile t = tc_tile_of(cfg);
  if (t.bq == 0 || tc_family_of(kind) < 0) return fail(LLG_E_INVALID, "unknown kind %d or cfg %d", kind, cfg);
  out[0] = t.pair ? 256 : 128;
  out[1] = t.bq;
  out[2] = t.pair ? 192 : tc_threads_of(kind);
  out[3] = tc_stage_bytes_of(kind, cfg);
  return LLG_OK;
}

// ---------------------------------------------------------------------------------------------------------------

int32_t llg_skinny_ranges(int32_t N, int32_t ksplit) {
  if (N < 1 || ksplit < 1) return 0;
  int64_t gx = 2 * (int64_t)sm_count() / ksplit;  // small CTAs run two to an SM
  if (gx < 1) gx = 1;
  return (int32_t)(gx < N ? gx : N);
}

int llg_skinny(const llg_skinny_args* a, void* stream) {
  if (!a) return fail(LLG_E_INVALID, "null arguments");
  const int ru = a->rows * 16 + a->unroll;
  if (!(ru == 0x12 || ru == 0x14 || ru == 0x18 || ru == 0x22 || ru == 0x24 || ru == 0x42))
    return fail(LLG_E_INVALID, "unsupported (rows, unroll) = (%d, %d); supported: (1,2) (1,4) (1,8) (2,2) (2,4) (4,2)",
                a->rows, a->unroll);
  if (!(a->lanes_per_row == 8 || a->lanes_per_row == 16 || a->lanes_per_row == 32))
    return fail(LLG_E_INVALID, "lanes_per_row must be 8, 16 or 32, got %d", a->lanes_per_row);
  if (a->warps < 1 || a->warps > 8) return fail(LLG_E_INVALID, "warps must be in [1, 8], got %d", a->warps);
  if (a->ksplit < 1 || a->ksplit > 64) return fail(LLG_E_INVALID, "ksplit must be in [1, 64], got %d", a->ksplit);
  if (!a->x || !a->w || !a->y) return fail(LLG_E_INVALID, "x, w, y must be device pointers");
  if (a->M < 1 || a->M > LLG_SKINNY_MAX_TOKENS) return fail(LLG_E_INVALID, "skinny: M must be in [1, 16], got %d", a->M);
  if (a->K <= 0 || a->K % 8) return fail(LLG_E_INVALID, "skinny: K must be a positive multiple of 8, got %d", a->K);
  if (a->N < 1) return fail(LLG_E_INVALID, "N or K too large");
  if (a->ldx % 8 || a->ldw % 8) return fail(LLG_E_INVALID, "x and w row strides must be multiples of 8 elements");
  if (!aligned(a->x, 16) || !aligned(a->w, 16)) return fail(LLG_E_INVALID, "x and w must be 16-byte aligned");
  const bool cluster = a->cluster && a->ksplit > 1;
  if (cluster && a->ksplit > 8) return fail(LLG_E_INVALID, "cluster split-K supports ksplit <= 8, got %d", a->ksplit);
  const bool use_ws = a->ksplit > 1 && !cluster;
  if (use_ws) {
    if (!a->ws || !a->counters) return fail(LLG_E_INVALID, "workspace must be contiguous float32, counters contiguous int32");
    if (a->ws_elems < (int64_t)a->ksplit * a->M * a->N)
      return fail(LLG_E_INVALID, "workspace has %lld floats, needs %lld", (long long)a->ws_elems,
                  (long long)a->ksplit * a->M * a->N);
    // one counter per row range; with fewer counters than llg_skinny_ranges() the launch uses fewer, longer ranges
    if (a->counters_elems < 1) return fail(LLG_E_INVALID, "counters has %lld, needs at least 1", (long long)a->counters_elems);
  }
  if (a->prefetch && !aligned(a->prefetch, 16))
    return fail(LLG_E_INVALID, "prefetch tensor must be contiguous and 16-byte aligned");

  SkinnyDev p{};
  p.x = a->x; p.w = a->w; p.y = a->y;
  p.ldx = a->ldx; p.ldw = a->ldw; p.ldy = a->ldy;
  p.M = a->M; p.N = a->N; p.K = a->K; p.ksplit = a->ksplit;
  p.ws = use_ws ? a->ws : nullptr;
  p.counters = use_ws ? reinterpret_cast<unsigned*>(a->counters) : nullptr;
  p.max_ranges = use_ws ? (int)(a->counters_elems < INT32_MAX ? a->counters_elems : INT32_MAX) : INT32_MAX;
  p.pf = a->prefetch; p.pf_bytes = a->prefetch ? a->prefetch_bytes : 0;
  p.out_fp32 = a->out_fp32 != 0;
  p.cluster = cluster;
  p.status = status_word_device_ptr();
  if (!p.status) return fail(LLG_E_CUDA, "no device status word");
  const bool pdl = pdl_on();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  switch (a->lanes_per_row) {
    case 8: e = skinny_launch_l8(p, a->rows, a->unroll, a->warps, a->f16 != 0, pdl, s); break;
    case 16: e = skinny_launch_l16(p, a->rows, a->unroll, a->warps, a->f16 != 0, pdl, s); break;
    default: e = skinny_launch_l32(p, a->rows, a->unroll, a->warps, a->f16 != 0, pdl, s); break;
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorInvalidConfiguration ? LLG_E_CONFIG : LLG_E_CUDA,
                "skinny: cannot launch M=%d N=%d K=%d rows=%d unroll=%d warps=%d (%s)", a->M, a->N, a->K, a->rows, a->unroll,
                a->warps, cudaGetErrorString(e));
  }
  return LLG_OK;
}

// ---------------------------------------------------------------------------------------------------------------

static int check_operand(const void* ptr, int64_t ld_bytes, const char* name) {
  if (!ptr) return fail(LLG_E_INVALID, "operands must be on CUDA");
  if (ld_bytes % 16) return fail(LLG_E_INVALID, "%s row stride must be a multiple of 16 bytes", name);
  if (!aligned(ptr, 16)) return fail(LLG_E_INVALID, "%s must be 16-byte aligned", name);
  return 0;
}

// validate_only: every check of the call, no tensor map, no launch
static int tc_gemm_run(const llg_tc_args* a, const llg_push_args* push, void* stream, bool validate_only = false) {
  if (!a) return fail(LLG_E_INVALID, "null arguments");
  KindSpec ks;
  if (!kind_spec(a->kind, &ks)) return fail(LLG_E_INVALID, "unknown kind %d", a->kind);
  if (a->cfg < 0 || a->cfg >= LLG_NUM_CFGS) return fail(LLG_E_INVALID, "cfg must be in [0, %d), got %d", LLG_NUM_CFGS, a->cfg);
  if (a->ksplit < 1 || a->ksplit > 64) return fail(LLG_E_INVALID, "ksplit must be in [1, 64], got %d", a->ksplit);
  if (int r = check_operand(a->a, a->lda_bytes, "a")) return r;
  if (int r = check_operand(a->b, a->ldb_bytes, "b")) return r;
  const int64_t P = a->a_rows, Q = a->b_rows;
  const int64_t K = a->a_row_bytes * 8 / ks.a_bits, Kb = a->b_row_bytes * 8 / ks.b_bits;
  if (K != Kb) return fail(LLG_E_INVALID, "a holds K=%lld but b holds K=%lld", (long long)K, (long long)Kb);
  if (K <= 0 || K % ks.k_align)
    return fail(LLG_E_INVALID, "K must be a positive multiple of %d for this kind, got %lld", ks.k_align, (long long)K);
  if (P < 1 || Q < 1 || P > INT32_MAX || Q > INT32_MAX || K > INT32_MAX) return fail(LLG_E_INVALID, "empty or too large problem");
  if (!a->y && !push) return fail(LLG_E_INVALID, "y must be 2-D with unit last stride");
  if (push) {
    if (push->world < 1 || push->world > 8 || push->rank < 0 || push->rank >= push->world)
      return fail(LLG_E_INVALID, "push: world must be in [1, 8] and rank inside it, got rank %d of %d", push->rank, push->world);
    if (!push->done) return fail(LLG_E_INVALID, "push: the local completion counter is missing");
    if (push->rows != (a->swap ? Q : P) || push->rows > LLG_AR_MAX_CTAS)
      return fail(LLG_E_INVALID, "push: rows must equal the token count of the GEMM and be at most %d, got %d", LLG_AR_MAX_CTAS,
                  push->rows);
    for (int d = 0; d < push->world; ++d)
      if (!push->dst[d] || !push->flags[d]) return fail(LLG_E_INVALID, "push: destination or flag pointer of rank %d is null", d);
  }
  if (a->out_dtype < LLG_DT_BF16 || a->out_dtype > LLG_DT_F32) return fail(LLG_E_INVALID, "y must be bfloat16, float16 or float32");
  const bool mixed = a->kind >= LLG_KIND_W8A16_BF16;
  if (mixed && !a->swap) return fail(LLG_E_INVALID, "mixed-precision kinds need the weight as operand a (swap)");

  TcDev p{};
  if (ks.a_sf) {
    if (!a->a_sf) return fail(LLG_E_INVALID, "this kind needs block scales for a");
    if (a->lda_sf % 4 || !aligned(a->a_sf, 4))
      return fail(LLG_E_INVALID, "a_sf needs unit column stride, a row stride that is a multiple of 4 and 4-byte alignment");
    p.a_sf = static_cast<const unsigned char*>(a->a_sf);
    p.lda_sf = a->lda_sf;
  }
  if (ks.b_sf) {
    if (!a->b_sf) return fail(LLG_E_INVALID, "this kind needs block scales for b");
    if (a->ldb_sf % 4 || !aligned(a->b_sf, 4))
      return fail(LLG_E_INVALID, "b_sf needs unit column stride, a row stride that is a multiple of 4 and 4-byte alignment");
    p.b_sf = static_cast<const unsigned char*>(a->b_sf);
    p.ldb_sf = a->ldb_sf;
  }
  if (a->row_scale_len != 0 && a->row_scale_len != 1 && a->row_scale_len != P)
    return fail(LLG_E_INVALID, "row_scale must have 1 or %lld elements, got %d", (long long)P, a->row_scale_len);
  if (a->col_scale_len != 0 && a->col_scale_len != 1 && a->col_scale_len != Q)
    return fail(LLG_E_INVALID, "col_scale must have 1 or %lld elements, got %d", (long long)Q, a->col_scale_len);
  if ((a->row_scale_len && !a->row_scale) || (a->col_scale_len && !a->col_scale))
    return fail(LLG_E_INVALID, "scale vector length given without a pointer");
  if (a->bias) {
    if (a->bias_dtype < LLG_DT_BF16 || a->bias_dtype > LLG_DT_F32)
      return fail(LLG_E_INVALID, "bias must be a contiguous bf16/f16/f32 vector of %lld elements", (long long)(a->bias_on_p ? P : Q));
  }
  const bool cluster = a->cluster && a->ksplit > 1;
  if (cluster && a->ksplit > 8) return fail(LLG_E_INVALID, "cluster split-K supports ksplit <= 8, got %d", a->ksplit);
  const TcTile tile = tc_tile_of(a->cfg);
  if (tile.pair && (a->ksplit > 1 || push))
    return fail(LLG_E_CONFIG, "config %d (256-row tiles on CTA pairs) runs without split-K and without the pushing epilogue", a->cfg);
  if (a->ksplit > 1 && !cluster) {
    const int64_t tiles = ((P + 127) / 128) * ((Q + tile.bq - 1) / tile.bq);
    if (!a->ws || !a->counters) return fail(LLG_E_INVALID, "workspace must be a contiguous 4-byte tensor, counters contiguous int32");
    if (a->ws_elems < (int64_t)a->ksplit * P * Q)
      return fail(LLG_E_INVALID, "workspace has %lld elements, needs %lld", (long long)a->ws_elems, (long long)a->ksplit * P * Q);
    if (a->counters_elems < tiles)
      return fail(LLG_E_INVALID, "counters has %lld, needs %lld", (long long)a->counters_elems, (long long)tiles);
    p.ws = a->ws;
    p.counters = reinterpret_cast<unsigned*>(a->counters);
  }
  if (a->prefetch && !aligned(a->prefetch, 16))
    return fail(LLG_E_INVALID, "prefetch tensor must be contiguous and 16-byte aligned");
  if (tc_stage_bytes_of(a->kind, a->cfg) == 0)
    return fail(LLG_E_CONFIG, "config %d cannot be launched for this kind: stage does not fit shared memory", a->cfg);

  if (validate_only) return LLG_OK;

  p.row_scale = a->row_scale; p.row_scale_len = a->row_scale_len;
  p.col_scale = a->col_scale; p.col_scale_len = a->col_scale_len;
  p.bias = a->bias; p.bias_dtype = a->bias ? a->bias_dtype : LLG_DT_NONE; p.bias_on_p = a->bias_on_p != 0;
  p.alpha_ptr = a->alpha_ptr; p.alpha = a->alpha;
  p.y = a->y; p.ldy = a->ldy; p.out_dtype = a->out_dtype;
  p.P = (int)P; p.Q = (int)Q; p.K = (int)K;
  p.k_atoms = (int)((a->a_row_bytes + 127) / 128);
  p.ksplit = a->ksplit; p.stages = a->stages;
  p.swap = a->swap != 0; p.cluster = cluster; p.a_is_weight = a->swap != 0;
  p.pf = a->prefetch; p.pf_bytes = a->prefetch ? a->prefetch_bytes : 0;
  p.status = status_word_device_ptr();
  if (!p.status) return fail(LLG_E_CUDA, "no device status word");
  if (push) {
    p.push_n = push->world; p.push_rank = push->rank; p.push_rows = push->rows; p.push_done = push->done;
    for (int d = 0; d < push->world; ++d) {
      p.push_y[d] = push->dst[d];
      p.push_flag[d] = push->flags[d];
    }
    p.y = push->dst[push->rank];
  }
  const uint32_t bq = (uint32_t)tile.bq;
  const uint32_t shape = ((bq >> 3) << 17) | (((tile.pair ? 256u : 128u) >> 4) << 24);  // N / 8 and M / 16 of one MMA
  switch (a->kind) {
    case LLG_KIND_BF16: case LLG_KIND_W8A16_BF16: case LLG_KIND_W4A16_BF16:
      p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | shape; p.bf16_act = 1; break;
    case LLG_KIND_F16: case LLG_KIND_W8A16_F16: case LLG_KIND_W4A16_F16:
      p.idesc = (1u << 4) | shape; break;
    case LLG_KIND_FP8: p.idesc = (1u << 4) | shape; break;          // e4m3 = format 0
    case LLG_KIND_INT8: p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | shape; break;
    case LLG_KIND_NVFP4: p.idesc = (1u << 7) | (1u << 10) | shape; break;  // e2m1, ue4m3 scales
  }

  // Row pitch of the A tiles. A 128-row MMA tile may own fewer rows: with a whole K range per CTA (no split-K) the
  // pitch is shrunk until the tiles fill the last round of SMs evenly, e.g. 14336 rows -> 148 tiles of 97 rows instead
  // of 112 tiles of 128 on 148 SMs. The TMA box is as tall as the pitch; the MMA still spans 128 rows.
  p.p_rows = 128;
  if (a->ksplit == 1 && !cluster && a->swap && !tile.pair) {
    const int64_t sms = sm_count() > 0 ? sm_count() : 1;
    const int64_t tq = (Q + tile.bq - 1) / tile.bq, tp0 = (P + 127) / 128;
    const int64_t rounds = (tp0 * tq + sms - 1) / sms;
    const int64_t want_tp = rounds * sms / tq;
    if (want_tp > tp0) {
      int64_t rows = (P + want_tp - 1) / want_tp;
      if (rows < 32) rows = 32;  // keep the TMA boxes reasonably tall
      if (rows < 128) p.p_rows = (int)rows;
    }
  }
  CUtensorMap ta, tb;
  // boxes: a CTA's rows of A and its rows of B (a CTA of a pair holds half of the B tile)
  if (!make_map(&ta, a->a, a->a_row_bytes, P, a->lda_bytes, p.p_rows, p.a_is_weight) ||
      !make_map(&tb, a->b, a->b_row_bytes, Q, a->ldb_bytes, tile.pair ? tile.bq / 2 : tile.bq, !p.a_is_weight))
    return fail(LLG_E_CUDA, "cuTensorMapEncodeTiled failed (operand layout not expressible as a TMA map)");

  CUtensorMap ts = ta, tt = tb;  // only read when sf_tma is set
  p.sf_tma = 0;
  const int fam = tc_family_of(a->kind);
  if (fam == FAM_W4A16 && p.a_sf && p.lda_sf % 16 == 0 && aligned(p.a_sf, 16) &&
      make_sf_map(&ts, p.a_sf, p.K / 16, P, p.lda_sf, p.p_rows))
    p.sf_tma = 1;
  if (fam == FAM_NVF4 && p.a_sf && p.b_sf && p.lda_sf % 16 == 0 && p.ldb_sf % 16 == 0 && aligned(p.a_sf, 16) &&
      aligned(p.b_sf, 16) && make_sf_map(&ts, p.a_sf, p.K / 16, P, p.lda_sf, p.p_rows) &&
      make_sf_map(&tt, p.b_sf, p.K / 16, Q, p.ldb_sf, tile.bq))
    p.sf_tma = 1;

  const bool pdl = pdl_on();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (tile.pair) e = tc_launch_pair(fam, ta, tb, p, tile.bq, pdl, s);
  else switch (fam) {
    case FAM_F16: e = tc_launch_f16(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
    case FAM_F8: e = tc_launch_f8(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
    case FAM_I8: e = tc_launch_i8(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
    case FAM_NVF4: e = tc_launch_nvf4(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
    case FAM_W8A16: e = tc_launch_w8a16(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
    default: e = tc_launch_w4a16(ta, tb, ts, tt, p, a->cfg, pdl, s); break;
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(e == cudaErrorInvalidConfiguration ? LLG_E_CONFIG : LLG_E_CUDA,
                "config %d cannot be launched for this kind: %s", a->cfg, cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_tc_gemm(const llg_tc_args* a, void* stream) { return tc_gemm_run(a, nullptr, stream); }

int llg_tc_gemm_push(const llg_tc_args* a, const llg_push_args* push, void* stream) {
  if (!push) return fail(LLG_E_INVALID, "null arguments");
  return tc_gemm_run(a, push, stream);
}

int llg_reduce_local(const void* recv, int64_t region_bytes, uint32_t* flags, void* out, const void* residual, void* q,
                     int64_t ldq, float* scale_out, int32_t rows, int32_t cols, int32_t dtype, float min_scale, int32_t world,
                     void* stream) {
  if (!recv || !flags) return fail(LLG_E_INVALID, "reduce: null pointer");
  if (world < 1 || world > 8) return fail(LLG_E_INVALID, "reduce: world must be in [1, 8], got %d", world);
  if (rows < 1 || rows > LLG_AR_MAX_CTAS)
    return fail(LLG_E_INVALID, "reduce: rows must be in [1, %d] (one CTA and one flag set per row), got %d", LLG_AR_MAX_CTAS, rows);
  if (cols < 8 || cols % 8 || cols > LLG_ARQ_MAX_COLS)
    return fail(LLG_E_INVALID, "reduce: cols must be a multiple of 8 in [8, %d], got %d", LLG_ARQ_MAX_COLS, cols);
  if (dtype != LLG_DT_BF16 && dtype != LLG_DT_F16) return fail(LLG_E_INVALID, "reduce: dtype must be bf16 or f16");
  if (region_bytes < (int64_t)rows * cols * 2 || region_bytes % 16 || !aligned(recv, 16))
    return fail(LLG_E_INVALID, "reduce: regions must be 16-byte aligned and hold rows * cols 16-bit values");
  if ((out && !aligned(out, 16)) || (residual && !aligned(residual, 16)))
    return fail(LLG_E_INVALID, "reduce: out and residual need 16-byte alignment");
  if (q && (!scale_out || ldq < cols || ldq % 8 || !aligned(q, 8)))
    return fail(LLG_E_INVALID, "reduce: q needs scale_out and 8-byte aligned rows (ldq %% 8 == 0, ldq >= cols)");
  if (!q && !out) return fail(LLG_E_INVALID, "reduce: nothing to write (neither out nor q)");
  unsigned* status = status_word_device_ptr();
  if (!status) return fail(LLG_E_CUDA, "no device status word");
  const cudaError_t e = reduce_local_launch(recv, region_bytes, flags, out, residual, q, ldq, scale_out, rows, cols, dtype,
                                            min_scale, world, status, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "reduce launch failed: %s", cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_allreduce_oneshot(const void* const* buffers_dev, uint32_t* const* flags_dev, void* out, int64_t bytes,
                          int32_t dtype, int32_t rank, int32_t world, int32_t ctas, void* stream) {
  if (!buffers_dev || !flags_dev || !out) return fail(LLG_E_INVALID, "all-reduce: null pointer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(LLG_E_INVALID, "all-reduce: world must be in [1, 8] and rank inside it, got rank %d of %d", rank, world);
  if (bytes <= 0 || bytes % 16 || !aligned(out, 16))
    return fail(LLG_E_INVALID, "all-reduce: size must be a positive multiple of 16 bytes and buffers 16-byte aligned");
  if (dtype < LLG_DT_BF16 || dtype > LLG_DT_F32) return fail(LLG_E_INVALID, "all-reduce: dtype must be bf16, f16 or f32");
  if (ctas < 1 || ctas > LLG_AR_MAX_CTAS) return fail(LLG_E_INVALID, "all-reduce: ctas must be in [1, %d]", LLG_AR_MAX_CTAS);
  unsigned* status = status_word_device_ptr();
  if (!status) return fail(LLG_E_CUDA, "no device status word");
  const cudaError_t e = allreduce_launch(buffers_dev, flags_dev, out, bytes / 16, rank, world, dtype, ctas, status,
                                         static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "all-reduce launch failed: %s", cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_allreduce_quant_fp8(const void* const* buffers_dev, uint32_t* const* flags_dev, void* out, void* q, int64_t ldq,
                            float* scale_out, int32_t rows, int32_t cols, int32_t dtype, float min_scale, int32_t rank,
                            int32_t world, void* stream) {
  if (!buffers_dev || !flags_dev || !q || !scale_out) return fail(LLG_E_INVALID, "all-reduce + quantize: null pointer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world)
    return fail(LLG_E_INVALID, "all-reduce: world must be in [1, 8] and rank inside it, got rank %d of %d", rank, world);
  if (rows < 1 || rows > LLG_AR_MAX_CTAS)
    return fail(LLG_E_INVALID, "all-reduce + quantize: rows must be in [1, %d] (one CTA and one flag set per row), got %d",
                LLG_AR_MAX_CTAS, rows);
  if (cols < 8 || cols % 8 || cols > LLG_ARQ_MAX_COLS)
    return fail(LLG_E_INVALID, "all-reduce + quantize: cols must be a multiple of 8 in [8, %d], got %d", LLG_ARQ_MAX_COLS, cols);
  if (dtype != LLG_DT_BF16 && dtype != LLG_DT_F16) return fail(LLG_E_INVALID, "all-reduce + quantize: dtype must be bf16 or f16");
  if (ldq < cols || ldq % 8 || !aligned(q, 8) || (out && !aligned(out, 16)))
    return fail(LLG_E_INVALID, "all-reduce + quantize: q needs 8-byte aligned rows (ldq %% 8 == 0, ldq >= cols), out 16-byte alignment");
  unsigned* status = status_word_device_ptr();
  if (!status) return fail(LLG_E_CUDA, "no device status word");
  const cudaError_t e = allreduce_quant_fp8_launch(buffers_dev, flags_dev, out, q, ldq, scale_out, rows, cols, dtype,
                                                   min_scale, rank, world, status, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "all-reduce + quantize launch failed: %s", cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_tc_gemm_static_ws(const llg_tc_args* args, void* stream) {
  if (!args) return fail(LLG_E_INVALID, "null arguments");
  // set-up, once per device, with that device current: the device address of the scratch array
  static unsigned char* base[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail("cudaGetDevice", e);
  if (dev < 0 || dev >= 64) return fail(LLG_E_INVALID, "device index %d not supported by the static workspace", dev);
  unsigned char* ptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!base[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return cuda_fail("cudaGetSymbolAddress(static workspace)", e);
      base[dev] = static_cast<unsigned char*>(p);
    }
    ptr = base[dev];
  }
  llg_tc_args a = *args;
  a.ws = nullptr; a.ws_elems = 0; a.counters = nullptr; a.counters_elems = 0;
  const bool cluster = a.cluster && a.ksplit > 1;
  int64_t tiles = 0;
  if (a.ksplit > 1 && !cluster) {
    // sizes are checked before any arithmetic on them
    const TcTile tile = tc_tile_of(a.cfg);
    if (tile.bq == 0) return fail(LLG_E_INVALID, "cfg must be in [0, %d), got %d", LLG_NUM_CFGS, a.cfg);
    if (a.ksplit > 64) return fail(LLG_E_INVALID, "ksplit must be in [1, 64], got %d", a.ksplit);
    if (a.a_rows < 1 || a.b_rows < 1 || a.a_rows > INT32_MAX || a.b_rows > INT32_MAX)
      return fail(LLG_E_INVALID, "empty or too large problem");
    const int64_t need = (int64_t)a.ksplit * a.a_rows * a.b_rows;  // < 2^6 * 2^31 * 2^31: no overflow
    tiles = ((a.a_rows + 127) / 128) * ((a.b_rows + tile.bq - 1) / tile.bq);
    if (need > LLG_STATIC_WS_ELEMS || tiles > LLG_STATIC_COUNTERS)
      return fail(LLG_E_INVALID, "static workspace too small: this GEMM needs %lld partials and %lld counters, the built-in "
                  "scratch holds %d and %d; use llg_tc_gemm with a caller-provided workspace", (long long)need,
                  (long long)tiles, LLG_STATIC_WS_ELEMS, LLG_STATIC_COUNTERS);
    a.ws = ptr;
    a.ws_elems = LLG_STATIC_WS_ELEMS;
    a.counters = reinterpret_cast<int32_t*>(ptr + kStaticWsBytes);
    a.counters_elems = LLG_STATIC_COUNTERS;
  }
  // the whole call is validated before anything is enqueued: a refused call must not touch the shared counters
  if (int r = tc_gemm_run(&a, nullptr, stream, true)) return r;
  if (tiles > 0) {
    // the array keeps whatever the last call left: the counters of this launch must start at zero
    e = cudaMemsetAsync(a.counters, 0, (size_t)tiles * 4, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail("clearing the static counters", e);
  }
  return tc_gemm_run(&a, nullptr, stream);
}

int llg_sf_relayout(const void* src, void* dst, int32_t rows, int32_t cols, int64_t ld, int32_t to_tiled, void* stream) {
  if (rows < 0 || cols < 0) return fail(LLG_E_INVALID, "scale relayout: negative size");
  if (rows == 0 || cols == 0) return LLG_OK;
  if (!src || !dst) return fail(LLG_E_INVALID, "scale relayout: null pointer");
  if (ld < cols) return fail(LLG_E_INVALID, "scale relayout: row pitch %lld is shorter than a row of %d bytes", (long long)ld, cols);
  if (!aligned(to_tiled ? dst : src, 16)) return fail(LLG_E_INVALID, "scale relayout: the tiled buffer needs 16-byte alignment");
  const cudaError_t e = sf_relayout_launch(src, dst, rows, cols, ld, to_tiled != 0, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "scale relayout launch failed: %s", cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_tc_gemm_host(const llg_tc_args* args, const void* x_host, void* x_dev, int64_t x_bytes, void* y_host,
                     int64_t y_bytes, void* stream) {
  if (!args || !x_host || !x_dev || !y_host) return fail(LLG_E_INVALID, "null arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(x_dev, x_host, (size_t)x_bytes, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return cuda_fail("host to device copy", e);
  if (int r = llg_tc_gemm(args, stream)) return r;
  e = cudaMemcpyAsync(y_host, args->y, (size_t)y_bytes, cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return cuda_fail("device to host copy", e);
  return LLG_OK;
}

// ---------------------------------------------------------------------------------------------------------------

int llg_quant(const llg_quant_args* a, void* stream) {
  if (!a) return fail(LLG_E_INVALID, "null arguments");
  if (a->in_dtype < LLG_DT_BF16 || a->in_dtype > LLG_DT_F32) return fail(LLG_E_INVALID, "quant: x must be bf16, f16 or f32");
  if (a->M < 0 || a->K < 0) return fail(LLG_E_INVALID, "quant: x must be a 2-D CUDA tensor with unit last stride");
  if (a->mode < LLG_QUANT_FP8_STATIC || a->mode > LLG_QUANT_NVFP4) return fail(LLG_E_INVALID, "quant: unknown mode %d", a->mode);
  if (a->mode == LLG_QUANT_NVFP4 && a->K % 16) return fail(LLG_E_INVALID, "quant: nvfp4 needs K %% 16 == 0");
  if (a->M == 0 || a->K == 0) return LLG_OK;  // empty: nothing to launch (and empty tensors have null pointers)
  switch (a->mode) {
    case LLG_QUANT_FP8_STATIC:
      if (!a->scale_in) return fail(LLG_E_INVALID, "quant: this mode needs scale_in float32[1]");
      break;
    case LLG_QUANT_FP8_PER_TOKEN:
    case LLG_QUANT_INT8_PER_TOKEN:
      if (!a->scale_out) return fail(LLG_E_INVALID, "quant: per-token modes need scale_out float32[M]");
      break;
    default:
      if (a->ldq % 8 || !aligned(a->q, 8)) return fail(LLG_E_INVALID, "quant: q must be [M, K/2] bytes with 8-byte aligned rows");
      if (!a->sf_out) return fail(LLG_E_INVALID, "quant: nvfp4 needs sf [M, K/16] bytes");
      if (!a->scale_in) return fail(LLG_E_INVALID, "quant: this mode needs scale_in float32[1]");
      break;
  }
  if (!a->x || !a->q) return fail(LLG_E_INVALID, "quant: q must be a 2-D 1-byte tensor with M rows");
  const cudaError_t e = quant_launch(*a, GatedExtra{nullptr, 0, nullptr, 0}, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "quant: launch failed (%s)", cudaGetErrorString(e));
  }
  return LLG_OK;
}

int llg_gated_quant(const llg_gated_quant_args* g, void* stream) {
  if (!g) return fail(LLG_E_INVALID, "null arguments");
  const llg_quant_args* a = &g->q;
  if (a->in_dtype < LLG_DT_BF16 || a->in_dtype > LLG_DT_F32) return fail(LLG_E_INVALID, "quant: x must be bf16, f16 or f32");
  if (a->mode != LLG_QUANT_FP8_PER_TOKEN && a->mode != LLG_QUANT_NVFP4 && a->mode != LLG_QUANT_NONE)
    return fail(LLG_E_INVALID, "gated quant: mode must be fp8 per token, nvfp4 or none, got %d", a->mode);
  if (a->M < 0 || a->K < 0) return fail(LLG_E_INVALID, "quant: x must be a 2-D CUDA tensor with unit last stride");
  if (a->mode == LLG_QUANT_NVFP4 && a->K % 16) return fail(LLG_E_INVALID, "quant: nvfp4 needs K %% 16 == 0");
  if (a->M == 0 || a->K == 0) return LLG_OK;
  if (!a->x || !g->up) return fail(LLG_E_INVALID, "gated quant: gate and up must be device pointers");
  if (a->mode == LLG_QUANT_NONE && !g->act) return fail(LLG_E_INVALID, "gated quant: mode none needs the activation output");
  if (a->mode != LLG_QUANT_NONE && !a->q) return fail(LLG_E_INVALID, "quant: q must be a 2-D 1-byte tensor with M rows");
  if (a->mode == LLG_QUANT_FP8_PER_TOKEN && !a->scale_out) return fail(LLG_E_INVALID, "quant: per-token modes need scale_out float32[M]");
  if (a->mode == LLG_QUANT_NVFP4 && (!a->sf_out || !a->scale_in || a->ldq % 8 || !aligned(a->q, 8)))
    return fail(LLG_E_INVALID, "quant: nvfp4 needs sf [M, K/16] bytes, scale_in float32[1] and 8-byte aligned q rows");
  const cudaError_t e = quant_launch(*a, GatedExtra{g->up, g->ldup, g->act, g->ldact}, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LLG_E_CUDA, "gated quant: launch failed (%s)", cudaGetErrorString(e));
  }
  return LLG_OK;
}

}  // extern "C"
