// torch.ops.lowlat_gemm.* as a C++ torch extension (module lowlat_gemm._C): the thin layer between tensors and the C ABI
// of libllg_core.so.
//
// Stands in for the reference's binding layer csrc/ops.cpp:420-451 - the same seven schemas, CUDA implementations for the
// compute ops, a Meta implementation for the functional skinny op, an empty Python module whose import registers them.
// Each op checks what only a tensor knows (device, dtype, rank, contiguity), puts raw pointers, sizes and strides into
// the C-ABI descriptor and calls the library on the current CUDA stream of the operand's device, under a device guard.
// Everything that can be decided from pointers and numbers is decided by the library, whose message
// ("lowlat_gemm: ...") becomes the RuntimeError.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <optional>

#include "../../include/llg_core.h"

namespace {

using at::Tensor;
using OptTensor = std::optional<Tensor>;

void lib_check(int rc) { TORCH_CHECK(rc == LLG_OK, llg_last_error()); }

int dt_code(at::ScalarType t) {
  switch (t) {
    case at::kBFloat16: return LLG_DT_BF16;
    case at::kHalf: return LLG_DT_F16;
    case at::kFloat: return LLG_DT_F32;
    default: return LLG_DT_NONE;
  }
}

void on_device_of(const Tensor& ref, const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.device() == ref.device(), "lowlat_gemm: ", name, " must be on ", ref.device());
}

void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

// prefetch range: a contiguous tensor on the same device; bytes = 0 or beyond the tensor mean "all of it"
template <class Args>
void set_prefetch(Args& a, const Tensor& ref, const OptTensor& t, int64_t nbytes) {
  if (!t.has_value()) return;
  on_device_of(ref, *t, "prefetch");
  TORCH_CHECK(t->is_contiguous(), "lowlat_gemm: prefetch tensor must be contiguous and 16-byte aligned");
  const int64_t total = t->numel() * t->element_size();
  a.prefetch = t->data_ptr();
  a.prefetch_bytes = (nbytes > 0 && nbytes < total) ? nbytes : total;
}

// ---- skinny ------------------------------------------------------------------------------------------------------

void skinny_run(const Tensor& y, const Tensor& x, const Tensor& w, const Tensor& ws, const Tensor& counters, int64_t rows,
                int64_t unroll, int64_t lanes_per_row, int64_t warps, int64_t ksplit, bool cluster, const OptTensor& prefetch,
                int64_t prefetch_bytes) {
  TORCH_CHECK(x.is_cuda(), "lowlat_gemm: x must be on CUDA");
  on_device_of(x, w, "w");
  on_device_of(x, y, "y");
  const bool half = x.scalar_type() == at::kHalf;
  TORCH_CHECK((half || x.scalar_type() == at::kBFloat16) && w.scalar_type() == x.scalar_type(),
              "lowlat_gemm: skinny: x and w must both be bfloat16 or both float16, got ", x.scalar_type(), " and ", w.scalar_type());
  TORCH_CHECK(y.scalar_type() == x.scalar_type() || y.scalar_type() == at::kFloat, "lowlat_gemm: skinny: output must be ",
              x.scalar_type(), " or float32, got ", y.scalar_type());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2, "lowlat_gemm: x, w, y must be 2-D");
  const int64_t m = x.size(0), k = x.size(1), n = w.size(0);
  TORCH_CHECK(w.size(1) == k, "lowlat_gemm: x is [", m, ", ", k, "] but w is [", n, ", ", w.size(1), "]");
  TORCH_CHECK(y.size(0) == m && y.size(1) == n, "lowlat_gemm: output must be [", m, ", ", n, "]");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1, "lowlat_gemm: x, w, y need unit stride in the last dimension");
  TORCH_CHECK(m <= INT32_MAX && n <= INT32_MAX && k <= INT32_MAX, "lowlat_gemm: N or K too large");
  llg_skinny_args a{};
  a.x = x.data_ptr(); a.ldx = x.stride(0);
  a.w = w.data_ptr(); a.ldw = w.stride(0);
  a.y = y.data_ptr(); a.ldy = y.stride(0);
  a.M = (int32_t)m; a.N = (int32_t)n; a.K = (int32_t)k;
  a.f16 = half; a.out_fp32 = y.scalar_type() == at::kFloat;
  a.rows = (int32_t)rows; a.unroll = (int32_t)unroll; a.lanes_per_row = (int32_t)lanes_per_row; a.warps = (int32_t)warps;
  a.ksplit = (int32_t)ksplit; a.cluster = cluster;
  if (ksplit > 1 && !cluster) {
    on_device_of(x, ws, "workspace");
    on_device_of(x, counters, "counters");
    TORCH_CHECK(ws.scalar_type() == at::kFloat && ws.is_contiguous() && counters.scalar_type() == at::kInt && counters.is_contiguous(),
                "lowlat_gemm: workspace must be contiguous float32, counters contiguous int32");
    a.ws = ws.data_ptr<float>(); a.ws_elems = ws.numel();
    a.counters = counters.data_ptr<int32_t>(); a.counters_elems = counters.numel();
  }
  set_prefetch(a, x, prefetch, prefetch_bytes);
  const c10::cuda::CUDAGuard guard(x.device());
  lib_check(llg_skinny(&a, stream_of(x)));
}

Tensor skinny(const Tensor& x, const Tensor& w, const Tensor& ws, const Tensor& counters, int64_t rows, int64_t unroll,
              int64_t lanes_per_row, int64_t warps, int64_t ksplit, bool out_fp32, bool cluster, const OptTensor& prefetch,
              int64_t prefetch_bytes) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2, "lowlat_gemm: x, w, y must be 2-D");
  Tensor y = at::empty({x.size(0), w.size(0)}, x.options().dtype(out_fp32 ? at::kFloat : x.scalar_type()));
  skinny_run(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster, prefetch, prefetch_bytes);
  return y;
}

Tensor skinny_meta(const Tensor& x, const Tensor& w, const Tensor&, const Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t,
                   bool out_fp32, bool, const OptTensor&, int64_t) {
  return at::empty({x.size(0), w.size(0)}, x.options().dtype(out_fp32 ? at::kFloat : x.scalar_type()));
}

void skinny_out(Tensor& y, const Tensor& x, const Tensor& w, const Tensor& ws, const Tensor& counters, int64_t rows, int64_t unroll,
                int64_t lanes_per_row, int64_t warps, int64_t ksplit, bool cluster, const OptTensor& prefetch, int64_t prefetch_bytes) {
  skinny_run(y, x, w, ws, counters, rows, unroll, lanes_per_row, warps, ksplit, cluster, prefetch, prefetch_bytes);
}

// ---- tensor-core GEMM --------------------------------------------------------------------------------------------

int a_bits_of(int64_t kind) {
  switch (kind) {
    case LLG_KIND_BF16: case LLG_KIND_F16: return 16;
    case LLG_KIND_FP8: case LLG_KIND_INT8: case LLG_KIND_W8A16_BF16: case LLG_KIND_W8A16_F16: return 8;
    case LLG_KIND_NVFP4: case LLG_KIND_W4A16_BF16: case LLG_KIND_W4A16_F16: return 4;
    default: return 0;
  }
}

void check_block_scales(const Tensor& ref, const OptTensor& sf, int64_t rows, int64_t kblocks, const char* name) {
  TORCH_CHECK(sf.has_value(), "lowlat_gemm: this kind needs block scales for ", name[0]);
  on_device_of(ref, *sf, name);
  TORCH_CHECK(sf->dim() == 2 && sf->element_size() == 1, "lowlat_gemm: ", name, " must be a 2-D 1-byte (e4m3) tensor");
  TORCH_CHECK(sf->size(0) == rows && sf->size(1) == kblocks, "lowlat_gemm: ", name, " must be [", rows, ", ", kblocks, "], got ",
              sf->sizes());
  TORCH_CHECK(sf->stride(1) == 1, "lowlat_gemm: ", name,
              " needs unit column stride, a row stride that is a multiple of 4 and 4-byte alignment");
}

void scale_vector(const Tensor& ref, const OptTensor& t, int64_t full, const char* name, const float** ptr, int32_t* len) {
  if (!t.has_value()) return;
  on_device_of(ref, *t, name);
  TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "lowlat_gemm: ", name, " must be a contiguous float32 tensor");
  TORCH_CHECK(t->numel() == 1 || t->numel() == full, "lowlat_gemm: ", name, " must have 1 or ", full, " elements, got ", t->numel());
  *ptr = t->data_ptr<float>();
  *len = t->numel() == 1 ? 1 : (int32_t)full;
}

void tc_gemm(Tensor& y, const Tensor& a, const Tensor& b, const OptTensor& a_sf, const OptTensor& b_sf, const OptTensor& row_scale,
             const OptTensor& col_scale, const OptTensor& bias, const OptTensor& alpha_t, double alpha, int64_t kind, bool swap,
             bool bias_on_p, int64_t cfg, int64_t stages, int64_t ksplit, const Tensor& ws, const Tensor& counters, bool cluster,
             const OptTensor& prefetch, int64_t prefetch_bytes) {
  const int bits = a_bits_of(kind);
  TORCH_CHECK(bits != 0, "lowlat_gemm: unknown kind ", kind);
  TORCH_CHECK(a.is_cuda(), "lowlat_gemm: operands must be on CUDA");
  on_device_of(a, b, "b");
  on_device_of(a, y, "y");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "lowlat_gemm: a and b must be 2-D");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "lowlat_gemm: a and b need unit stride in the last dimension");
  const int64_t p = a.size(0), q = b.size(0);
  TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1, "lowlat_gemm: y must be 2-D with unit last stride");
  TORCH_CHECK(y.size(0) == (swap ? q : p) && y.size(1) == (swap ? p : q), "lowlat_gemm: y must be [", swap ? q : p, ", ",
              swap ? p : q, "], got ", y.sizes());
  TORCH_CHECK(dt_code(y.scalar_type()) != LLG_DT_NONE, "lowlat_gemm: y must be bfloat16, float16 or float32");
  llg_tc_args t{};
  t.kind = (int32_t)kind; t.cfg = (int32_t)cfg; t.stages = (int32_t)stages; t.ksplit = (int32_t)ksplit;
  t.cluster = cluster; t.swap = swap;
  t.a = a.data_ptr(); t.a_rows = p; t.a_row_bytes = a.size(1) * a.element_size(); t.lda_bytes = a.stride(0) * a.element_size();
  t.b = b.data_ptr(); t.b_rows = q; t.b_row_bytes = b.size(1) * b.element_size(); t.ldb_bytes = b.stride(0) * b.element_size();
  const int64_t k = t.a_row_bytes * 8 / bits;
  const bool need_a = bits == 4, need_b = kind == LLG_KIND_NVFP4;
  if (need_a) {
    check_block_scales(a, a_sf, p, k / 16, "a_sf");
    t.a_sf = a_sf->data_ptr(); t.lda_sf = a_sf->stride(0);
  }
  if (need_b) {
    check_block_scales(a, b_sf, q, k / 16, "b_sf");
    t.b_sf = b_sf->data_ptr(); t.ldb_sf = b_sf->stride(0);
  }
  scale_vector(a, row_scale, p, "row_scale", &t.row_scale, &t.row_scale_len);
  scale_vector(a, col_scale, q, "col_scale", &t.col_scale, &t.col_scale_len);
  if (bias.has_value()) {
    on_device_of(a, *bias, "bias");
    const int64_t n_bias = bias_on_p ? p : q;
    TORCH_CHECK(dt_code(bias->scalar_type()) != LLG_DT_NONE && bias->is_contiguous() && bias->numel() == n_bias,
                "lowlat_gemm: bias must be a contiguous bf16/f16/f32 vector of ", n_bias, " elements");
    t.bias = bias->data_ptr(); t.bias_dtype = dt_code(bias->scalar_type());
  }
  t.bias_on_p = bias_on_p;
  if (alpha_t.has_value()) {
    on_device_of(a, *alpha_t, "alpha");
    TORCH_CHECK(alpha_t->scalar_type() == at::kFloat && alpha_t->numel() == 1, "lowlat_gemm: alpha tensor must be one float32");
    t.alpha_ptr = alpha_t->data_ptr<float>();
  }
  t.alpha = (float)alpha;
  t.y = y.data_ptr(); t.ldy = y.stride(0); t.out_dtype = dt_code(y.scalar_type());
  if (ksplit > 1 && !cluster) {
    on_device_of(a, ws, "workspace");
    on_device_of(a, counters, "counters");
    TORCH_CHECK(ws.element_size() == 4 && ws.is_contiguous() && counters.scalar_type() == at::kInt && counters.is_contiguous(),
                "lowlat_gemm: workspace must be a contiguous 4-byte tensor, counters contiguous int32");
    t.ws = ws.data_ptr(); t.ws_elems = ws.numel();
    t.counters = counters.data_ptr<int32_t>(); t.counters_elems = counters.numel();
  }
  set_prefetch(t, a, prefetch, prefetch_bytes);
  const c10::cuda::CUDAGuard guard(a.device());
  lib_check(llg_tc_gemm(&t, stream_of(a)));
}

// ---- quantizers --------------------------------------------------------------------------------------------------

void quant(const Tensor& x, Tensor& q, const OptTensor& sf, const OptTensor& scale_in, const OptTensor& scale_out, int64_t mode,
           double min_scale) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "lowlat_gemm: quant: x must be a 2-D CUDA tensor with unit last stride");
  on_device_of(x, q, "q");
  TORCH_CHECK(dt_code(x.scalar_type()) != LLG_DT_NONE, "lowlat_gemm: quant: x must be bf16, f16 or f32");
  const int64_t m = x.size(0), k = x.size(1);
  TORCH_CHECK(q.dim() == 2 && q.size(0) == m && q.stride(1) == 1 && q.element_size() == 1,
              "lowlat_gemm: quant: q must be a 2-D 1-byte tensor with M rows");
  TORCH_CHECK(m <= INT32_MAX && k <= INT32_MAX, "lowlat_gemm: quant: x too large");
  llg_quant_args a{};
  a.mode = (int32_t)mode; a.in_dtype = dt_code(x.scalar_type());
  a.x = x.data_ptr(); a.ldx = x.stride(0); a.q = q.data_ptr(); a.ldq = q.stride(0);
  a.min_scale = (float)min_scale; a.M = (int32_t)m; a.K = (int32_t)k;
  const bool per_token = mode == LLG_QUANT_FP8_PER_TOKEN || mode == LLG_QUANT_INT8_PER_TOKEN;
  const bool takes_scale = mode == LLG_QUANT_FP8_STATIC || mode == LLG_QUANT_NVFP4;
  if (per_token) {
    TORCH_CHECK(q.size(1) == k, "lowlat_gemm: quant: q must be [M, K]");
    TORCH_CHECK(scale_out.has_value() && scale_out->scalar_type() == at::kFloat && scale_out->is_contiguous() && scale_out->numel() == m,
                "lowlat_gemm: quant: per-token modes need scale_out float32[M]");
    on_device_of(x, *scale_out, "scale_out");
    a.scale_out = scale_out->data_ptr<float>();
  }
  if (takes_scale) {
    TORCH_CHECK(scale_in.has_value() && scale_in->scalar_type() == at::kFloat && scale_in->numel() == 1,
                "lowlat_gemm: quant: this mode needs scale_in float32[1]");
    on_device_of(x, *scale_in, "scale_in");
    a.scale_in = scale_in->data_ptr<float>();
  }
  if (mode == LLG_QUANT_FP8_STATIC) TORCH_CHECK(q.size(1) == k, "lowlat_gemm: quant: q must be [M, K]");
  if (mode == LLG_QUANT_NVFP4) {
    TORCH_CHECK(k % 16 == 0, "lowlat_gemm: quant: nvfp4 needs K % 16 == 0");
    TORCH_CHECK(q.size(1) == k / 2, "lowlat_gemm: quant: q must be [M, K/2] bytes with 8-byte aligned rows");
    TORCH_CHECK(sf.has_value() && sf->dim() == 2 && sf->size(0) == m && sf->size(1) == k / 16 && sf->element_size() == 1 &&
                    sf->stride(1) == 1, "lowlat_gemm: quant: nvfp4 needs sf [M, K/16] bytes");
    on_device_of(x, *sf, "sf");
    a.sf_out = sf->data_ptr(); a.ldsf = sf->stride(0);
  }
  const c10::cuda::CUDAGuard guard(x.device());
  lib_check(llg_quant(&a, stream_of(x)));
}

// ---- facts and switches ------------------------------------------------------------------------------------------

std::vector<int64_t> tc_info(int64_t kind, int64_t cfg) {
  int32_t out[4];
  lib_check(llg_tc_info((int32_t)kind, (int32_t)cfg, out));
  return {out[0], out[1], out[2], out[3]};
}

void set_pdl(bool on) { llg_set_pdl(on ? 1 : 0); }
bool pdl_enabled() { return llg_pdl_enabled() != 0; }

}  // namespace

TORCH_LIBRARY(lowlat_gemm, m) {
  m.def("skinny(Tensor x, Tensor w, Tensor ws, Tensor counters, int rows, int unroll, int lanes_per_row, int warps, int ksplit, "
        "bool out_fp32=False, bool cluster=False, Tensor? prefetch=None, int prefetch_bytes=0) -> Tensor");
  m.def("skinny_out(Tensor(a!) y, Tensor x, Tensor w, Tensor ws, Tensor counters, int rows, int unroll, int lanes_per_row, "
        "int warps, int ksplit, bool cluster=False, Tensor? prefetch=None, int prefetch_bytes=0) -> ()");
  m.def("tc_gemm(Tensor(a!) y, Tensor a, Tensor b, Tensor? a_sf, Tensor? b_sf, Tensor? row_scale, Tensor? col_scale, Tensor? bias, "
        "Tensor? alpha_t, float alpha, int kind, bool swap, bool bias_on_p, int cfg, int stages, int ksplit, Tensor ws, "
        "Tensor counters, bool cluster=False, Tensor? prefetch=None, int prefetch_bytes=0) -> ()");
  m.def("quant(Tensor x, Tensor(a!) q, Tensor(b!)? sf, Tensor? scale_in, Tensor(c!)? scale_out, int mode, float min_scale) -> ()");
  m.def("tc_info(int kind, int cfg) -> int[]", &tc_info);
  m.def("set_pdl(bool on) -> ()", &set_pdl);
  m.def("pdl_enabled() -> bool", &pdl_enabled);
}

TORCH_LIBRARY_IMPL(lowlat_gemm, CUDA, m) {
  m.impl("skinny", &skinny);
  m.impl("skinny_out", &skinny_out);
  m.impl("tc_gemm", &tc_gemm);
  m.impl("quant", &quant);
}

TORCH_LIBRARY_IMPL(lowlat_gemm, Meta, m) { m.impl("skinny", &skinny_meta); }

PYBIND11_MODULE(_C, m) { m.doc() = "registers torch.ops.lowlat_gemm on import"; }
