// Test infrastructure, not product code. C entry points over the REFERENCE's own torch-free launchers, so that its
// quantizer kernels (csrc/quant.cu, behind quant_launch, csrc/quant.h:31) and its GEMV (csrc/gemv.cuh through
// launch_lpr<LPR>, csrc/params.h:37-38) can be run on a GPU from a test and their output bytes compared with this
// repository's kernels and with the numpy oracle. The reference sources are compiled where they lie (see the Makefile
// next to this file); nothing of them is copied here. The two process-wide helpers the reference's launchers expect from
// its csrc/tc_info.cu:67-78 (PDL switch, SM count) are supplied here so that file, which pulls in the mma.sync GEMM,
// need not be built.
#include <cuda_runtime.h>

#include "params.h"
#include "quant.h"

namespace llg {
bool pdl_enabled() { return false; }
int sm_count_current() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}
}  // namespace llg

extern "C" {

// mode / in_dtype as in csrc/quant.h:9-22. Returns 0 on success, 1 when the launcher refused, 2 on a CUDA error.
__attribute__((visibility("default"))) int ref_quant(int mode, int in_dtype, const void* x, long long ldx, void* q,
                                                     long long ldq, void* sf_out, long long ldsf, const float* scale_in,
                                                     float* scale_out, float min_scale, int M, int K) {
  llg::QuantParams p{};
  p.mode = mode; p.in_dtype = in_dtype; p.x = x; p.ldx = ldx; p.q = q; p.ldq = ldq; p.sf_out = sf_out; p.ldsf = ldsf;
  p.scale_in = scale_in; p.scale_out = scale_out; p.min_scale = min_scale; p.M = M; p.K = K;
  if (!llg::quant_launch(p, nullptr)) return 1;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 2;
}

// The reference's GEMV, workspace or cluster split-K. counters must be zero on entry.
__attribute__((visibility("default"))) int ref_gemv(const void* x, const void* w, void* y, long long ldx, long long ldw,
                                                    long long ldy, int M, int N, int K, int f16, int out_fp32, int rows,
                                                    int unroll, int lanes_per_row, int warps, int ksplit, int cluster,
                                                    float* ws, unsigned* counters) {
  llg::Params p{};
  p.x = x; p.w = w; p.y = y; p.ldx = ldx; p.ldw = ldw; p.ldy = ldy; p.M = M; p.N = N; p.K = K; p.ksplit = ksplit;
  p.ws = ws; p.counters = counters; p.out_fp32 = out_fp32 != 0; p.f16 = f16 != 0; p.cluster = cluster != 0;
  const llg::LaunchConfig c{rows, unroll, lanes_per_row, warps, ksplit};
  bool ok = false;
  switch (lanes_per_row) {
    case 8: ok = llg::launch_lpr<8>(p, c, nullptr); break;
    case 16: ok = llg::launch_lpr<16>(p, c, nullptr); break;
    case 32: ok = llg::launch_lpr<32>(p, c, nullptr); break;
    default: break;
  }
  if (!ok) return 1;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
