// Skinny GEMV instantiations with 32 virtual lanes per weight row.
#include "skinny_stream.cuh"

namespace llg {

cudaError_t skinny_launch_l32(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  return sk_launch_lpr<32>(p, rows, unroll, warps, f16, pdl, s);
}

}  // namespace llg
