// Skinny GEMV instantiations with 8 virtual lanes per weight row.
#include "skinny_stream.cuh"

namespace llg {

cudaError_t skinny_launch_l8(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  return sk_launch_lpr<8>(p, rows, unroll, warps, f16, pdl, s);
}

}  // namespace llg
