// Skinny GEMV instantiations with 32 lanes per weight row.
#include "skinny_kernel.cuh"

namespace llg {

cudaError_t skinny_launch_l32(const SkinnyDev& p, int rows, int unroll, int warps, bool f16, bool pdl, cudaStream_t s) {
  return skinny_launch_lpr<32>(p, rows, unroll, warps, f16, pdl, s);
}

}  // namespace llg
