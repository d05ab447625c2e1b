// tcgen05 GEMM on CTA pairs (256-row tiles): instantiations for the kinds whose operands go to the MMA unconverted.
#include "umma_pair.cuh"

namespace llg {

cudaError_t tc_launch_pair(int family, const CUtensorMap& ta, const CUtensorMap& tb, const TcDev& p, int bq, bool pdl, cudaStream_t s) {
  switch (family) {
    case FAM_F16: return pair_launch_family<FAM_F16>(ta, tb, p, bq, pdl, s);
    case FAM_F8: return pair_launch_family<FAM_F8>(ta, tb, p, bq, pdl, s);
    case FAM_I8: return pair_launch_family<FAM_I8>(ta, tb, p, bq, pdl, s);
    default: return cudaErrorInvalidConfiguration;
  }
}

int tc_pair_stage_bytes(int family, int bq) {
  if (family != FAM_F16 && family != FAM_F8 && family != FAM_I8) return 0;
  return bq == 128 ? PairGeo<128>::kStageBytes : bq == 256 ? PairGeo<256>::kStageBytes : 0;
}

}  // namespace llg
