// tcgen05 GEMM instantiations of one kernel family (all tile configs).
#include "umma_gemm.cuh"

namespace llg {

cudaError_t tc_launch_f16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& ts, const CUtensorMap& tt, const TcDev& p, int cfg, bool pdl, cudaStream_t s) {
  return umma_launch_family<FAM_F16>(ta, tb, ts, tt, p, cfg, pdl, s);
}

int tc_stage_bytes_f16(int cfg) { return umma_stage_bytes<FAM_F16>(cfg); }

}  // namespace llg
