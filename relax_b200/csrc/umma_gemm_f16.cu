#include "umma_gemm_inst.cuh"
namespace rb200 {
namespace um {
int launch_gemm_f16(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& tw, cudaStream_t stream) {
  return launch_inst<16, kZeroConstInt, 0, kSrcGlobal>(pp, l, tx, tw, stream);
}
}  // namespace um
}  // namespace rb200
