#include "umma_gemm_inst.cuh"
namespace rb200 {
namespace um {
int launch_gemm_i4c(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream) {
  return launch_gs<4, kZeroConstInt>(pp, l, tx, stream);
}
}  // namespace um
}  // namespace rb200
