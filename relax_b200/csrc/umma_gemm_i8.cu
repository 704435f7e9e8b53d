#include "umma_gemm_inst.cuh"
namespace rb200 {
namespace um {
int launch_gemm_i8(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream) {
  if (l.zmode == kZeroConstInt) return launch_gs<8, kZeroConstInt>(pp, l, tx, stream);
  return launch_gs<8, kZeroGeneral>(pp, l, tx, stream);
}
}  // namespace um
}  // namespace rb200
