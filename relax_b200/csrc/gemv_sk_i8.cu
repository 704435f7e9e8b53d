#include "gemv_sk_inst.cuh"
namespace rb200 {
namespace sk {
int launch_sk_i8(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
                 cudaStream_t stream) {
  return launch_bits<8>(pp, l, tx, ts, tz, stream);
}
}  // namespace sk
}  // namespace rb200
