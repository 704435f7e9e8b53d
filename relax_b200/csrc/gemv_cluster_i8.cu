#include <cstring>

#include "gemv_cluster_inst.cuh"
namespace rb200 {
namespace gc {
int launch_cluster_i8(const ClusterParams& cp, const ClusterLaunch& l, const CUtensorMap& ts,
                      const CUtensorMap& tz, cudaStream_t stream) {
  return launch_bits<8>(cp, l, ts, tz, stream);
}
}  // namespace gc
}  // namespace rb200
