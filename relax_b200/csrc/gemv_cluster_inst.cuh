// Instantiation + dispatch of gemv_cluster_kernel for one weight width (included by the
// per-width translation units so they compile in parallel).
#pragma once
#include "gemv_cluster.cuh"

namespace rb200 {
namespace gc {

// Shared memory of one CTA for a given pipeline depth.
inline size_t smem_for(const ClusterLaunch& l, int stages) {
  return (size_t)stages * l.stage_bytes + l.fixed_bytes + (size_t)(2 * stages + 3) * sizeof(uint64_t);
}

template <int BITS, int MT, int ZMODE, int GROUP, int SRC>
int launch_inst(ClusterParams cp, const ClusterLaunch& l, const CUtensorMap& ts,
                const CUtensorMap& tz, cudaStream_t stream) {
  auto kern = gemv_cluster_kernel<BITS, MT, ZMODE, GROUP, SRC>;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters[4];  // co-resident clusters for S = 1, 2, 4, 8
  static thread_local size_t max_clusters_smem = 0;
  int dev = 0;
  RB200_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    RB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
    max_clusters_smem = 0;
  }
  // pipeline depth from the per-CTA shared-memory budget (1 KB per CTA is reserved by the system)
  const size_t budget = (size_t)(228 * 1024) / l.ctas_per_sm - 1024;
  int stages = (int)((budget - l.fixed_bytes - 64) / l.stage_bytes);
  if (stages > 12) stages = 12;
  if (stages < 1) stages = 1;
  const size_t smem = smem_for(l, stages);

  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  // Measured: launched as a programmatic dependent this kernel gains nothing at m <= 16 and loses
  // 5-10 us at m > 16, so it does not opt in; it still lets its own dependents start early.
  attr[1].val.programmaticStreamSerializationAllowed = 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;

  if (max_clusters_smem != smem) {
    for (int i = 0; i < 4; ++i) {
      const int s = 1 << i;
      attr[0].val.clusterDim.x = (unsigned)s;
      cfg.gridDim = dim3((unsigned)(s * l.sm_count * 4), 1, 1);
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
      if (e != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      max_clusters[i] = n;
    }
    max_clusters_smem = smem;
  }

  // split factor: rounds of tiles per cluster times the chunks a rank streams per tile, plus a
  // charge per tile for publishing and summing partials
  int best = -1, best_clusters = 0;
  double best_cost = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int s = 1 << i;
    if (s > l.cpt || max_clusters[i] <= 0) continue;
    const int nc = l.n_tiles < max_clusters[i] ? l.n_tiles : max_clusters[i];
    const int rounds = (l.n_tiles + nc - 1) / nc;
    const double cost = rounds * ((double)((l.cpt + s - 1) / s) + (s > 1 ? 0.6 : 0.0));
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
      best_clusters = nc;
    }
  }
  RB200_CHECK(best > 0, "no feasible cluster configuration (shared memory %zu bytes)", smem);
  cp.split = best;
  cp.g.stages = stages;
  attr[0].val.clusterDim.x = (unsigned)best;
  cfg.gridDim = dim3((unsigned)(best_clusters * best), 1, 1);
  RB200_CUDA(cudaLaunchKernelEx(&cfg, kern, cp, ts, tz));
  return 0;
}

template <int BITS, int MT, int ZMODE>
int launch_gs(const ClusterParams& cp, const ClusterLaunch& l, const CUtensorMap& ts,
              const CUtensorMap& tz, cudaStream_t stream) {
#define RB200_CASE(G, S) \
  if (l.group_code == (G) && l.src == (S)) return launch_inst<BITS, MT, ZMODE, G, S>(cp, l, ts, tz, stream)
  RB200_CASE(32, kSrcGlobal);
  RB200_CASE(64, kSrcGlobal);
  RB200_CASE(128, kSrcGlobal);
  RB200_CASE(0, kSrcGlobal);
  RB200_CASE(-1, kSrcGlobal);
  if (BITS == 4) RB200_CASE(32, kSrcSmemNK);
  RB200_CASE(32, kSrcSmemKN);
  RB200_CASE(64, kSrcSmemKN);
  RB200_CASE(128, kSrcSmemKN);
#undef RB200_CASE
  RB200_CHECK(false, "no decode kernel for group code %d with scale source %d", l.group_code, l.src);
  return -1;
}

template <int BITS>
int launch_bits(const ClusterParams& cp, const ClusterLaunch& l, const CUtensorMap& ts,
                const CUtensorMap& tz, cudaStream_t stream) {
#define RB200_MZ(M, Z) \
  if (l.mt == (M) && l.zmode == (Z)) return launch_gs<BITS, M, Z>(cp, l, ts, tz, stream)
  RB200_MZ(1, kZeroConstInt);
  RB200_MZ(2, kZeroConstInt);
  RB200_MZ(4, kZeroConstInt);
  RB200_MZ(1, kZeroGeneral);
  RB200_MZ(2, kZeroGeneral);
  RB200_MZ(4, kZeroGeneral);
#undef RB200_MZ
  RB200_CHECK(false, "bad m-tile count %d / zero mode %d", l.mt, l.zmode);
  return -1;
}

}  // namespace gc
}  // namespace rb200
