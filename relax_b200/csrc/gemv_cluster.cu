// Host side of the cluster decode kernel: picks the split factor, the pipeline depth and how
// scales reach the consumers, builds the TMA tensor maps, launches.
#include <cstdlib>
#include <cstring>

#include "gemv_cluster.cuh"
#include "tensormap.h"

namespace rb200 {
namespace gc {

size_t cluster_stage_bytes(int bits, int mt, int zmode, int src) {
  const int frag = bits == 4 ? 64 : 32;
  const int chunk = frag * kBlocksPerChunk;
  const int xpitch = chunk * 2 + (bits == 4 ? 16 : 64);
  size_t b = (size_t)kConsumerWarps * kBlocksPerChunk * kTileBytes;
  b += (size_t)((mt * 8 * xpitch + 127) / 128) * 128;
  if (src != kSrcGlobal) b += kScaleBoxBytes * ((zmode == kZeroGeneral) ? 2 : 1);
  return b;
}

}  // namespace gc

int gemv_cluster_run(const GemvParams& p_in, int bits, int zmode, int sm_count, cudaStream_t stream) {
  using namespace gc;
  const int frag = bits == 4 ? 64 : 32;
  const int chunk = frag * kBlocksPerChunk;
  const int lane_run = frag / 4;
  ClusterParams cp;
  memset(&cp, 0, sizeof(cp));
  cp.g = p_in;
  GemvParams& p = cp.g;
  ClusterLaunch l;
  memset(&l, 0, sizeof(l));
  l.bits = bits;
  l.zmode = zmode;
  l.mt = p.m <= 8 ? 1 : (p.m <= 16 ? 2 : 4);

  if (p.group <= 0 || p.group >= p.k) {
    l.group_code = 0;
  } else {
    RB200_CHECK(p.group % lane_run == 0 && p.k % p.group == 0,
                "group_size=%d must divide k=%d and be a multiple of %d", p.group, p.k, lane_run);
    l.group_code = (p.group == 32 || p.group == 64 || p.group == 128) ? p.group : -1;
  }

  // how scales travel: TMA tiles when the layout is one of the two regular forms
  l.src = kSrcGlobal;
  const int64_t kg = l.group_code > 0 ? p.k / p.group : 0;
  const bool z_ok = p.z == nullptr || (reinterpret_cast<uintptr_t>(p.z) & 15u) == 0;
  const bool s_al = (reinterpret_cast<uintptr_t>(p.s) & 15u) == 0 && z_ok;
  if (l.group_code > 0 && s_al) {
    if (p.s_g == 1 && p.s_n == kg && bits == 4 && p.group == 32 && (kg * 2) % 16 == 0)
      l.src = kSrcSmemNK;
    else if (p.s_n == 1 && p.s_g == p.n && chunk % p.group == 0)
      l.src = kSrcSmemKN;
  }
  CUtensorMap ts, tz;
  memset(&ts, 0, sizeof(ts));
  memset(&tz, 0, sizeof(tz));
  cp.has_z_tile = 0;
  if (l.src == kSrcSmemNK) {
    if (make_tensor_map_2d(&ts, p.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, kg, p.n, kg * 2, 8, kTileRows,
                           CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
    cp.s_box_bytes = 8 * kTileRows * 2;
    tz = ts;
    if (zmode == kZeroGeneral && p.z) {
      if (make_tensor_map_2d(&tz, p.z, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, kg, p.n, kg * 2, 8, kTileRows,
                             CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
        return -1;
      cp.has_z_tile = 1;
    }
  } else if (l.src == kSrcSmemKN) {
    const unsigned gpc = (unsigned)(chunk / p.group);
    if (make_tensor_map_2d(&ts, p.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.n, kg, (unsigned long long)p.n * 2,
                           kTileRows, gpc, CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
    cp.s_box_bytes = gpc * kTileRows * 2;
    tz = ts;
    if (zmode == kZeroGeneral && p.z) {
      if (make_tensor_map_2d(&tz, p.z, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.n, kg,
                             (unsigned long long)p.n * 2, kTileRows, gpc, CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
        return -1;
      cp.has_z_tile = 1;
    }
  }

  const int cpt = (p.k + chunk - 1) / chunk;
  const int n_tiles = (p.n + kTileRows - 1) / kTileRows;
  p.chunks_per_tile = cpt;
  p.total_iters = (long long)cpt * n_tiles;

  l.n_tiles = n_tiles;
  l.cpt = cpt;
  l.sm_count = sm_count;
  l.ctas_per_sm = 2;
  l.stage_bytes = cluster_stage_bytes(bits, l.mt, zmode, l.src);
  l.fixed_bytes = (size_t)2 * kConsumerWarps * l.mt * 512;

  if (bits == 4) return launch_cluster_i4(cp, l, ts, tz, stream);
  return launch_cluster_i8(cp, l, ts, tz, stream);
}

}  // namespace rb200
