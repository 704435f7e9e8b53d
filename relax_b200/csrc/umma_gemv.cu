// Host side + instantiations of the tcgen05 decode kernel.
#include "umma_gemv.cuh"

#include <cstdlib>
#include <cstring>


namespace rb200 {
namespace ug {

template <int ZMODE, int GROUP, int SRC>
int launch_inst(const Params& pp, int grid, size_t smem, cudaStream_t stream) {
  auto kern = umma_gemv_kernel<ZMODE, GROUP, SRC>;
  static thread_local int configured_device = -1;
  int dev = 0;
  RB200_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    RB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  static const bool debug = getenv("RB200_DEBUG") != nullptr;
  if (debug) {
    int occ = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kThreads, smem);
    cudaFuncAttributes fa;
    cudaFuncGetAttributes(&fa, kern);
    int occ0 = -1, occ64 = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ0, kern, kThreads, 0);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ64, kern, kThreads, 65536);
    fprintf(stderr, "[rb200] umma_gemv grid=%d smem=%zu stages=%d nb=%d occupancy=%d CTAs/SM (regs %d static smem %zu local %zu maxthr %d; occ@0=%d occ@64K=%d)\n", grid, smem,
            pp.g.stages, pp.nb, occ, fa.numRegs, fa.sharedSizeBytes, fa.localSizeBytes, fa.maxThreadsPerBlock, occ0, occ64);
  }
  kern<<<grid, kThreads, smem, stream>>>(pp);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

template <int ZMODE>
int launch_gs(int group_code, int src, const Params& pp, int grid, size_t smem, cudaStream_t stream) {
#define RB200_CASE(G, S) \
  if (group_code == (G) && src == (S)) return launch_inst<ZMODE, G, S>(pp, grid, smem, stream)
  RB200_CASE(32, kSrcGlobal);
  RB200_CASE(64, kSrcGlobal);
  RB200_CASE(128, kSrcGlobal);
  RB200_CASE(0, kSrcGlobal);
  RB200_CASE(-1, kSrcGlobal);
  RB200_CASE(32, kSrcSmemNK);
  RB200_CASE(32, kSrcSmemKN);
  RB200_CASE(64, kSrcSmemKN);
  RB200_CASE(128, kSrcSmemKN);
#undef RB200_CASE
  RB200_CHECK(false, "no tcgen05 decode kernel for group code %d with scale source %d", group_code, src);
  return -1;
}

}  // namespace ug

int umma_gemv_run(const GemvParams& p_in, int bits, int zmode, int sm_count, float* partial,
                  size_t partial_bytes, unsigned* flags, size_t flag_count, unsigned epoch,
                  cudaStream_t stream) {
  using namespace ug;
  // coverage: int4, whole 128-row tiles, TMA-loadable x
  if (bits != 4 || p_in.n % kTileRows != 0 || p_in.k % kKBlock != 0 || p_in.m > 32) return 1;
  if ((reinterpret_cast<uintptr_t>(p_in.x) & 15u) != 0 || (p_in.ldx * 2) % 16 != 0) return 1;
  static const bool disabled = getenv("RB200_GEMV_NO_TCGEN05") != nullptr;
  if (disabled) return 1;

  Params pp;
  memset(&pp, 0, sizeof(pp));
  pp.g = p_in;
  GemvParams& p = pp.g;
  pp.nb = p.m <= 16 ? 16 : 32;

  int group_code;
  if (p.group <= 0 || p.group >= p.k) {
    group_code = 0;
  } else {
    RB200_CHECK(p.group % 16 == 0 && p.k % p.group == 0,
                "group_size=%d must divide k=%d and be a multiple of 16", p.group, p.k);
    group_code = (p.group == 32 || p.group == 64 || p.group == 128) ? p.group : -1;
  }
  int src = kSrcGlobal;
  const int64_t kg = group_code != 0 ? p.k / p.group : 0;
  const bool al = (reinterpret_cast<uintptr_t>(p.s) & 15u) == 0 &&
                  (p.z == nullptr || (reinterpret_cast<uintptr_t>(p.z) & 15u) == 0);
  static const bool no_tma = getenv("RB200_GEMV_NO_SCALE_TMA") != nullptr;
  if (group_code > 0 && al && !no_tma) {
    if (p.s_g == 1 && p.s_n == kg && p.group == 32 && (kg * 2) % 16 == 0) src = kSrcSmemNK;
    else if (p.s_n == 1 && p.s_g == p.n && kChunk % p.group == 0) src = kSrcSmemKN;
  }

  if (src != kSrcGlobal && zmode == kZeroGeneral && p.z) pp.has_z_tile = 1;

  const int cpt = (p.k + kChunk - 1) / kChunk;
  const int n_tiles = p.n / kTileRows;
  p.chunks_per_tile = cpt;
  p.total_iters = (long long)cpt * n_tiles;
  static const int env_stages = getenv("RB200_GEMV_STAGES") ? atoi(getenv("RB200_GEMV_STAGES")) : 0;
  static const int env_grid = getenv("RB200_GEMV_GRID") ? atoi(getenv("RB200_GEMV_GRID")) : 0;
  long long grid = (long long)sm_count;  // one persistent CTA per SM (tensor-memory kernels get occupancy 1)
  if (env_grid > 0) grid = env_grid;
  if (grid > p.total_iters) grid = p.total_iters;

  const Layout lay = make_layout(pp.nb, src, zmode);
  const size_t fixed = 1024 /* alignment slack */ + (size_t)(2 * 16 + 2 * kNumA + 2 * kNumD) * sizeof(uint64_t) + 16;
  const size_t budget = (size_t)227 * 1024;
  int stages = (int)((budget - fixed) / lay.stage_bytes);
  if (env_stages > 0) stages = env_stages;
  if (stages > 16) stages = 16;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const size_t smem = (size_t)stages * lay.stage_bytes + fixed;

  const size_t need_partial = (size_t)grid * pp.nb * kTileRows * sizeof(float);
  RB200_CHECK(partial_bytes >= need_partial && flag_count >= (size_t)grid * 4,
              "split-k scratch too small: need %zu bytes and %lld flags", need_partial, grid);
  pp.partial = partial;
  pp.flags = flags;
  pp.epoch = epoch;

  if (zmode == kZeroConstInt)
    return launch_gs<kZeroConstInt>(group_code, src, pp, (int)grid, smem, stream);
  return launch_gs<kZeroGeneral>(group_code, src, pp, (int)grid, smem, stream);
}

}  // namespace rb200
