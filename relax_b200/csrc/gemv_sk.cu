// Host side of the stream-k decode kernel: scale staging mode, pipeline depth, grid, launch.
#include "gemv_sk.cuh"

#include <cstdlib>
#include <cstring>

namespace rb200 {

int gemv_sk_run(const GemvParams& p_in, int bits, int zmode, int sm_count, float* partial, size_t partial_bytes,
                unsigned* flags, size_t flag_count, cudaStream_t stream) {
  using namespace sk;
  const int frag = bits == 4 ? 64 : 32;
  const int chunk = frag * kBlocksPerChunk;
  const int lane_run = frag / 4;
  Params pp;
  memset(&pp, 0, sizeof(pp));
  pp.g = p_in;
  GemvParams& p = pp.g;
  Launch l;
  memset(&l, 0, sizeof(l));
  l.bits = bits;
  l.zmode = zmode;
  l.mt = p.m <= 8 ? 1 : (p.m <= 16 ? 2 : 4);
  RB200_CHECK(p.m >= 1 && p.m <= 32, "decode kernel handles 1 <= m <= 32, got m=%d", p.m);
  RB200_CHECK((reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 && p.ldx % 8 == 0,
              "x must be 16-byte aligned with a row pitch that is a multiple of 8 elements");

  if (p.group <= 0 || p.group >= p.k) {
    l.group_code = 0;
  } else {
    RB200_CHECK(p.group % lane_run == 0 && p.k % p.group == 0,
                "group_size=%d must divide k=%d and be a multiple of %d", p.group, p.k, lane_run);
    l.group_code = (p.group == 32 || p.group == 64 || p.group == 128) ? p.group : -1;
  }
  // scales ride the cp.async loader when they have one of the two regular layouts
  l.src = kSrcGlobal;
  const int64_t kg = l.group_code != 0 ? p.k / p.group : 0;
  const bool al = (reinterpret_cast<uintptr_t>(p.s) & 15u) == 0 &&
                  (p.z == nullptr || (reinterpret_cast<uintptr_t>(p.z) & 15u) == 0);
  if (l.group_code > 0 && al) {
    if (p.s_g == 1 && p.s_n == kg && bits == 4 && p.group == 32 && (kg * 2) % 16 == 0) l.src = kSrcSmemNK;
    else if (p.s_n == 1 && p.s_g == p.n && chunk % p.group == 0 && p.n % 8 == 0) l.src = kSrcSmemKN;
  }
  if (l.src != kSrcGlobal && zmode == kZeroGeneral && p.z) pp.has_z_tile = 1;

  const int cpt = (p.k + chunk - 1) / chunk;
  const int n_tiles = (p.n + kTileRows - 1) / kTileRows;
  p.chunks_per_tile = cpt;
  p.total_iters = (long long)cpt * n_tiles;

  const int ctas_per_sm = 2;
  const int xpitch = chunk * 2 + (bits == 4 ? 16 : 64);
  size_t sb = (size_t)kConsumerWarps * kBlocksPerChunk * kTileBytes + (size_t)((l.mt * 8 * xpitch + 127) / 128) * 128;
  if (l.src != kSrcGlobal) sb += kScaleBoxBytes * (zmode == kZeroGeneral ? 2 : 1);
  const size_t budget = (size_t)(228 * 1024) / ctas_per_sm - 1024;
  int stages = (int)((budget - 512) / sb);
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  p.stages = stages;
  l.smem_bytes = (size_t)stages * sb + (size_t)stages * 2 * sizeof(uint64_t);
  long long grid = (long long)sm_count * ctas_per_sm;
  if (grid > p.total_iters) grid = p.total_iters;
  l.grid = (int)grid;

  const size_t need = (size_t)l.grid * 2 * kConsumerWarps * l.mt * 128 * sizeof(float);
  RB200_CHECK(partial_bytes >= need && flag_count >= (size_t)l.grid * kConsumerWarps,
              "split-k scratch too small: need %zu bytes and %d flags", need, l.grid * kConsumerWarps);
  pp.partial = partial;
  pp.flags = flags;
  pp.wait_limit_ms = wait_limit_ms();
  if (bits == 4) return launch_sk_i4(pp, l, stream);
  return launch_sk_i8(pp, l, stream);
}

}  // namespace rb200
