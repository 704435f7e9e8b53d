// Host side of the stream-k decode kernel: scale staging mode, pipeline depth, grid, launch.
#include "gemv_sk.cuh"

#include "tensormap.h"

#include <cstdlib>
#include <cstring>

namespace rb200 {

int gemv_sk_run(const GemvParams& p_in, int bits, int zmode, int sm_count, float* partial, size_t partial_bytes,
                unsigned* flags, size_t flag_count, const sk::ArCtx* ar, const sk::GroupCtx* grp, cudaStream_t stream) {
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
  const int x_blocks = chunk / 64;
  size_t sb = (size_t)kConsumerWarps * kBlocksPerChunk * kTileBytes + (size_t)x_blocks * l.mt * 8 * 128;
  if (l.src != kSrcGlobal) sb += kScaleBoxBytes * (zmode == kZeroGeneral ? 2 : 1);
  const size_t budget = (size_t)(228 * 1024) / ctas_per_sm - 1024;
  int stages = (int)((budget - 1024 - 512) / sb);
  if (stages > sk::kConsumerWarps) stages = sk::kConsumerWarps;  // one consumer warp starts each stage
  if (stages < 2) stages = 2;
  p.stages = stages;
  l.smem_bytes = 1024 + (size_t)stages * sb + (size_t)(stages + 1) * 2 * sizeof(uint64_t);  // 1 KB: alignment slack
  // self-test with several ranks in one launch: every rank gets an equal share of the SMs
  const int emulate = (ar && ar->world > 1 && ar->emulate > 1) ? ar->emulate : 1;
  RB200_CHECK(emulate == 1 || emulate == ar->world, "emulate=%d must equal world=%d", emulate, ar ? ar->world : 0);
  long long grid = (long long)(sm_count / emulate) * ctas_per_sm;
  if (grid > p.total_iters) grid = p.total_iters;
  RB200_CHECK(grid >= 1, "no SMs left per emulated rank");
  RB200_CHECK(p.total_iters * grid < (1ll << 31), "problem too large for the decode kernel's 32-bit work split");
  l.grid = (int)grid * emulate;
  l.cooperative = emulate > 1 ? 1 : 0;

  const size_t need = (size_t)l.grid * 2 * kConsumerWarps * l.mt * 128 * sizeof(float);
  RB200_CHECK(partial_bytes >= need && flag_count >= (size_t)l.grid * kConsumerWarps,
              "split-k scratch too small: need %zu bytes and %d flags", need, l.grid * kConsumerWarps);
  pp.partial = partial;
  pp.flags = flags;
  pp.wait_limit_ms = wait_limit_ms();
  if (grp) {
    RB200_CHECK(!(ar && ar->world > 1), "the grouped form has no all-reduce epilogue");
    pp.grp = *grp;
  }
  if (ar && ar->world > 1) {
    RB200_CHECK(ar->world <= kArMaxRanks && ar->rank >= 0 && ar->rank < ar->world, "bad all-reduce rank %d / world %d",
                ar->rank, ar->world);
    RB200_CHECK((unsigned)(p.n / 16) <= ar->max_blocks, "n=%d exceeds the all-reduce workspace (room for n <= %u)", p.n,
                ar->max_blocks * 16);
    RB200_CHECK(p.epi.act != kActSwiglu, "the fused gate/up activation cannot be combined with the all-reduce epilogue");
    pp.ar = *ar;
  }

  // tensor maps: x as [64-k block][row][64 k] (rows past m and blocks past k read as zero), the
  // scale / zero tensors as 2-D tiles when they are staged
  RB200_CHECK(p.k % 64 == 0, "the stream-k decode kernel needs k %% 64 == 0 (k=%d)", p.k);
  CUtensorMap tx, ts, tz;
  {
    const unsigned long long dims[3] = {64ull, (unsigned long long)p.m, (unsigned long long)(p.k / 64)};
    const unsigned long long strides[2] = {(unsigned long long)p.ldx * 2ull, 128ull};
    const unsigned box[3] = {64u, (unsigned)(l.mt * 8), (unsigned)x_blocks};
    if (make_tensor_map(&tx, p.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
      return -1;
  }
  ts = tx;
  tz = tx;
  pp.s_box_bytes = 0;
  if (l.src == kSrcSmemNK) {
    if (make_tensor_map_2d(&ts, p.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, kg, p.n, kg * 2, 8, kTileRows,
                           CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
    pp.s_box_bytes = 8 * kTileRows * 2;
    if (pp.has_z_tile && make_tensor_map_2d(&tz, p.z, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, kg, p.n, kg * 2, 8, kTileRows,
                                            CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
  } else if (l.src == kSrcSmemKN) {
    const unsigned gpc = (unsigned)(chunk / p.group);
    if (make_tensor_map_2d(&ts, p.s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.n, kg, (unsigned long long)p.n * 2, kTileRows,
                           gpc, CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
    pp.s_box_bytes = gpc * kTileRows * 2;
    if (pp.has_z_tile && make_tensor_map_2d(&tz, p.z, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.n, kg,
                                            (unsigned long long)p.n * 2, kTileRows, gpc, CU_TENSOR_MAP_SWIZZLE_NONE) != 0)
      return -1;
  }
  if (bits == 4) return launch_sk_i4(pp, l, tx, ts, tz, stream);
  return launch_sk_i8(pp, l, tx, ts, tz, stream);
}

}  // namespace rb200
