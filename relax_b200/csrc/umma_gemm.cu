// Host side of the tcgen05 prefill kernel: coverage test, tile plan, x tensor map, dispatch.
#include "umma_gemm.cuh"

#include <cstdlib>
#include <cstring>

#include "tensormap.h"

namespace rb200 {

static int run_common(const GemvParams& p_in, int bits, int zmode, int sm_count, const int64_t* indptr,
                      int indptr_has_prev, int num_experts, int64_t w_expert_bytes, int64_t s_expert_stride, bool grouped,
                      cudaStream_t stream) {
  using namespace um;
  // coverage: whole 128-row tiles, whole 64-k blocks, TMA-loadable x, 16-byte row stores
  const bool covered = p_in.n % kTileRows == 0 && p_in.k % kKBlock == 0 &&
                       (reinterpret_cast<uintptr_t>(p_in.x) & 15u) == 0 && (p_in.ldx * 2) % 16 == 0 &&
                       (reinterpret_cast<uintptr_t>(p_in.out) & 15u) == 0 && (p_in.ldo * 2) % 16 == 0;
  if (!covered) {
    RB200_CHECK(!grouped, "grouped GEMM needs n %% 128 == 0, k %% 64 == 0 and 16-byte aligned x / out rows "
                "(n=%d, k=%d)", p_in.n, p_in.k);
    return 1;
  }
  RB200_CHECK(num_experts >= 1 && num_experts <= kMaxExperts, "num_experts=%d outside [1, %d]", num_experts,
              kMaxExperts);

  Params pp;
  memset(&pp, 0, sizeof(pp));
  pp.g = p_in;
  GemvParams& p = pp.g;
  pp.indptr = indptr;
  pp.indptr_has_prev = indptr_has_prev;
  pp.num_experts = num_experts;
  pp.w_expert_bytes = w_expert_bytes;
  pp.s_expert_stride = s_expert_stride;
  if (grouped) {
    // The split of the rows is known only on the device.  One tcgen05.mma occupies the tensor
    // pipe for the same time at any N up to 192 and 26 % longer at 256, so the tile is as wide
    // as an expert's share is likely to be: 128 or 192 batch rows when the rows, spread evenly
    // over the experts, stay well inside that (an expert above the width takes a second tile),
    // 256 otherwise.
    const long long even = p.m / num_experts;
    if (p.m < kMaxNb) pp.nb = (p.m + 31) / 32 * 32;
    else pp.nb = even <= 96 ? 128 : (even <= 160 ? 192 : kMaxNb);
  } else {
    // balanced batch tiles of at most 256 rows, padded to the 32 rows the epilogue split needs
    const int m_tiles = (p.m + kMaxNb - 1) / kMaxNb;
    pp.nb = (((p.m + m_tiles - 1) / m_tiles) + 31) / 32 * 32;
  }

  Launch l;
  l.zmode = zmode;
  l.src = ug::kSrcGlobal;
  l.group_code = 0;
  if (bits != 16) {
    if (p.group <= 0 || p.group >= p.k) {
      l.group_code = 0;
    } else {
      RB200_CHECK(p.group % 16 == 0 && p.k % p.group == 0,
                  "group_size=%d must divide k=%d and be a multiple of 16", p.group, p.k);
      l.group_code = (bits == 4 && (p.group == 32 || p.group == 64 || p.group == 128)) ? p.group : -1;
    }
    const int64_t kg = l.group_code != 0 ? p.k / p.group : 0;
    const bool al = (reinterpret_cast<uintptr_t>(p.s) & 15u) == 0 &&
                    (p.z == nullptr || (reinterpret_cast<uintptr_t>(p.z) & 15u) == 0) &&
                    (s_expert_stride * 2) % 16 == 0;
    if (bits == 4 && l.group_code > 0 && al) {
      if (p.s_g == 1 && p.s_n == kg && p.group == 32 && (kg * 2) % 16 == 0) l.src = ug::kSrcSmemNK;
      else if (p.s_n == 1 && p.s_g == p.n && (p.n * 2) % 16 == 0) l.src = ug::kSrcSmemKN;
    }
    if (l.src != ug::kSrcGlobal && zmode == kZeroGeneral && p.z) pp.has_z_tile = 1;
    RB200_CHECK(p.s_n != 0 && s_expert_stride % p.s_n == 0, "expert stride of the scales must be a multiple of their row stride");
  }

  long long grid = sm_count;  // one persistent CTA per SM (a tensor-memory kernel gets occupancy 1)
  pp.k_splits = 1;
  if (!grouped) {
    const long long tiles = (long long)(p.n / kTileRows) * ((p.m + pp.nb - 1) / pp.nb);
    // fewer tiles than half the SMs: cut k, in whole weight stages, so that the idle SMs take part
    const int kb_total = p.k / kKBlock;
    const int blocks_per_chunk = bits == 16 ? 1 : (bits == 4 ? 4 : 2);
    int split = (int)(sm_count / tiles);
    if (split > 8) split = 8;
    if (split > sm_count / tiles) split = (int)(sm_count / tiles);
    const int chunks = (kb_total + blocks_per_chunk - 1) / blocks_per_chunk;
    while (split > 1 && chunks / split * blocks_per_chunk < 8) --split;  // every split at least 8 MMA blocks
    if (split > 1 && tiles * split <= sm_count) {
      const size_t need = (size_t)tiles * split * pp.nb * kTileRows * sizeof(float);
      DeviceScratch* sc = device_scratch(need, (size_t)tiles * 2);
      if (!sc) return -1;
      pp.k_splits = split;
      pp.partial = sc->partials;
      pp.tickets = sc->counters;
    }
    if (grid > tiles * pp.k_splits) grid = tiles * pp.k_splits;
  }
  l.grid = (int)grid;

  const size_t budget = (size_t)227 * 1024;
  int xs = kMaxXStages;
  while (xs > 2 && smem_bytes(pp.nb, xs) > budget) --xs;
  pp.x_stages = xs;
  l.smem = smem_bytes(pp.nb, xs);

  CUtensorMap tx;
  if (make_tensor_map_2d(&tx, p.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (unsigned long long)p.k,
                         (unsigned long long)p.m, (unsigned long long)p.ldx * 2, kKBlock, (unsigned)pp.nb,
                         CU_TENSOR_MAP_SWIZZLE_128B) != 0)
    return -1;

  if (bits == 16) {
    CUtensorMap tw;
    const unsigned long long dims[3] = {(unsigned long long)p.k, (unsigned long long)p.n, (unsigned long long)num_experts};
    const unsigned long long strides[2] = {(unsigned long long)p.k * 2, (unsigned long long)w_expert_bytes};
    const unsigned box[3] = {kKBlock, kTileRows, 1};
    if (make_tensor_map(&tw, p.w, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B) != 0)
      return -1;
    return launch_gemm_f16(pp, l, tx, tw, stream);
  }
  if (bits == 4) {
    if (zmode == kZeroConstInt) return launch_gemm_i4c(pp, l, tx, stream);
    return launch_gemm_i4g(pp, l, tx, stream);
  }
  return launch_gemm_i8(pp, l, tx, stream);
}

int umma_gemm_run(const GemvParams& p, int bits, int zmode, int sm_count, cudaStream_t stream) {
  return run_common(p, bits, zmode, sm_count, nullptr, 0, 1, 0, 0, false, stream);
}

int umma_group_gemm_run(const GemvParams& p, int bits, int zmode, int sm_count, const int64_t* indptr,
                        int indptr_has_prev, int num_experts, int64_t w_expert_bytes, int64_t s_expert_stride,
                        cudaStream_t stream) {
  RB200_CHECK(indptr != nullptr, "indptr must be non-NULL");
  return run_common(p, bits, zmode, sm_count, indptr, indptr_has_prev, num_experts, w_expert_bytes, s_expert_stride, true,
                    stream);
}

}  // namespace rb200
