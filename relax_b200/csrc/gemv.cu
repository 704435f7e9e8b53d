// Decode-path kernel: out[m, n] = epilogue( sum_k x[m, k] * wq[n, k] ) for m <= 32.
//
// The weight stream is the only large operand, so the kernel is organised around keeping HBM
// busy: a producer warp stages 16 KB weight tiles (plus the matching x slice) into a ring of
// shared-memory stages with bulk async copies; eight consumer warps each own one 16-row block
// of the CTA's 128-row tile, read their 128-bit fragment-ordered weight words, decode them in
// registers (lop3/prmt + exact fp16 ops) and feed m16n8k16 MMAs that accumulate in fp32.
// The iteration space (n-tile, k-chunk) is cut into equal contiguous ranges, one per CTA, so
// every CTA streams the same number of bytes whatever N and K are; a tile whose k-range is
// shared by several CTAs is finished by the last of them to arrive (ticket counter), which
// adds the fp32 partials in CTA order - deterministic - and applies the epilogue.
//
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at small m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and for the reference's own
// GEMV / LowBatchGEMV schedules (python/tvm/dlight/gpu/gemv.py:216-530, low_batch_gemv.py:300-613).
#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileRows = kConsumerWarps * 16;  // 128 output rows per CTA tile
constexpr int kBlocksPerChunk = 4;              // fragment k-blocks per stage
constexpr int kTileBytes = 512;

template <int BITS>
struct Geo {
  static constexpr int kFrag = BITS == 4 ? 64 : 32;          // k per fragment tile
  static constexpr int kChunk = kFrag * kBlocksPerChunk;     // k per stage (256 / 128)
  static constexpr int kXPitch = kChunk * 2 + (BITS == 4 ? 16 : 64);  // bytes, bank-conflict free
  static constexpr int kWBytes = kConsumerWarps * kBlocksPerChunk * kTileBytes;  // 16 KB
};

template <int BITS, int MT>
struct StageBytes {
  static constexpr int value = Geo<BITS>::kWBytes + ((MT * 8 * Geo<BITS>::kXPitch + 127) / 128) * 128;
};

__device__ __forceinline__ long long range_start(long long cta, long long total, long long grid) {
  return cta * total / grid;
}

// GROUP: 32 / 64 / 128 compile-time group sizes, 0 = one scale per output channel, -1 = any
// group size given at run time (a multiple of the per-lane run of 16 (int4) / 8 (int8) k).
template <int BITS, int GROUP>
struct ScalePlan {
  static constexpr int kFrag = Geo<BITS>::kFrag;
  static constexpr int kChunk = Geo<BITS>::kChunk;
  // k extent covered by one fetched scale (per lane)
  static constexpr int kSpan = GROUP == 0 ? kChunk : (GROUP < 0 ? kFrag : (GROUP > kChunk ? kChunk : (GROUP < kFrag ? kFrag : GROUP)));
  static constexpr int kCount = kChunk / kSpan;  // scale fetches per row per stage
};

template <int BITS, int MT, int ZMODE, int GROUP>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvParams p) {
  using G = Geo<BITS>;
  using SP = ScalePlan<BITS, GROUP>;
  constexpr int kStage = StageBytes<BITS, MT>::value;
  extern __shared__ __align__(128) uint8_t smem[];

  const int stages = p.stages;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStage);
  uint64_t* empty_bar = full_bar + stages;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // zero the x regions once: rows >= m are never written again and must read as 0
  for (int s = 0; s < stages; ++s) {
    uint32_t* xs = reinterpret_cast<uint32_t*>(smem + (size_t)s * kStage + G::kWBytes);
    for (int i = tid; i < (kStage - G::kWBytes) / 4; i += kThreads) xs[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    mbar_fence_init();
  }
  fence_proxy_async();
  __syncthreads();

  const long long total = p.total_iters;
  const long long grid = gridDim.x;
  const long long it0 = range_start(blockIdx.x, total, grid);
  const long long it1 = range_start(blockIdx.x + 1, total, grid);
  const int cpt = p.chunks_per_tile;
  const int kb_total = p.k / G::kFrag;  // fragment k-blocks per row block
  const int n_blocks = p.n / 16;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer warp
    int stage = 0;
    uint32_t phase = 0;
    long long tile = it0 / cpt;
    int chunk = (int)(it0 % cpt);
    for (long long it = it0; it < it1; ++it) {
      if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, p.status)) break;
      const int kb0 = chunk * kBlocksPerChunk;
      const int nkb = min(kBlocksPerChunk, kb_total - kb0);
      const int blk0 = (int)tile * kConsumerWarps;
      const int nblk = min(kConsumerWarps, n_blocks - blk0);
      uint8_t* sbase = smem + (size_t)stage * kStage;
      const uint32_t wbytes = (uint32_t)nkb * kTileBytes * nblk;  // one contiguous run per stage
      const uint32_t xbytes = (uint32_t)nkb * G::kFrag * 2;
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], wbytes + xbytes * p.m);
      __syncwarp();
      if (lane == 0) {
        const uint8_t* src = p.w + frag_stage_offset(tile, chunk, n_blocks, kb_total);
        bulk_g2s(sbase, src, wbytes, &full_bar[stage]);
      }
      for (int r = lane; r < p.m; r += 32) {
        const __half* src = p.x + (size_t)r * p.ldx + (size_t)kb0 * G::kFrag;
        bulk_g2s(sbase + G::kWBytes + r * G::kXPitch, src, xbytes, &full_bar[stage]);
      }
      if (++chunk == cpt) {
        chunk = 0;
        ++tile;
      }
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int t = lane & 3;
  const ZeroConsts zc = make_zero_consts(ZMODE, p.zero_const);
  const uint32_t zconst_h2 = h2_bcast(__float2half_rn(p.zero_const));
  const int group = GROUP > 0 ? GROUP : (GROUP == 0 ? p.k : p.group);
  const int lane_k = t * (G::kFrag / 4);  // first k of this lane inside a fragment tile

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // packed scale (and zero) registers for one stage: low half = row g, high half = row g+8
  uint32_t s_cur[SP::kCount], s_nxt[SP::kCount];
  uint32_t z_cur[SP::kCount], z_nxt[SP::kCount];

  auto fetch_scales = [&](long long tile_i, int chunk_i, uint32_t (&sv)[SP::kCount],
                          uint32_t (&zv)[SP::kCount]) {
    const int blk = (int)tile_i * kConsumerWarps + warp;
    if (blk >= n_blocks) return;
    const int64_t n_g = (int64_t)blk * 16 + g;
#pragma unroll
    for (int i = 0; i < SP::kCount; ++i) {
      int k = chunk_i * G::kChunk + i * SP::kSpan + (SP::kSpan == G::kFrag ? lane_k : 0);
      if (k >= p.k) k = p.k - 1;  // tail chunk: value unused
      const int64_t grp = GROUP == 0 ? 0 : k / group;
      const int64_t o_g = n_g * p.s_n + grp * p.s_g;
      const int64_t o_g8 = o_g + 8 * p.s_n;
      sv[i] = ld_nc_u16(p.s + o_g) | (ld_nc_u16(p.s + o_g8) << 16);
      if (ZMODE == kZeroGeneral) {
        zv[i] = p.z ? (ld_nc_u16(p.z + o_g) | (ld_nc_u16(p.z + o_g8) << 16)) : 0u;
      }
    }
  };

  int stage = 0;
  uint32_t phase = 0;
  long long tile = it0 / cpt;
  int chunk = (int)(it0 % cpt);
  int seg_first_chunk = chunk;  // first chunk of the segment being accumulated
  bool first_segment = true;

  if (it0 < it1) fetch_scales(tile, chunk, s_nxt, z_nxt);

  for (long long it = it0; it < it1; ++it) {
#pragma unroll
    for (int i = 0; i < SP::kCount; ++i) {
      s_cur[i] = s_nxt[i];
      z_cur[i] = z_nxt[i];
    }
    // prefetch the next stage's scales before waiting on this stage's data
    {
      long long ntile = tile;
      int nchunk = chunk + 1;
      if (nchunk == cpt) {
        nchunk = 0;
        ++ntile;
      }
      if (it + 1 < it1) fetch_scales(ntile, nchunk, s_nxt, z_nxt);
    }

    if (!mbar_wait_bounded(&full_bar[stage], phase, p.status)) return;

    const int kb0 = chunk * kBlocksPerChunk;
    const int nkb = min(kBlocksPerChunk, kb_total - kb0);
    const int blk = (int)tile * kConsumerWarps + warp;
    const uint8_t* sbase = smem + (size_t)stage * kStage;
    if (blk < n_blocks) {
      const uint4* wsm = reinterpret_cast<const uint4*>(sbase + warp * (nkb * kTileBytes));
      const uint8_t* xsm = sbase + G::kWBytes + g * G::kXPitch + t * (G::kFrag / 2);
#pragma unroll
      for (int kb = 0; kb < kBlocksPerChunk; ++kb) {
        if (kb < nkb) {
          const uint4 wv = wsm[kb * 32 + frag_unit_pos(lane)];
          constexpr int si_div = SP::kSpan / G::kFrag;  // fragment tiles per fetched scale
          const uint32_t sp = s_cur[kb / si_div];
          const uint32_t s_g = prmt(sp, sp, 0x1010u);
          const uint32_t s_g8 = prmt(sp, sp, 0x3232u);
          uint32_t z_g = zconst_h2, z_g8 = zconst_h2;
          if (ZMODE == kZeroGeneral && p.z) {
            const uint32_t zp = z_cur[kb / si_div];
            z_g = prmt(zp, zp, 0x1010u);
            z_g8 = prmt(zp, zp, 0x3232u);
          }
          if (BITS == 4) {
            uint4 xv[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const uint4* xp = reinterpret_cast<const uint4*>(xsm + mt * 8 * G::kXPitch + kb * 128);
              xv[mt][0] = xp[0];
              xv[mt][1] = xp[1];
            }
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t a[4];
              decode_int4_word<ZMODE>(ww[j], zc, s_g, s_g8, z_g, z_g8, a);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const uint4& xr = xv[mt][j >> 1];
                const uint32_t b0 = (j & 1) ? xr.z : xr.x;
                const uint32_t b1 = (j & 1) ? xr.w : xr.y;
                mma_16816(acc[mt], a, b0, b1);
              }
            }
          } else {
            uint4 xv[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              xv[mt] = *reinterpret_cast<const uint4*>(xsm + mt * 8 * G::kXPitch + kb * 64);
            uint32_t a[4];
            decode_int8_pair<ZMODE>(wv.x, wv.y, zc, s_g, s_g8, z_g, z_g8, a);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_16816(acc[mt], a, xv[mt].x, xv[mt].y);
            decode_int8_pair<ZMODE>(wv.z, wv.w, zc, s_g, s_g8, z_g, z_g8, a);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_16816(acc[mt], a, xv[mt].z, xv[mt].w);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);

    const bool tile_end = (chunk + 1 == cpt);
    if (tile_end || it + 1 == it1) {
      // ---------------------------------------------------------- finish a segment
      if (blk < n_blocks) {
        const bool whole = (seg_first_chunk == 0) && tile_end;
        bool do_store = whole;
        if (!whole) {
          const int slot = (int)blockIdx.x * 2 + (first_segment ? 0 : 1);
          float* dst = p.partial + ((size_t)(slot * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = acc[mt][c];
          __threadfence();
          __syncwarp();
          // contributors of this tile: CTAs whose range meets [tile*cpt, (tile+1)*cpt)
          const long long lo_it = tile * cpt;
          const long long hi_it = lo_it + cpt - 1;
          const int first_cta = (int)(((lo_it + 1) * grid - 1) / total);
          const int last_cta = (int)(((hi_it + 1) * grid - 1) / total);
          int ticket = 0;
          if (lane == 0) ticket = atomicAdd(&p.counters[blk], 1);
          ticket = __shfl_sync(0xffffffffu, ticket, 0);
          if (ticket == last_cta - first_cta) {
            __threadfence();
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
            for (int c_id = first_cta; c_id <= last_cta; ++c_id) {
              const long long cs = range_start(c_id, total, grid);
              const int sl = c_id * 2 + ((cs / cpt) == tile ? 0 : 1);
              const float* src = p.partial + ((size_t)(sl * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[mt][c] += __ldcg(src + mt * 128 + c * 32);
            }
            if (lane == 0) p.counters[blk] = 0;  // ready for the next launch
            do_store = true;
          }
        }
        if (do_store) {
          const int64_t n0 = (int64_t)blk * 16 + g;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int64_t m = mt * 8 + t * 2 + (c & 1);
              const int64_t n = n0 + (c >> 1) * 8;
              if (m < p.m) p.out[m * p.ldo + n] = __float2half_rn(apply_epilogue(acc[mt][c], p.epi, m, n));
            }
          }
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][c] = 0.0f;
      first_segment = false;
      seg_first_chunk = 0;
    }

    if (++chunk == cpt) {
      chunk = 0;
      ++tile;
    }
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
  }
}

template <int BITS, int MT, int ZMODE, int GROUP>
int launch_one(const GemvParams& p, int grid, size_t smem, cudaStream_t stream) {
  auto kern = gemv_kernel<BITS, MT, ZMODE, GROUP>;
  static thread_local int configured_device = -1;
  int dev = 0;
  RB200_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    RB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  kern<<<grid, kThreads, smem, stream>>>(p);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

template <int BITS, int MT, int ZMODE>
int launch_group(const GemvParams& p, int group_code, int grid, size_t smem, cudaStream_t stream) {
  switch (group_code) {
    case 32:
      return launch_one<BITS, MT, ZMODE, 32>(p, grid, smem, stream);
    case 64:
      return launch_one<BITS, MT, ZMODE, 64>(p, grid, smem, stream);
    case 128:
      return launch_one<BITS, MT, ZMODE, 128>(p, grid, smem, stream);
    case 0:
      return launch_one<BITS, MT, ZMODE, 0>(p, grid, smem, stream);
    default:
      return launch_one<BITS, MT, ZMODE, -1>(p, grid, smem, stream);
  }
}

template <int BITS, int MT>
int launch_zmode(const GemvParams& p, int zmode, int group_code, int grid, size_t smem,
                 cudaStream_t stream) {
  if (zmode == kZeroConstInt) return launch_group<BITS, MT, kZeroConstInt>(p, group_code, grid, smem, stream);
  return launch_group<BITS, MT, kZeroGeneral>(p, group_code, grid, smem, stream);
}

template <int BITS>
int launch_mt(const GemvParams& p, int mt, int zmode, int group_code, int grid, size_t smem,
              cudaStream_t stream) {
  switch (mt) {
    case 1:
      return launch_zmode<BITS, 1>(p, zmode, group_code, grid, smem, stream);
    case 2:
      return launch_zmode<BITS, 2>(p, zmode, group_code, grid, smem, stream);
    default:
      return launch_zmode<BITS, 4>(p, zmode, group_code, grid, smem, stream);
  }
}

template <int BITS>
size_t stage_bytes_rt(int mt) {
  return mt == 1 ? StageBytes<BITS, 1>::value : (mt == 2 ? StageBytes<BITS, 2>::value : StageBytes<BITS, 4>::value);
}

}  // namespace

int gemv_plan(int bits, int m, int n, int k, int sm_count, int ctas_per_sm_hint, int stages_hint,
              GemvPlan* plan) {
  const int frag = bits == 4 ? 64 : 32;
  RB200_CHECK(m >= 1 && m <= 32, "decode kernel handles 1 <= m <= 32, got m=%d", m);
  RB200_CHECK(n % 16 == 0, "n=%d must be a multiple of 16", n);
  RB200_CHECK(k % frag == 0, "k=%d must be a multiple of %d for %d-bit weights", k, frag, bits);
  plan->mt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
  const int chunk = frag * kBlocksPerChunk;
  plan->chunks_per_tile = (k + chunk - 1) / chunk;
  plan->n_tiles = (n + kTileRows - 1) / kTileRows;
  plan->total_iters = (long long)plan->n_tiles * plan->chunks_per_tile;
  const size_t sb = bits == 4 ? stage_bytes_rt<4>(plan->mt) : stage_bytes_rt<8>(plan->mt);
  int ctas_per_sm = ctas_per_sm_hint > 0 ? ctas_per_sm_hint : 2;
  // stages: fill the per-SM shared memory budget (about 220 KB across resident CTAs)
  const size_t budget = (size_t)(228 * 1024) / ctas_per_sm - 1024;  // 1 KB per CTA is reserved
  int stages = (int)((budget - 256) / sb);
  if (stages_hint > 0) stages = stages_hint;
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  plan->stages = stages;
  plan->smem_bytes = (size_t)stages * sb + (size_t)stages * 2 * sizeof(uint64_t);
  long long grid = (long long)sm_count * ctas_per_sm;
  if (grid > plan->total_iters) grid = plan->total_iters;
  plan->grid = (int)grid;
  plan->partial_bytes = (size_t)plan->grid * 2 * kConsumerWarps * plan->mt * 128 * sizeof(float);
  plan->counter_ints = (size_t)(n / 16);
  return 0;
}

int gemv_launch(const GemvParams& p_in, const GemvPlan& plan, int bits, int zmode, cudaStream_t stream) {
  GemvParams p = p_in;
  p.stages = plan.stages;
  p.chunks_per_tile = plan.chunks_per_tile;
  p.total_iters = plan.total_iters;
  const int lane_run = (bits == 4 ? 64 : 32) / 4;
  int group_code;
  if (p.group <= 0 || p.group >= p.k) {
    group_code = 0;
  } else {
    RB200_CHECK(p.group % lane_run == 0 && p.k % p.group == 0,
                "group_size=%d must divide k=%d and be a multiple of %d", p.group, p.k, lane_run);
    group_code = (p.group == 32 || p.group == 64 || p.group == 128) ? p.group : -1;
  }
  if (bits == 4) return launch_mt<4>(p, plan.mt, zmode, group_code, plan.grid, plan.smem_bytes, stream);
  return launch_mt<8>(p, plan.mt, zmode, group_code, plan.grid, plan.smem_bytes, stream);
}

}  // namespace rb200
