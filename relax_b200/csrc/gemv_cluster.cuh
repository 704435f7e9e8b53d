// Decode-path kernel, cluster variant (the default for m <= 32).
//
// Same streaming structure as gemv.cu - a producer warp fills a ring of shared-memory stages
// with bulk async copies, eight consumer warps decode 128-bit fragment words in registers and
// issue m16n8k16 MMAs with fp32 accumulators - with three differences that the profile of the
// first version asked for:
//   * split-k runs inside persistent thread-block clusters: the S CTAs of a cluster walk the
//     128-row tiles together, each streaming 1/S of a tile's k-chunks; partial fragments are
//     published in the CTA's own shared memory and summed through distributed shared memory by
//     a leader that rotates from tile to tile.  Hand-off is two mbarriers per CTA ("partials of
//     all ranks are ready" at the leader, "your partials were consumed" at each rank) with
//     cluster-scope release/acquire, so the bulk-copy pipeline never drains between tiles and no
//     global memory, fence or ticket is involved;
//   * scales and zero points ride the same asynchronous pipeline (one TMA tile per stage) when
//     their layout allows it, so no consumer waits on a global load;
//   * each m-tile accumulates into two independent fragment chains, halving the MMA dependency
//     chain.
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at small m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and the reference's GEMV / LowBatchGEMV
// schedules (python/tvm/dlight/gpu/gemv.py:216-530, low_batch_gemv.py:300-613).
#pragma once

#include <cuda.h>

#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace gc {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileRows = kConsumerWarps * 16;
constexpr int kBlocksPerChunk = 4;
constexpr int kTileBytes = 512;
constexpr int kScaleBoxBytes = 2048;  // one staged scale (or zero) tile

// where the consumers get scales / zero points from
enum ScaleSrc : int {
  kSrcGlobal = 0,   // direct global loads, any layout (strides) and group size
  kSrcSmemNK = 1,   // staged [128 rows][8 groups] from a [N, K/32] tensor (int4, group 32)
  kSrcSmemKN = 2,   // staged [groups][128 rows] from a [K/g, N] tensor (g in 32/64/128)
};

template <int BITS>
struct Geo {
  static constexpr int kFrag = BITS == 4 ? 64 : 32;
  static constexpr int kChunk = kFrag * kBlocksPerChunk;
  static constexpr int kXPitch = kChunk * 2 + (BITS == 4 ? 16 : 64);
  static constexpr int kWBytes = kConsumerWarps * kBlocksPerChunk * kTileBytes;
};

template <int BITS, int MT, int ZMODE, int SRC>
struct StageLayout {
  static constexpr int kXBytes = ((MT * 8 * Geo<BITS>::kXPitch + 127) / 128) * 128;
  static constexpr int kSOff = Geo<BITS>::kWBytes + kXBytes;
  static constexpr int kSBytes = SRC == kSrcGlobal ? 0 : kScaleBoxBytes;
  static constexpr int kZOff = kSOff + kSBytes;
  static constexpr int kZBytes = (SRC != kSrcGlobal && ZMODE == kZeroGeneral) ? kScaleBoxBytes : 0;
  static constexpr int kBytes = kZOff + kZBytes;
};

struct ClusterParams {
  GemvParams g;
  int split;           // cluster size S (1..8)
  int has_z_tile;      // zero points staged through shared memory
  unsigned s_box_bytes;  // bytes one scale TMA delivers
};

#ifdef __CUDACC__

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// arrive on an mbarrier that lives in another CTA of the cluster (address from map_to_rank)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (clock64() - t0 > (1ll << 31)) {
      if (status) atomicExch(status, kStatusWaitTimeout);
      return false;
    }
  }
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

template <int BITS, int GROUP>
struct ScalePlan {
  static constexpr int kFrag = Geo<BITS>::kFrag;
  static constexpr int kChunk = Geo<BITS>::kChunk;
  static constexpr int kSpan =
      GROUP == 0 ? kChunk : (GROUP < 0 ? kFrag : (GROUP > kChunk ? kChunk : (GROUP < kFrag ? kFrag : GROUP)));
  static constexpr int kCount = kChunk / kSpan;
};

template <int BITS, int MT, int ZMODE, int GROUP, int SRC>
__global__ void __launch_bounds__(kThreads, 2)
    gemv_cluster_kernel(const ClusterParams cp, const __grid_constant__ CUtensorMap tmap_s,
                        const __grid_constant__ CUtensorMap tmap_z) {
  using G = Geo<BITS>;
  using L = StageLayout<BITS, MT, ZMODE, SRC>;
  using SP = ScalePlan<BITS, GROUP>;
  constexpr int kStage = L::kBytes;
  extern __shared__ __align__(128) uint8_t smem[];
  const GemvParams& p = cp.g;

  const int stages = p.stages;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int S = cp.split;
  // [stages][kStage] | partial fragments red[2][8 warps][MT][4][32] fp32 | mbarriers
  constexpr int kRedFloats = kConsumerWarps * MT * 128;  // one buffer
  float* red = reinterpret_cast<float*>(smem + (size_t)stages * kStage);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStage + 2 * kRedFloats * 4);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* ready_bar = empty_bar + stages;  // [1]  leader side: every rank's warps published
  uint64_t* free_bar = ready_bar + 1;        // [2]  per buffer: the leader has summed my partials

  const int rank = S > 1 ? (int)cluster_ctarank() : 0;
  const int cluster_id = blockIdx.x / S;
  const int n_clusters = gridDim.x / S;

  for (int s = 0; s < stages; ++s) {
    uint32_t* xs = reinterpret_cast<uint32_t*>(smem + (size_t)s * kStage + G::kWBytes);
    for (int i = tid; i < L::kXBytes / 4; i += kThreads) xs[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    mbar_init(ready_bar, S * kConsumerWarps);
    mbar_init(&free_bar[0], kConsumerWarps);
    mbar_init(&free_bar[1], kConsumerWarps);
    mbar_fence_init();
  }
  fence_proxy_async();
  __syncthreads();
  if (S > 1) cluster_sync_all();  // peers' mbarriers exist before anyone arrives on them
  griddep_launch_dependents();

  const int cpt = p.chunks_per_tile;
  const int c0 = (int)((long long)rank * cpt / S);
  const int c1 = (int)((long long)(rank + 1) * cpt / S);
  const int kb_total = p.k / G::kFrag;
  const int n_blocks = p.n / 16;
  const int n_tiles = (n_blocks + kConsumerWarps - 1) / kConsumerWarps;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer warp
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    bool dep_waited = false;
    for (int tile = cluster_id; tile < n_tiles && ok; tile += n_clusters) {
      const int blk0 = tile * kConsumerWarps;
      const int nblk = min(kConsumerWarps, n_blocks - blk0);
      for (int chunk = c0; chunk < c1; ++chunk) {
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, p.status)) {
          ok = false;
          break;
        }
        const int kb0 = chunk * kBlocksPerChunk;
        const int nkb = min(kBlocksPerChunk, kb_total - kb0);
        uint8_t* sbase = smem + (size_t)stage * kStage;
        const uint32_t wbytes = (uint32_t)nkb * kTileBytes * nblk;  // one contiguous run per stage
        const uint32_t xbytes = (uint32_t)nkb * G::kFrag * 2;
        uint32_t tx = wbytes + xbytes * p.m;
        if (SRC != kSrcGlobal) tx += cp.s_box_bytes * (cp.has_z_tile ? 2u : 1u);
        if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], tx);
        __syncwarp();
        if (lane == 0) {
          const uint8_t* src = p.w + frag_stage_offset(tile, chunk, n_blocks, kb_total);
          bulk_g2s(sbase, src, wbytes, &full_bar[stage]);
        }
        if (SRC != kSrcGlobal) {
          // coordinates: NK tensor {group, row}; KN tensor {row, group}
          constexpr int kGroupsPerChunk = GROUP > 0 ? (G::kChunk / GROUP) : 1;
          const int gc0 = chunk * kGroupsPerChunk;
          if (lane == 8) {
            if (SRC == kSrcSmemNK) tma_load_2d(sbase + L::kSOff, &tmap_s, gc0, blk0 * 16, &full_bar[stage]);
            else tma_load_2d(sbase + L::kSOff, &tmap_s, blk0 * 16, gc0, &full_bar[stage]);
          }
          if (ZMODE == kZeroGeneral && lane == 9 && cp.has_z_tile) {
            if (SRC == kSrcSmemNK) tma_load_2d(sbase + L::kZOff, &tmap_z, gc0, blk0 * 16, &full_bar[stage]);
            else tma_load_2d(sbase + L::kZOff, &tmap_z, blk0 * 16, gc0, &full_bar[stage]);
          }
        }
        // activations may come from the previous kernel on the stream: read them after it ended
        if (!dep_waited) {
          griddep_wait();
          dep_waited = true;
        }
        for (int r = lane; r < p.m; r += 32) {
          const __half* src = p.x + (size_t)r * p.ldx + (size_t)kb0 * G::kFrag;
          bulk_g2s(sbase + G::kWBytes + r * G::kXPitch, src, xbytes, &full_bar[stage]);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
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
  const int lane_k = t * (G::kFrag / 4);
  const uint32_t half_sel = (t >> 1) ? 0x3232u : 0x1010u;  // which of two packed groups a lane pair uses

  float acc[MT][2][4];
  uint32_t s_cur[SP::kCount], s_nxt[SP::kCount];
  uint32_t z_cur[SP::kCount], z_nxt[SP::kCount];

  int stage = 0;
  uint32_t phase = 0;
  int round = 0;        // tiles this cluster has finished
  int leads_done = 0;   // tiles this CTA has led
  bool ok = true;

  for (int tile = cluster_id; tile < n_tiles && ok; tile += n_clusters, ++round) {
    const int blk = tile * kConsumerWarps + warp;
    const bool active = blk < n_blocks;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][c][j] = 0.0f;

    auto fetch_global = [&](int chunk_i, uint32_t (&sv)[SP::kCount], uint32_t (&zv)[SP::kCount]) {
      if (SRC != kSrcGlobal || !active) return;
      const int64_t n_g = (int64_t)blk * 16 + g;
#pragma unroll
      for (int i = 0; i < SP::kCount; ++i) {
        int k = chunk_i * G::kChunk + i * SP::kSpan + (SP::kSpan == G::kFrag ? lane_k : 0);
        if (k >= p.k) k = p.k - 1;
        const int64_t grp = GROUP == 0 ? 0 : k / group;
        const int64_t o_g = n_g * p.s_n + grp * p.s_g;
        const int64_t o_g8 = o_g + 8 * p.s_n;
        sv[i] = ld_nc_u16(p.s + o_g) | (ld_nc_u16(p.s + o_g8) << 16);
        if (ZMODE == kZeroGeneral) zv[i] = p.z ? (ld_nc_u16(p.z + o_g) | (ld_nc_u16(p.z + o_g8) << 16)) : 0u;
      }
    };
    if (c0 < c1) fetch_global(c0, s_nxt, z_nxt);

    for (int chunk = c0; chunk < c1; ++chunk) {
      if (SRC == kSrcGlobal) {
#pragma unroll
        for (int i = 0; i < SP::kCount; ++i) {
          s_cur[i] = s_nxt[i];
          z_cur[i] = z_nxt[i];
        }
        if (chunk + 1 < c1) fetch_global(chunk + 1, s_nxt, z_nxt);
      }
      if (!mbar_wait_bounded(&full_bar[stage], phase, p.status)) {
        ok = false;
        break;
      }
      const int kb0 = chunk * kBlocksPerChunk;
      const int nkb = min(kBlocksPerChunk, kb_total - kb0);
      const uint8_t* sbase = smem + (size_t)stage * kStage;
      if (active) {
        const uint4* wsm = reinterpret_cast<const uint4*>(sbase + warp * (nkb * kTileBytes));
        const uint8_t* xsm = sbase + G::kWBytes + g * G::kXPitch + t * (G::kFrag / 2);
        // staged scale rows of this lane (kSrcSmemNK: 8 groups of rows g and g+8)
        uint4 nk_s_g, nk_s_g8, nk_z_g, nk_z_g8;
        if (SRC == kSrcSmemNK) {
          const uint4* sp = reinterpret_cast<const uint4*>(sbase + L::kSOff) + warp * 16 + g;
          nk_s_g = sp[0];
          nk_s_g8 = sp[8];
          if (ZMODE == kZeroGeneral && cp.has_z_tile) {
            const uint4* zp = reinterpret_cast<const uint4*>(sbase + L::kZOff) + warp * 16 + g;
            nk_z_g = zp[0];
            nk_z_g8 = zp[8];
          }
        }
#pragma unroll
        for (int kb = 0; kb < kBlocksPerChunk; ++kb) {
          if (kb < nkb) {
            const uint4 wv = wsm[kb * 32 + frag_unit_pos(lane)];
            uint32_t s_g, s_g8, z_g = zconst_h2, z_g8 = zconst_h2;
            if (SRC == kSrcGlobal) {
              constexpr int si_div = SP::kSpan / G::kFrag;
              const uint32_t sp = s_cur[kb / si_div];
              s_g = prmt(sp, sp, 0x1010u);
              s_g8 = prmt(sp, sp, 0x3232u);
              if (ZMODE == kZeroGeneral && p.z) {
                const uint32_t zp = z_cur[kb / si_div];
                z_g = prmt(zp, zp, 0x1010u);
                z_g8 = prmt(zp, zp, 0x3232u);
              }
            } else if (SRC == kSrcSmemNK) {
              // int4, group 32: fragment tile kb holds groups 2kb, 2kb+1 = one 32-bit register
              const uint32_t a = kb == 0 ? nk_s_g.x : (kb == 1 ? nk_s_g.y : (kb == 2 ? nk_s_g.z : nk_s_g.w));
              const uint32_t b = kb == 0 ? nk_s_g8.x : (kb == 1 ? nk_s_g8.y : (kb == 2 ? nk_s_g8.z : nk_s_g8.w));
              s_g = prmt(a, a, half_sel);
              s_g8 = prmt(b, b, half_sel);
              if (ZMODE == kZeroGeneral && cp.has_z_tile) {
                const uint32_t za = kb == 0 ? nk_z_g.x : (kb == 1 ? nk_z_g.y : (kb == 2 ? nk_z_g.z : nk_z_g.w));
                const uint32_t zb = kb == 0 ? nk_z_g8.x : (kb == 1 ? nk_z_g8.y : (kb == 2 ? nk_z_g8.z : nk_z_g8.w));
                z_g = prmt(za, za, half_sel);
                z_g8 = prmt(zb, zb, half_sel);
              }
            } else {
              // [groups][128 rows]: group row of this lane inside the chunk
              const int gl = (kb * G::kFrag + lane_k) / (GROUP > 0 ? GROUP : 1);
              const __half* sp = reinterpret_cast<const __half*>(sbase + L::kSOff) + gl * kTileRows + warp * 16 + g;
              s_g = h2_bcast(sp[0]);
              s_g8 = h2_bcast(sp[8]);
              if (ZMODE == kZeroGeneral && cp.has_z_tile) {
                const __half* zp = reinterpret_cast<const __half*>(sbase + L::kZOff) + gl * kTileRows + warp * 16 + g;
                z_g = h2_bcast(zp[0]);
                z_g8 = h2_bcast(zp[8]);
              }
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
                  mma_16816(acc[mt][j & 1], a, b0, b1);
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
              for (int mt = 0; mt < MT; ++mt) mma_16816(acc[mt][0], a, xv[mt].x, xv[mt].y);
              decode_int8_pair<ZMODE>(wv.z, wv.w, zc, s_g, s_g8, z_g, z_g8, a);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) mma_16816(acc[mt][1], a, xv[mt].z, xv[mt].w);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (!ok) break;

    // fold the two chains
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mt][0][c] += acc[mt][1][c];

    bool store = (S == 1);
    if (S > 1) {
      const int buf = round & 1;
      const int leader = round % S;
      // my buffer `buf` was last used for tile round-2: its leader must have summed it
      if (round >= 2) {
        if (!mbar_wait_cluster_bounded(&free_bar[buf], (uint32_t)(((round >> 1) - 1) & 1), p.status)) {
          ok = false;
          break;
        }
      }
      float* dst = red + (size_t)buf * kRedFloats + (size_t)warp * MT * 128 + lane;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = acc[mt][0][c];
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_rank(smem_u32(ready_bar), (uint32_t)leader));
      if (rank == leader) {
        if (!mbar_wait_cluster_bounded(ready_bar, (uint32_t)(leads_done & 1), p.status)) {
          ok = false;
          break;
        }
        ++leads_done;
        const uint32_t base = smem_u32(red + (size_t)buf * kRedFloats + (size_t)warp * MT * 128 + lane);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[mt][0][c] = 0.0f;
        for (int r = 0; r < S; ++r) {  // fixed rank order: deterministic
          const uint32_t ra = map_to_rank(base, (uint32_t)r);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mt][0][c] += ld_dsmem_f32(ra + (mt * 128 + c * 32) * 4);
        }
        __syncwarp();
        if (lane < S) mbar_arrive_remote(map_to_rank(smem_u32(&free_bar[buf]), (uint32_t)lane));
        store = true;
      }
    }
    if (store && active) {
      griddep_wait();  // the previous kernel may still read what this store overwrites
      if (p.epi.act == kActSwiglu) {
        const int64_t f = (int64_t)blk * 8 + g;  // rows g / g+8 are gate_f / up_f (interleaved repack)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int64_t m = mt * 8 + t * 2 + cc;
            if (m < p.m) p.out[m * p.ldo + f] = __float2half_rn(silu_mul(acc[mt][0][cc], acc[mt][0][cc + 2]));
          }
        continue;
      }
      const int64_t n0 = (int64_t)blk * 16 + g;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int64_t m = mt * 8 + t * 2 + (c & 1);
          const int64_t n = n0 + (c >> 1) * 8;
          if (m < p.m) p.out[m * p.ldo + n] = __float2half_rn(apply_epilogue(acc[mt][0][c], p.epi, m, n));
        }
      }
    }
  }

  // nobody leaves while a leader may still read its partials: wait for the last hand-backs
  if (S > 1 && ok) {
    for (int r = max(0, round - 2); r < round; ++r)
      mbar_wait_cluster_bounded(&free_bar[r & 1], (uint32_t)((r >> 1) & 1), p.status);
  }
}

#endif  // __CUDACC__

struct ClusterLaunch {
  int bits, mt, zmode, group_code, src;
  int n_tiles, cpt, sm_count;
  int ctas_per_sm;      // residency target used to size the pipeline
  size_t stage_bytes;   // one pipeline stage
  size_t fixed_bytes;   // partial-fragment buffers
};

// implemented per bit width (two translation units, so they compile in parallel)
int launch_cluster_i4(const ClusterParams& cp, const ClusterLaunch& l, const CUtensorMap& ts,
                      const CUtensorMap& tz, cudaStream_t stream);
int launch_cluster_i8(const ClusterParams& cp, const ClusterLaunch& l, const CUtensorMap& ts,
                      const CUtensorMap& tz, cudaStream_t stream);
size_t cluster_stage_bytes(int bits, int mt, int zmode, int src);

}  // namespace gc

// Host entry: plans (split factor, stages, scale staging) and launches the cluster kernel.
int gemv_cluster_run(const GemvParams& p, int bits, int zmode, int sm_count, cudaStream_t stream);

}  // namespace rb200
