// Decode-path kernel (m <= 32), the default: warp-MMA consumers on a stream-k split.
//
// What measurements on B200 settled before this version was written:
//  * mma.sync.m16n8k16 sustains one MMA per 8 clocks per SM sub-partition - a 16x16 weight
//    fragment (128 packed bytes) per 2 clocks per SM, far above the HBM rate - while tcgen05.mma
//    pays off only from a batch of a hundred rows up.  Small batches belong on the warp MMA.
//  * the async copy engine is paid per contiguous segment (about 170 clocks each when one thread
//    issues them), not per byte.  Hence the stage-contiguous fragment layout (one 16 KB bulk copy
//    per stage) and 16-byte cp.async for x and the scale tiles.
//  * the kernel is bound by instruction issue, not by bytes: every warp that polls a barrier
//    takes issue slots from the eight warps doing the arithmetic.  So one feeder warp (not two)
//    serves the ring, it sleeps between polls, and the consumers' inner loop carries no test
//    that can be decided outside it (ragged last chunk, inactive row block).
//  * global fix-up through fences and tickets costs 6-8 us per launch.  Here a CTA does the
//    pieces of tiles it shares with neighbours first (the tail piece goes to a global slot + a
//    flag right away, the head piece stays in registers), then its whole tiles, and only at the
//    very end adds the neighbours' slots - written long before - to its head piece.
//
//   feeder warp   : per (128-row tile, k-chunk) stage one bulk async copy of the packed weights
//                   (lane 0), the scale / zero tiles and the x slice by 16-byte cp.async (all
//                   lanes), everything counted on the stage's mbarrier.  Weights and scales of
//                   the first ring-full of stages are requested before the kernel waits for its
//                   predecessor on the stream; x only after.
//   8 consumers   : one 16-row block each; 128-bit fragment words from shared memory, bit-exact
//                   decode in registers, m16n8k16 MMAs into fp32 fragments
//
// Split-k flags are plain 0 / 1 words: the writer of a tail piece sets its flag after the
// partial sums, the one owner that consumes the piece clears it again, so a launch leaves the
// flags as it found them and a CUDA graph may replay it any number of times.
//
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at small m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and the reference's GEMV / LowBatchGEMV
// schedules (python/tvm/dlight/gpu/gemv.py:216-530, low_batch_gemv.py:300-613).
#pragma once

#include <type_traits>

#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace sk {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + feeder
constexpr int kTileRows = kConsumerWarps * 16;
constexpr int kBlocksPerChunk = 4;
constexpr int kTileBytes = 512;
constexpr int kScaleBoxBytes = 2048;

enum ScaleSrc : int { kSrcGlobal = 0, kSrcSmemNK = 1, kSrcSmemKN = 2 };

template <int BITS>
struct Geo {
  static constexpr int kFrag = BITS == 4 ? 64 : 32;
  static constexpr int kChunk = kFrag * kBlocksPerChunk;                 // 256 / 128 k per stage
  static constexpr int kXPitch = kChunk * 2 + (BITS == 4 ? 16 : 64);     // bank-conflict free
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

struct Params {
  GemvParams g;
  float* partial;     // [grid][2][8 warps][MT][4][32] fp32: slot 0 tail piece (for the owner), slot 1 own head piece
  unsigned* flags;    // [grid][8]: 1 while a tail piece waits for its owner, 0 at rest
  int has_z_tile;
  unsigned wait_limit_ms;  // bound of the fix-up wait (0: about two seconds)
};

#ifdef __CUDACC__

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long range_start(long long cta, long long total, long long grid) {
  return cta * total / grid;
}

enum PieceKind : int { kWhole = 0, kTail = 1, kHead = 2 };
struct Piece {
  int tile, c0, c1, kind;
};
// Pieces of a CTA's contiguous iteration range in execution order: the tail piece (a tile begun
// by an earlier CTA), the head piece (a tile this CTA begins and others finish), whole tiles.
__device__ __forceinline__ bool get_piece(long long it0, long long it1, int cpt, int idx, Piece& pc) {
  if (it0 >= it1) return false;
  const int first_tile = (int)(it0 / cpt), last_tile = (int)((it1 - 1) / cpt);
  const int fc0 = (int)(it0 % cpt);
  const int lc1 = (int)((it1 - 1) % cpt) + 1;
  const bool has_tail = fc0 != 0;
  const bool single = first_tile == last_tile;
  const bool has_head = lc1 != cpt && !(single && has_tail);
  int n = 0;
  if (has_tail) {
    if (idx == n) {
      pc.tile = first_tile;
      pc.c0 = fc0;
      pc.c1 = single ? lc1 : cpt;
      pc.kind = kTail;
      return true;
    }
    ++n;
  }
  if (has_head) {
    if (idx == n) {
      pc.tile = last_tile;
      pc.c0 = 0;
      pc.c1 = lc1;
      pc.kind = kHead;
      return true;
    }
    ++n;
  }
  const int w0 = first_tile + (has_tail ? 1 : 0);
  const int w1 = last_tile - ((has_head || (single && has_tail)) ? 1 : 0);  // inclusive
  const int wi = idx - n;
  if (w0 + wi <= w1) {
    pc.tile = w0 + wi;
    pc.c0 = 0;
    pc.c1 = cpt;
    pc.kind = kWhole;
    return true;
  }
  return false;
}

template <int BITS, int GROUP>
struct ScalePlan {
  static constexpr int kFrag = Geo<BITS>::kFrag;
  static constexpr int kChunk = Geo<BITS>::kChunk;
  static constexpr int kSpan =
      GROUP == 0 ? kChunk : (GROUP < 0 ? kFrag : (GROUP > kChunk ? kChunk : (GROUP < kFrag ? kFrag : GROUP)));
  static constexpr int kCount = kChunk / kSpan;
};

// Feeder-side wait: a failed poll is followed by a sleep, so a feeder that is ahead of the
// consumers costs them next to no issue slots.  Bounded like every other wait.
__device__ __forceinline__ bool mbar_wait_sleepy(uint64_t* bar, uint32_t parity, int* status) {
#pragma unroll 1
  for (int i = 0; i < (1 << 23); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(200);
  }
  if (status) atomicExch(status, kStatusWaitTimeout);
  return false;
}

template <int BITS, int MT, int ZMODE, int GROUP, int SRC>
__global__ void __launch_bounds__(kThreads, 2) gemv_sk_kernel(const Params pp) {
  using G = Geo<BITS>;
  using L = StageLayout<BITS, MT, ZMODE, SRC>;
  using SP = ScalePlan<BITS, GROUP>;
  constexpr int kStage = L::kBytes;
  constexpr int kChains = MT <= 2 ? 2 : 1;  // independent MMA chains per m-tile
  extern __shared__ __align__(128) uint8_t smem[];
  const GemvParams& p = pp.g;

  const int stages = p.stages;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStage);
  uint64_t* empty_bar = full_bar + stages;

  // x rows >= m are never written by the feeder and must read as zero
  for (int s = 0; s < stages; ++s) {
    uint32_t* xs = reinterpret_cast<uint32_t*>(smem + (size_t)s * kStage + G::kWBytes);
    for (int i = tid; i < L::kXBytes / 4; i += kThreads) xs[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1 + 32);  // lane 0's expect_tx arrival + 32 lanes of cp.async
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    mbar_fence_init();
  }
  fence_proxy_async();
  __syncthreads();
  griddep_launch_dependents();

  const int cta = blockIdx.x;
  const long long total = p.total_iters;
  const long long grid = gridDim.x;
  const long long it0 = range_start(cta, total, grid);
  const long long it1 = range_start(cta + 1, total, grid);
  const int cpt = p.chunks_per_tile;
  const int kb_total = p.k / G::kFrag;
  const int n_blocks = p.n / 16;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ feeder
    const int64_t kg = GROUP > 0 ? p.k / GROUP : 0;
    constexpr int kXChunks = G::kChunk * 2 / 16;  // 16-byte pieces per x row per stage (32 / 16)

    auto feed_w = [&](int tile, int chunk, int stage) {  // packed weights + scale / zero tiles
      uint8_t* sbase = smem + (size_t)stage * kStage;
      if (lane == 0) {
        const int nblk = min(kConsumerWarps, n_blocks - tile * kConsumerWarps);
        const int nkb = min(kBlocksPerChunk, kb_total - chunk * kBlocksPerChunk);
        const uint32_t wbytes = (uint32_t)(nkb * nblk) * kTileBytes;  // contiguous in the fragment layout
        mbar_arrive_expect_tx(&full_bar[stage], wbytes);
        bulk_g2s(sbase, p.w + frag_stage_offset(tile, chunk, n_blocks, kb_total), wbytes, &full_bar[stage]);
      }
      const int64_t n0 = (int64_t)tile * kTileRows;
      if (SRC == kSrcSmemNK) {
        // [128 rows][8 groups]: 16 bytes per row
        const int64_t g0 = (int64_t)chunk * 8;
        const int64_t left = (kg - g0) * 2;
        const uint32_t sv = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = lane + 32 * i;
          const bool in = n0 + row < p.n;
          const int64_t o = (in ? (n0 + row) : 0) * kg + (sv ? g0 : 0);
          cp_async16(sbase + L::kSOff + row * 16, p.s + o, in ? sv : 0u);
          if (ZMODE == kZeroGeneral && pp.has_z_tile) cp_async16(sbase + L::kZOff + row * 16, p.z + o, in ? sv : 0u);
        }
      } else if (SRC == kSrcSmemKN) {
        // [groups of the chunk][128 rows]: 256 bytes per group row
        constexpr int kG = GROUP > 0 ? (G::kChunk / GROUP) : 1;
        for (int i = lane; i < kG * 16; i += 32) {
          const int gl = i >> 4, cc = i & 15;
          const int64_t grow = (int64_t)chunk * kG + gl;
          const bool in = grow < kg && n0 + cc * 8 < p.n;
          const int64_t o = (in ? grow : 0) * p.n + (in ? n0 + cc * 8 : 0);
          cp_async16(sbase + L::kSOff + gl * 256 + cc * 16, p.s + o, in ? 16u : 0u);
          if (ZMODE == kZeroGeneral && pp.has_z_tile) cp_async16(sbase + L::kZOff + gl * 256 + cc * 16, p.z + o, in ? 16u : 0u);
        }
      }
    };
    auto feed_x = [&](int chunk, int stage) {  // x[r, chunk*kChunk + c*8 .. +8) -> row r of the stage's x tile
      uint8_t* sbase = smem + (size_t)stage * kStage;
      for (int i = lane; i < p.m * kXChunks; i += 32) {
        const int r = i / kXChunks, c = i % kXChunks;
        const int64_t kcol = (int64_t)chunk * G::kChunk + c * 8;
        const uint32_t v = kcol < p.k ? 16u : 0u;
        cp_async16(sbase + G::kWBytes + r * G::kXPitch + c * 16, p.x + (int64_t)r * p.ldx + (v ? kcol : 0), v);
      }
      cp_async_arrive(&full_bar[stage]);
    };

    // The first ring-full of stages needs no wait (every stage starts empty): request their
    // weights and scales at once, then wait for the previous kernel on the stream - activations
    // may be its output - and only then fetch x for them.
    Piece pc;
    int idx = 0, chunk = 0;
    bool have = get_piece(it0, it1, cpt, 0, pc);
    if (have) chunk = pc.c0;
    auto advance = [&]() {
      if (++chunk >= pc.c1) {
        have = get_piece(it0, it1, cpt, ++idx, pc);
        if (have) chunk = pc.c0;
      }
    };
    {
      Piece pc0 = pc;
      const int idx0 = idx, chunk0 = chunk;
      const bool have0 = have;
      int primed = 0;
      for (; have && primed < stages; ++primed) {
        feed_w(pc.tile, chunk, primed);
        advance();
      }
      griddep_wait();
      pc = pc0;
      idx = idx0;
      chunk = chunk0;
      have = have0;
      for (int s = 0; s < primed; ++s) {
        feed_x(chunk, s);
        advance();
      }
    }
    int stage = 0;        // after a full ring the next stage to fill is 0 again (primed == stages),
    uint32_t phase = 1;   // now on its second use; with fewer iterations than stages nothing is left
    bool ok = true;
    while (ok && have) {
      if (!mbar_wait_sleepy(&empty_bar[stage], phase ^ 1u, p.status)) {
        ok = false;
        break;
      }
      feed_w(pc.tile, chunk, stage);
      feed_x(chunk, stage);
      advance();
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    return;
  }

  // -------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int t = lane & 3;
  const ZeroConsts zc = make_zero_consts(ZMODE, p.zero_const);
  const uint32_t zconst_h2 = h2_bcast(__float2half_rn(p.zero_const));
  const int group = GROUP > 0 ? GROUP : (GROUP == 0 ? p.k : p.group);
  const int lane_k = t * (G::kFrag / 4);
  const uint32_t half_sel = (t >> 1) ? 0x3232u : 0x1010u;
  const int unit = frag_unit_pos(lane);

  float acc[MT][kChains][4];
  // the head piece waits for the other CTAs' parts: in registers for one or two m-tiles, in this
  // CTA's own global slot for four (the register file then fits two CTAs per SM)
  constexpr bool kHeadInRegs = MT <= 2;
  float head[kHeadInRegs ? MT : 1][4];
  bool have_head = false;
  int head_tile = 0;
  uint32_t s_cur[SP::kCount], s_nxt[SP::kCount];
  uint32_t z_cur[SP::kCount], z_nxt[SP::kCount];

  int stage = 0;
  uint32_t phase = 0;
  const uint8_t* sbase = smem;
  bool ok = true;
  Piece pc;

  auto store_tile = [&](const float (&v)[MT][4], int tile_i) {
    const int blk = tile_i * kConsumerWarps + warp;
    if (blk >= n_blocks) return;
    if (p.epi.act == kActSwiglu) {
      // rows g / g+8 of the block are gate_f / up_f of f = 8 blk + g (interleaved repack)
      const int64_t f = (int64_t)blk * 8 + g;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int64_t m = mt * 8 + t * 2 + cc;
          if (m < p.m) p.out[m * p.ldo + f] = __float2half_rn(silu_mul(v[mt][cc], v[mt][cc + 2]));
        }
      return;
    }
    const int64_t n0 = (int64_t)blk * 16 + g;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int64_t m = mt * 8 + t * 2 + (c & 1);
        const int64_t n = n0 + (c >> 1) * 8;
        if (m < p.m) p.out[m * p.ldo + n] = __float2half_rn(apply_epilogue(v[mt][c], p.epi, m, n));
      }
  };

  for (int idx = 0; ok && get_piece(it0, it1, cpt, idx, pc); ++idx) {
    const int blk = pc.tile * kConsumerWarps + warp;
    const bool active = blk < n_blocks;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int c = 0; c < kChains; ++c)
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
    if (pc.c0 < pc.c1) fetch_global(pc.c0, s_nxt, z_nxt);

    // One stage of this warp's row block.  `full` (a compile-time tag): all four k-blocks of
    // the chunk exist, so the unrolled body carries no test; the ragged last chunk of a k that
    // is not a multiple of the chunk takes the tested copy.
    auto consume = [&](auto full, int nkb) {
      constexpr bool kFull = decltype(full)::value;
      const uint4* wsm = reinterpret_cast<const uint4*>(sbase + warp * ((kFull ? kBlocksPerChunk : nkb) * kTileBytes)) + unit;
      const uint8_t* xsm = sbase + G::kWBytes + g * G::kXPitch + t * (G::kFrag / 2);
      uint4 nk_s_g, nk_s_g8, nk_z_g, nk_z_g8;
      if (SRC == kSrcSmemNK) {
        const uint4* sp = reinterpret_cast<const uint4*>(sbase + L::kSOff) + warp * 16 + g;
        nk_s_g = sp[0];
        nk_s_g8 = sp[8];
        if (ZMODE == kZeroGeneral && pp.has_z_tile) {
          const uint4* zp = reinterpret_cast<const uint4*>(sbase + L::kZOff) + warp * 16 + g;
          nk_z_g = zp[0];
          nk_z_g8 = zp[8];
        }
      }
#pragma unroll
      for (int kb = 0; kb < kBlocksPerChunk; ++kb) {
        if (kFull || kb < nkb) {
          const uint4 wv = wsm[kb * 32];
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
            const uint32_t a = kb == 0 ? nk_s_g.x : (kb == 1 ? nk_s_g.y : (kb == 2 ? nk_s_g.z : nk_s_g.w));
            const uint32_t b = kb == 0 ? nk_s_g8.x : (kb == 1 ? nk_s_g8.y : (kb == 2 ? nk_s_g8.z : nk_s_g8.w));
            s_g = prmt(a, a, half_sel);
            s_g8 = prmt(b, b, half_sel);
            if (ZMODE == kZeroGeneral && pp.has_z_tile) {
              const uint32_t za = kb == 0 ? nk_z_g.x : (kb == 1 ? nk_z_g.y : (kb == 2 ? nk_z_g.z : nk_z_g.w));
              const uint32_t zb = kb == 0 ? nk_z_g8.x : (kb == 1 ? nk_z_g8.y : (kb == 2 ? nk_z_g8.z : nk_z_g8.w));
              z_g = prmt(za, za, half_sel);
              z_g8 = prmt(zb, zb, half_sel);
            }
          } else {
            const int gl = (kb * G::kFrag + lane_k) / (GROUP > 0 ? GROUP : 1);
            const __half* sp = reinterpret_cast<const __half*>(sbase + L::kSOff) + gl * kTileRows + warp * 16 + g;
            s_g = h2_bcast(sp[0]);
            s_g8 = h2_bcast(sp[8]);
            if (ZMODE == kZeroGeneral && pp.has_z_tile) {
              const __half* zp = reinterpret_cast<const __half*>(sbase + L::kZOff) + gl * kTileRows + warp * 16 + g;
              z_g = h2_bcast(zp[0]);
              z_g8 = h2_bcast(zp[8]);
            }
          }
          if (BITS == 4) {
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
            uint4 xv[MT][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if ((j & 1) == 0) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                  xv[mt][j >> 1] = *reinterpret_cast<const uint4*>(xsm + mt * 8 * G::kXPitch + kb * 128 + (j >> 1) * 16);
              }
              uint32_t a[4];
              decode_int4_word<ZMODE>(ww[j], zc, s_g, s_g8, z_g, z_g8, a);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                const uint4& xr = xv[mt][j >> 1];
                const uint32_t b0 = (j & 1) ? xr.z : xr.x;
                const uint32_t b1 = (j & 1) ? xr.w : xr.y;
                mma_16816(acc[mt][j % kChains], a, b0, b1);
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
            for (int mt = 0; mt < MT; ++mt) mma_16816(acc[mt][kChains - 1], a, xv[mt].z, xv[mt].w);
          }
        }
      }
    };

    for (int chunk = pc.c0; chunk < pc.c1; ++chunk) {
      if (SRC == kSrcGlobal) {
#pragma unroll
        for (int i = 0; i < SP::kCount; ++i) {
          s_cur[i] = s_nxt[i];
          z_cur[i] = z_nxt[i];
        }
        if (chunk + 1 < pc.c1) fetch_global(chunk + 1, s_nxt, z_nxt);
      }
      if (!mbar_wait_parked(&full_bar[stage], phase, p.status)) {
        ok = false;
        break;
      }
      if (active) {
        const int nkb = kb_total - chunk * kBlocksPerChunk;
        if (nkb >= kBlocksPerChunk) consume(std::true_type{}, kBlocksPerChunk);
        else consume(std::false_type{}, nkb);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      sbase += kStage;
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
        sbase = smem;
      }
    }
    if (!ok) break;

    if (kChains == 2) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mt][0][c] += acc[mt][kChains - 1][c];
    }
    float fin[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) fin[mt][c] = acc[mt][0][c];

    // outputs and scratch may still be in use by the previous kernel until it has ended
    griddep_wait();
    if (pc.kind == kWhole) {
      store_tile(fin, pc.tile);
    } else if (pc.kind == kHead) {
      have_head = true;
      head_tile = pc.tile;
      if (kHeadInRegs) {
#pragma unroll
        for (int mt = 0; mt < (kHeadInRegs ? MT : 1); ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) head[mt][c] = fin[mt][c];
      } else {
        float* dst = pp.partial + ((size_t)((cta * 2 + 1) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = fin[mt][c];
      }
    } else {
      // tail piece: publish for the owner (the CTA that holds this tile's first chunk)
      float* dst = pp.partial + ((size_t)((cta * 2) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = fin[mt][c];
      __threadfence();
      __syncwarp();
      if (lane == 0) st_release_u32(pp.flags + cta * kConsumerWarps + warp, 1u);
    }
  }

  // ---------------------------------------------------------------- fix-up of the owned tile
  if (ok && have_head) {
    const long long hi_it = (long long)head_tile * cpt + cpt - 1;
    const int last_cta = (int)(((hi_it + 1) * grid - 1) / total);
    const unsigned long long limit_ns = (pp.wait_limit_ms ? (unsigned long long)pp.wait_limit_ms : 2000ull) * 1000000ull;
    bool flags_ok = true;
    for (int c = cta + 1; c <= last_cta && flags_ok; ++c) {
      const unsigned* f = pp.flags + c * kConsumerWarps + warp;
      if (ld_acquire_u32(f) != 0u) continue;
      unsigned long long t0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      while (ld_acquire_u32(f) == 0u) {
        __nanosleep(64);
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > limit_ns) {  // give up, report, leave the tile unwritten
          if (p.status) atomicExch(p.status, kStatusWaitTimeout);
          flags_ok = false;
          break;
        }
      }
    }
    flags_ok = __all_sync(0xffffffffu, flags_ok);
    if (flags_ok) {
      float sum[MT][4];
      if (kHeadInRegs) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) sum[mt][cc] = head[kHeadInRegs ? mt : 0][cc];
      } else {
        const float* own = pp.partial + ((size_t)((cta * 2 + 1) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) sum[mt][cc] = own[mt * 128 + cc * 32];  // written by this same thread
      }
      for (int c = cta + 1; c <= last_cta; ++c) {  // fixed CTA order: deterministic
        const float* src = pp.partial + ((size_t)((c * 2) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) sum[mt][cc] += __ldcg(src + mt * 128 + cc * 32);
      }
      // every slot has exactly one consumer (this warp): hand the flags back at rest.  The
      // next launch writes them only after this grid has completed.
      __syncwarp();
      if (lane == 0)
        for (int c = cta + 1; c <= last_cta; ++c) pp.flags[c * kConsumerWarps + warp] = 0u;
      store_tile(sum, head_tile);
    }
  }
}

#endif  // __CUDACC__

struct Launch {
  int bits, mt, zmode, group_code, src;
  int grid;
  size_t smem_bytes;
};
int launch_sk_i4(const Params& pp, const Launch& l, cudaStream_t stream);
int launch_sk_i8(const Params& pp, const Launch& l, cudaStream_t stream);

}  // namespace sk

// Host entry: plans and launches the stream-k decode kernel.  `partial` / `flags` are scratch;
// the flags must be zero before the first launch and are left zero by every launch.
int gemv_sk_run(const GemvParams& p, int bits, int zmode, int sm_count, float* partial, size_t partial_bytes,
                unsigned* flags, size_t flag_count, cudaStream_t stream);

}  // namespace rb200
