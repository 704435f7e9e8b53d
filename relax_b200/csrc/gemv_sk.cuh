// Decode-path kernel (m <= 32), the default: warp-MMA consumers on a stream-k split.
//
// What measurements on B200 settled before this version was written:
//  * mma.sync.m16n8k16 sustains one MMA per 8 clocks per SM sub-partition - a 16x16 weight
//    fragment (128 packed bytes) per 2 clocks per SM, far above the HBM rate - while one
//    tcgen05.mma (M = 128, K = 16) occupies the tensor pipe for 108 clocks whatever its N up to
//    192: with the batch as N it caps the weight stream near 2.8 TB/s.  Small batches belong on
//    the warp MMA; tcgen05 pays off from a batch of a hundred rows up.
//  * the async copy engine is paid per contiguous segment, not per byte.  Hence the
//    stage-contiguous fragment layout: one 16 KB bulk copy per stage.
//  * a warp that issues a 16-byte cp.async stalls until the address is translated - more than a
//    microsecond at every kernel start, when the weight and scale pages are cold.  Everything a
//    stage needs therefore travels as bulk / TMA copies, which never stall their issuer.
//  * registers are handed out per SM sub-partition: a ninth warp (a dedicated producer) costs
//    every thread 32 of its 128 registers, and a polling producer takes issue slots from the
//    arithmetic.  There is no producer warp: a ring-full of stages is requested at start-up by
//    the first lanes of as many warps, and afterwards the warp that finishes a stage last
//    requests its next fill.
//  * the only divisions are in the work split, once per warp, 32-bit: 64-bit divisions in a
//    per-piece helper cost microseconds at every kernel start.
//  * global fix-up through fences and tickets costs 6-8 us per launch.  Here a CTA does the
//    pieces of tiles it shares with neighbours first (the tail piece goes to a global slot + a
//    flag right away, the head piece stays in registers), then its whole tiles, and only at the
//    very end adds the neighbours' slots - written long before - to its head piece.
//
//   8 warps, each one 16-row block of the CTA's 128-row tile; per stage: 128-bit fragment words
//   from shared memory, bit-exact decode in registers, m16n8k16 MMAs into fp32 fragments
//
// Split-k flags are plain 0 / 1 words: the writer of a tail piece sets its flag after the
// partial sums, the one owner that consumes the piece clears it again, so a launch leaves the
// flags as it found them and a CUDA graph may replay it any number of times.
//
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at small m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and the reference's GEMV / LowBatchGEMV
// schedules (python/tvm/dlight/gpu/gemv.py:216-530, low_batch_gemv.py:300-613).
#pragma once

#include <cuda.h>

#include <type_traits>

#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace sk {

constexpr int kConsumerWarps = 8;
constexpr int kThreads = kConsumerWarps * 32;  // no producer warp: whoever empties a stage refills it
constexpr int kTileRows = kConsumerWarps * 16;
constexpr int kBlocksPerChunk = 4;
constexpr int kTileBytes = 512;
constexpr int kScaleBoxBytes = 2048;

enum ScaleSrc : int { kSrcGlobal = 0, kSrcSmemNK = 1, kSrcSmemKN = 2 };

template <int BITS>
struct Geo {
  static constexpr int kFrag = BITS == 4 ? 64 : 32;
  static constexpr int kChunk = kFrag * kBlocksPerChunk;                 // 256 / 128 k per stage
  static constexpr int kXBlocks = kChunk / 64;                           // 64-k (128-byte) x blocks per stage
  static constexpr int kWBytes = kConsumerWarps * kBlocksPerChunk * kTileBytes;
};

template <int BITS, int MT, int ZMODE, int SRC>
struct StageLayout {
  // x tile of a stage: [64-k block][batch row][128 bytes], 128-byte swizzled by the TMA load
  static constexpr int kXBlockBytes = MT * 8 * 128;
  static constexpr int kXBytes = Geo<BITS>::kXBlocks * kXBlockBytes;
  static constexpr int kSOff = Geo<BITS>::kWBytes + kXBytes;
  static constexpr int kSBytes = SRC == kSrcGlobal ? 0 : kScaleBoxBytes;
  static constexpr int kZOff = kSOff + kSBytes;
  static constexpr int kZBytes = (SRC != kSrcGlobal && ZMODE == kZeroGeneral) ? kScaleBoxBytes : 0;
  static constexpr int kBytes = kZOff + kZBytes;
};

// Row-parallel epilogue fused with the sum over ranks (world > 1).  Every rank owns a workspace
// its peers can address:
//   [ header 256 B: u32 calls, u32 ctas_done |
//     data [2 regions][kArMaxRanks][max_blocks][kArSlotWords] x 8 bytes ]
// A warp that has the final fp32 fragment of a 16-row block writes it into slot [rank][block] of
// EVERY rank's workspace (its own included) as 8-byte words {value, call number}: an aligned
// 8-byte store arrives whole, so the word is its own flag and no fence is needed anywhere (a
// system-scope fence costs several microseconds, two of them per exchange more than the matmul).
// At the very end of the kernel the same warp reads its own copy of every rank's slot, polling -
// bounded - each word until it carries the call number, adds the values in rank order (so every
// rank forms the same bits), applies the epilogue, rounds once and stores.
// The call number is kept on the device (header), which makes the launch graph-replayable; the
// two data regions alternate with its parity, because a peer may still be reading call i when
// this rank is already publishing call i + 1 (it cannot reach call i + 2: that needs the peer's
// words of call i + 1, which the peer writes after it finished call i), and a word left from
// call i - 2 never carries the number of call i.
constexpr int kArMaxRanks = 8;
constexpr int kArSlotWords = 4 * 128;  // four m-tiles of one 16-row block, one 8-byte word per value
constexpr size_t kArHeaderBytes = 256;
struct ArCtx {
  uint8_t* ws[kArMaxRanks];  // ws[r]: rank r's workspace as this GPU addresses it
  int rank, world;           // world <= 1: no exchange
  unsigned max_blocks;       // 16-row blocks a region has room for
  // self-test on one GPU: the launch holds `emulate` ranks, every one gridDim / emulate CTAs
  // (launched cooperatively, so that all of them are resident while they wait on one another);
  // CTA b belongs to rank b / (gridDim / emulate), which uses its own slice of the split-k
  // scratch and writes rows [rank * m, (rank + 1) * m) of out.  0: an ordinary launch.
  int emulate;
};
__host__ __device__ __forceinline__ size_t ar_workspace_bytes(unsigned max_blocks) {
  return kArHeaderBytes + (size_t)2 * kArMaxRanks * max_blocks * kArSlotWords * 8;
}

// Grouped (expert) form at decode size: one launch per expert over the same x / out; the rows
// [indptr[expert - 1], indptr[expert]) of x are that expert's batch (indptr on the device, end
// offsets).  A launch whose expert has no rows returns at once.
struct GroupCtx {
  const int64_t* indptr;  // nullptr: the ungrouped form, rows [0, m)
  int expert;
  int has_prev;           // expert 0 starts at indptr[-1] (a sub-range of a longer table), not at row 0
};

struct Params {
  GemvParams g;
  ArCtx ar;
  GroupCtx grp;
  float* partial;     // [grid][2][8 warps][MT][4][32] fp32: slot 0 tail piece (for the owner), slot 1 own head piece
  unsigned* flags;    // [grid][8]: 1 while a tail piece waits for its owner, 0 at rest
  int has_z_tile;
  unsigned s_box_bytes;    // bytes one scale (or zero) TMA tile delivers
  unsigned wait_limit_ms;  // bound of the fix-up wait (0: about two seconds)
};

#ifdef __CUDACC__

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
enum PieceKind : int { kWhole = 0, kTail = 1, kHead = 2 };
struct Piece {
  int tile, c0, c1, kind;
};
// A CTA's contiguous range [it0, it1) of (tile, chunk) iterations, cut into pieces in execution
// order: the tail piece (a tile begun by an earlier CTA), the head piece (a tile this CTA begins
// and others finish), then whole tiles.  Built once per warp (the only divisions of the kernel,
// 32-bit); piece(idx) afterwards is compares and adds.
struct PiecePlan {
  int first_tile, last_tile, fc0, lc1, cpt;
  int w0, w1;  // whole tiles w0 .. w1 inclusive
  bool has_tail, has_head, single, any;

  __device__ __forceinline__ void build(unsigned cta, unsigned total, unsigned grid, int cpt_) {
    const unsigned it0 = cta * total / grid;  // total * grid < 2^31 (checked by the host)
    const unsigned it1 = (cta + 1) * total / grid;
    cpt = cpt_;
    any = it0 < it1;
    first_tile = (int)(it0 / (unsigned)cpt_);
    fc0 = (int)(it0 - (unsigned)first_tile * (unsigned)cpt_);
    const unsigned l = any ? it1 - 1 : it0;
    last_tile = (int)(l / (unsigned)cpt_);
    lc1 = (int)(l - (unsigned)last_tile * (unsigned)cpt_) + 1;
    has_tail = fc0 != 0;
    single = first_tile == last_tile;
    has_head = lc1 != cpt_ && !(single && has_tail);
    w0 = first_tile + (has_tail ? 1 : 0);
    w1 = last_tile - ((has_head || (single && has_tail)) ? 1 : 0);
  }
  __device__ __forceinline__ bool piece(int idx, Piece& pc) const {
    if (!any) return false;
    int n = 0;
    if (has_tail) {
      if (idx == 0) {
        pc.tile = first_tile;
        pc.c0 = fc0;
        pc.c1 = single ? lc1 : cpt;
        pc.kind = kTail;
        return true;
      }
      n = 1;
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
    const int t = w0 + idx - n;
    if (t <= w1) {
      pc.tile = t;
      pc.c0 = 0;
      pc.c1 = cpt;
      pc.kind = kWhole;
      return true;
    }
    return false;
  }
};

template <int BITS, int GROUP>
struct ScalePlan {
  static constexpr int kFrag = Geo<BITS>::kFrag;
  static constexpr int kChunk = Geo<BITS>::kChunk;
  static constexpr int kSpan =
      GROUP == 0 ? kChunk : (GROUP < 0 ? kFrag : (GROUP > kChunk ? kChunk : (GROUP < kFrag ? kFrag : GROUP)));
  static constexpr int kCount = kChunk / kSpan;
};

__device__ __forceinline__ void st_volatile_v2(uint2* p, uint32_t x, uint32_t y) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned atom_inc_acq_rel_shared(unsigned* p) {
  unsigned old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(smem_u32(p)) : "memory");
  return old;
}

// AR: compiled with the all-reduce epilogue (a separate instantiation, so that the plain kernel
// carries none of its code or registers).
template <int BITS, int MT, int ZMODE, int GROUP, int SRC, bool AR = false>
__global__ void __launch_bounds__(kThreads, 2)
    gemv_sk_kernel(const Params pp, const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_s,
                   const __grid_constant__ CUtensorMap tmap_z) {
  using G = Geo<BITS>;
  using L = StageLayout<BITS, MT, ZMODE, SRC>;
  using SP = ScalePlan<BITS, GROUP>;
  constexpr int kStage = L::kBytes;
  constexpr int kChains = MT <= 2 ? 2 : 1;  // independent MMA chains per m-tile (four m-tiles are four already)
  extern __shared__ uint8_t smem_raw[];
  // stages start on 1 KB boundaries: the x tile's 128-byte swizzle is a function of the address
  // (an offset from the array, not a pointer rebuilt from an integer: the compiler must keep
  // seeing shared memory, or every fragment read turns into a generic load)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const GemvParams& p = pp.g;

  const int stages = p.stages;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)stages * kStage);
  unsigned* drained = reinterpret_cast<unsigned*>(full_bar + stages);  // per stage: warps done with its current fill

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);  // the issuing lane's expect_tx arrival; the copies complete the bytes
      drained[s] = 0u;
    }
    drained[stages] = 0u;  // warps of this CTA through with the all-reduce epilogue
    mbar_fence_init();
  }
  fence_proxy_async();
  __syncthreads();
  griddep_launch_dependents();

  // batch rows of this launch inside x / out
  int m_lo = 0, m_rows = p.m;
  if (pp.grp.indptr) {
    griddep_wait();  // the row table is the routing kernel's output
    const int64_t r0 = (pp.grp.expert || pp.grp.has_prev) ? pp.grp.indptr[pp.grp.expert - 1] : 0;
    int64_t r1 = pp.grp.indptr[pp.grp.expert];
    if (r1 > p.m) r1 = p.m;  // never past the rows x / out hold
    if (r1 <= r0) return;    // every thread of every CTA alike; nothing is in flight yet
    m_lo = (int)r0;
    m_rows = (int)(r1 - r0) < MT * 8 ? (int)(r1 - r0) : MT * 8;
  }

  // rank-dependent values (one launch = one rank, except in the self-test: see ArCtx::emulate)
  int ar_rank = pp.ar.rank;
  unsigned grid = gridDim.x;
  int cta = blockIdx.x;
  float* sk_partial = pp.partial;
  unsigned* sk_flags = pp.flags;
  __half* out_base = p.out;
  if (AR && pp.ar.emulate > 1) {
    grid = gridDim.x / (unsigned)pp.ar.emulate;
    ar_rank = (int)(blockIdx.x / grid);
    cta = (int)(blockIdx.x % grid);
    sk_partial += (size_t)ar_rank * grid * 2 * kConsumerWarps * MT * 128;
    sk_flags += (size_t)ar_rank * grid * kConsumerWarps;
    out_base += (size_t)ar_rank * p.m * p.ldo;
  }
  const unsigned total = (unsigned)p.total_iters;  // the host checks that total * grid fits 32 bits
  const int cpt = p.chunks_per_tile;
  PiecePlan plan;
  plan.build((unsigned)cta, total, grid, cpt);
  const int kb_total = p.k / G::kFrag;
  const int n_blocks = p.n / 16;

  // ---------------------------------------------------------------- filling one stage
  // Everything a stage needs travels on the async copy engine and is counted in bytes on the
  // stage's barrier; the issuing lane never waits on a load (16-byte cp.async copies did: their
  // issue stalled for a microsecond and more at every kernel start).
  //   weights : one bulk copy, contiguous in the fragment layout
  //   scales / zero points : one TMA tile each (when their layout is one of the regular forms)
  //   x : one TMA tile [64-k blocks][MT*8 rows][128 B], 128-byte swizzle (conflict-free fragment
  //       reads); rows past m and k past the end read as zero
  constexpr uint32_t kXTx = (uint32_t)L::kXBytes;
  auto feed_w = [&](int tile, int chunk, int stage) {  // one lane: weights + scale / zero tiles
    uint8_t* sb = smem + (size_t)stage * kStage;
    const int nblk = min(kConsumerWarps, n_blocks - tile * kConsumerWarps);
    const int nkb = min(kBlocksPerChunk, kb_total - chunk * kBlocksPerChunk);
    const uint32_t wbytes = (uint32_t)(nkb * nblk) * kTileBytes;
    uint32_t tx = wbytes + kXTx;
    if (SRC != kSrcGlobal) tx += pp.s_box_bytes * ((ZMODE == kZeroGeneral && pp.has_z_tile) ? 2u : 1u);
    mbar_arrive_expect_tx(&full_bar[stage], tx);
    bulk_g2s(sb, p.w + frag_stage_offset(tile, chunk, n_blocks, kb_total), wbytes, &full_bar[stage]);
    if (SRC != kSrcGlobal) {
      // coordinates: NK tensor {group, row}; KN tensor {row, group}
      constexpr int kGroupsPerChunk = GROUP > 0 ? (G::kChunk / GROUP) : 1;
      const int gc0 = chunk * kGroupsPerChunk, r0 = tile * kTileRows;
      if (SRC == kSrcSmemNK) tma_load_2d(sb + L::kSOff, &tmap_s, gc0, r0, &full_bar[stage]);
      else tma_load_2d(sb + L::kSOff, &tmap_s, r0, gc0, &full_bar[stage]);
      if (ZMODE == kZeroGeneral && pp.has_z_tile) {
        if (SRC == kSrcSmemNK) tma_load_2d(sb + L::kZOff, &tmap_z, gc0, r0, &full_bar[stage]);
        else tma_load_2d(sb + L::kZOff, &tmap_z, r0, gc0, &full_bar[stage]);
      }
    }
  };
  auto feed_x = [&](int chunk, int stage) {  // one lane: the x tile of the stage
    tma_load_3d(smem + (size_t)stage * kStage + G::kWBytes, &tmap_x, 0, m_lo, chunk * G::kXBlocks, &full_bar[stage]);
  };
  // Walker over this CTA's (tile, chunk) stages in execution order.
  struct Walker {
    Piece pc;
    int idx, chunk;
    bool have;
  };
  auto w_begin = [&](Walker& w) {
    w.idx = 0;
    w.have = plan.piece(0, w.pc);
    w.chunk = w.have ? w.pc.c0 : 0;
  };
  auto w_next = [&](Walker& w) {
    if (++w.chunk >= w.pc.c1) {
      w.have = plan.piece(++w.idx, w.pc);
      if (w.have) w.chunk = w.pc.c0;
    }
  };

  // -------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int t = lane & 3;
  const ZeroConsts zc = make_zero_consts(ZMODE, p.zero_const);
  const uint32_t zconst_h2 = h2_bcast(__float2half_rn(p.zero_const));
  const int group = GROUP > 0 ? GROUP : (GROUP == 0 ? p.k : p.group);
  const int lane_k = t * (G::kFrag / 4);
  const uint32_t half_sel = (t >> 1) ? 0x3232u : 0x1010u;
  const int unit = frag_unit_pos(lane);
  // byte offset of this lane's x pieces inside a 128-byte swizzled row: int4 - pieces 2t and 2t + 1
  // of the 64-k block; int8 - piece t of the even / odd 32-k fragment tile of the block
  const int x_off[2] = {BITS == 4 ? ((2 * t) ^ g) << 4 : (t ^ g) << 4, BITS == 4 ? ((2 * t + 1) ^ g) << 4 : ((4 + t) ^ g) << 4};

  float acc[MT][kChains][4];
  // the head piece waits for the other CTAs' parts: in registers for one or two m-tiles, in this
  // CTA's own global slot for four (the register file then fits two CTAs per SM)
  constexpr bool kHeadInRegs = MT <= 2;
  float head[kHeadInRegs ? MT : 1][4];
  bool have_head = false;
  bool head_published = false;
  int head_tile = 0;
  uint32_t s_cur[SP::kCount], s_nxt[SP::kCount];
  uint32_t z_cur[SP::kCount], z_nxt[SP::kCount];

  // Start-up: lane 0 of consumer warp w requests the first fill of stage w - a ring-full of
  // copies leaves within one warp's instruction latency instead of queueing behind one another.
  // Weights and scales do not depend on the previous kernel on the stream and go out at once;
  // x follows after the dependency wait.
  if (warp < stages) {
    Walker w;
    w_begin(w);
    for (int i = 0; i < warp && w.have; ++i) w_next(w);
    if (w.have) {
      if (lane == 0) feed_w(w.pc.tile, w.chunk, warp);
      griddep_wait();
      if (lane == 0) feed_x(w.chunk, warp);
      __syncwarp();
    }
  }

  // `ahead` names the iteration that will next be loaded into the stage being consumed: one
  // ring-length past the consumer.  Every warp tracks it; the warp that finishes a stage last
  // (shared-memory counter) issues that load.
  Walker ahead;
  w_begin(ahead);
  for (int i = 0; i < stages && ahead.have; ++i) w_next(ahead);

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
          if (m < m_rows) out_base[(m_lo + m) * p.ldo + f] = __float2half_rn(silu_mul(v[mt][cc], v[mt][cc + 2]));
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
        if (m < m_rows) out_base[(m_lo + m) * p.ldo + n] = __float2half_rn(apply_epilogue(v[mt][c], p.epi, m_lo + m, n));
      }
  };

  // ---- all-reduce side of the epilogue (see ArCtx)
  const bool ar_on = AR && pp.ar.world > 1;
  unsigned ar_call = 0;
  auto ar_slot = [&](int r, unsigned call, int src, int blk) -> uint2* {
    return reinterpret_cast<uint2*>(pp.ar.ws[r] + kArHeaderBytes) +
           ((size_t)((call & 1u) * kArMaxRanks + (unsigned)src) * pp.ar.max_blocks + (unsigned)blk) * kArSlotWords;
  };
  // this rank's part of a block is final: hand it to every rank
  auto ar_publish = [&](const float (&v)[MT][4], int tile_i) {
    const int blk = tile_i * kConsumerWarps + warp;
    if (blk >= n_blocks) return;
    for (int r = 0; r < pp.ar.world; ++r) {
      uint2* dst = ar_slot(r, ar_call, ar_rank, blk) + lane;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) st_volatile_v2(dst + (mt * 4 + c) * 32, __float_as_uint(v[mt][c]), ar_call);
    }
  };
  // all ranks' parts of a block: wait for the words, add in rank order, finish
  auto ar_finish = [&](int tile_i, unsigned long long limit_ns) -> bool {
    const int blk = tile_i * kConsumerWarps + warp;
    if (blk >= n_blocks) return true;
    float sum[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) sum[mt][c] = 0.0f;
    bool arrived = true;
    // One rank after the other (requesting the words of several ranks together before looking at
    // any of them measured slower: 272 against 262 us per step at four ranks).  While a rank's
    // words are not all there, ALL of them are requested again together - one trip to memory per
    // try, not one per word.
    for (int r = 0; r < pp.ar.world && arrived; ++r) {
      const uint2* src = ar_slot(ar_rank, ar_call, r, blk) + lane;
      uint2 w[MT][4];
      unsigned long long t0 = 0ull;
      for (;;) {
        bool all = true;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) w[mt][c] = ld_volatile_v2(src + (mt * 4 + c) * 32);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) all = all && (w[mt][c].y == ar_call);
        if (all) break;
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t0 == 0ull) t0 = t1;
        if (t1 - t0 > limit_ns) {
          if (p.status) atomicExch(p.status, kStatusWaitTimeout);
          arrived = false;
          break;
        }
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) sum[mt][c] += __uint_as_float(w[mt][c].x);
      arrived = __all_sync(0xffffffffu, arrived);
    }
    if (!arrived) return false;
    store_tile(sum, tile_i);
    return true;
  };

  for (int idx = 0; ok && plan.piece(idx, pc); ++idx) {
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
      // this lane's 16-byte pieces of x: row g of every m-tile, swizzled position (piece ^ g)
      const uint8_t* xsm = sbase + G::kWBytes + g * 128;
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
                  xv[mt][j >> 1] = *reinterpret_cast<const uint4*>(xsm + kb * L::kXBlockBytes + mt * 1024 + x_off[j >> 1]);
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
              xv[mt] = *reinterpret_cast<const uint4*>(xsm + (kb >> 1) * L::kXBlockBytes + mt * 1024 + x_off[kb & 1]);
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
      if (lane == 0 && atom_inc_acq_rel_shared(&drained[stage]) == kConsumerWarps - 1) {
        drained[stage] = 0u;  // visible to the other warps through the stage's barrier, like the data
        if (ahead.have) {
          feed_w(ahead.pc.tile, ahead.chunk, stage);
          feed_x(ahead.chunk, stage);
        }
      }
      w_next(ahead);
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
    if (ar_on && ar_call == 0) ar_call = *reinterpret_cast<volatile unsigned*>(pp.ar.ws[ar_rank]) + 1u;
    if (pc.kind == kWhole) {
      if (ar_on) ar_publish(fin, pc.tile);
      else store_tile(fin, pc.tile);
    } else if (pc.kind == kHead) {
      have_head = true;
      head_tile = pc.tile;
      if (kHeadInRegs) {
#pragma unroll
        for (int mt = 0; mt < (kHeadInRegs ? MT : 1); ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) head[mt][c] = fin[mt][c];
      } else {
        float* dst = sk_partial + ((size_t)((cta * 2 + 1) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = fin[mt][c];
      }
    } else {
      // tail piece: publish for the owner (the CTA that holds this tile's first chunk)
      float* dst = sk_partial + ((size_t)((cta * 2) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[mt * 128 + c * 32] = fin[mt][c];
      __threadfence();
      __syncwarp();
      if (lane == 0) st_release_u32(sk_flags + cta * kConsumerWarps + warp, 1u);
    }
  }

  // ---------------------------------------------------------------- fix-up of the owned tile
  if (ok && have_head) {
    // the last CTA whose range reaches into the owned tile
    const unsigned hi_it = (unsigned)head_tile * (unsigned)cpt + (unsigned)cpt - 1u;
    const int last_cta = (int)(((hi_it + 1u) * grid - 1u) / total);
    const unsigned long long limit_ns = (pp.wait_limit_ms ? (unsigned long long)pp.wait_limit_ms : 2000ull) * 1000000ull;
    // one contributor per lane: all flags are polled at once (polled one after another, every
    // contributor cost a round trip to L2 even when its flag was long set)
    bool flags_ok = true;
    for (int c0 = cta + 1; c0 <= last_cta && flags_ok; c0 += 32) {
      const int c = c0 + lane;
      if (c <= last_cta) {
        const unsigned* f = sk_flags + c * kConsumerWarps + warp;
        if (ld_acquire_u32(f) == 0u) {
          unsigned long long t0;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
          while (ld_acquire_u32(f) == 0u) {
            __nanosleep(256);
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > limit_ns) {  // give up, report, leave the tile unwritten
              if (p.status) atomicExch(p.status, kStatusWaitTimeout);
              flags_ok = false;
              break;
            }
          }
        }
      }
      flags_ok = __all_sync(0xffffffffu, flags_ok);
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
        const float* own = sk_partial + ((size_t)((cta * 2 + 1) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) sum[mt][cc] = own[mt * 128 + cc * 32];  // written by this same thread
      }
      for (int c = cta + 1; c <= last_cta; ++c) {  // fixed CTA order: deterministic
        const float* src = sk_partial + ((size_t)((c * 2) * kConsumerWarps + warp) * MT) * 128 + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) sum[mt][cc] += __ldcg(src + mt * 128 + cc * 32);
      }
      // every slot has exactly one consumer (this warp): hand the flags back at rest.  The
      // next launch writes them only after this grid has completed.
      __syncwarp();
      if (lane == 0)
        for (int c = cta + 1; c <= last_cta; ++c) sk_flags[c * kConsumerWarps + warp] = 0u;
      if (ar_on) {
        ar_publish(sum, head_tile);
        head_published = true;
      } else {
        store_tile(sum, head_tile);
      }
    }
  }

  // ---------------------------------------------------------------- sum over ranks
  if (ar_on) {
    const unsigned long long limit_ns = (pp.wait_limit_ms ? (unsigned long long)pp.wait_limit_ms : 2000ull) * 1000000ull;
    if (ok) {
      // the blocks this warp published: its whole tiles, then the tile it owns
      bool fine = true;
      for (int idx = 0; fine && plan.piece(idx, pc); ++idx)
        if (pc.kind == kWhole) fine = ar_finish(pc.tile, limit_ns);
      if (fine && head_published) ar_finish(head_tile, limit_ns);
    }
    // the call is over when every warp of the grid is through: the last CTA advances the
    // device-side call number (read by the next launch after its dependency wait)
    griddep_wait();
    if (ar_call == 0) ar_call = *reinterpret_cast<volatile unsigned*>(pp.ar.ws[ar_rank]) + 1u;
    __syncwarp();
    if (lane == 0 && atom_inc_acq_rel_shared(&drained[stages]) == kConsumerWarps - 1) {
      unsigned* hdr = reinterpret_cast<unsigned*>(pp.ar.ws[ar_rank]);
      if (atomicAdd(hdr + 1, 1u) == grid - 1u) {
        hdr[1] = 0u;
        *reinterpret_cast<volatile unsigned*>(hdr) = ar_call;
      }
    }
  }
}

#endif  // __CUDACC__

struct Launch {
  int bits, mt, zmode, group_code, src;
  int grid;
  int cooperative;  // all CTAs must be resident together (emulated ranks wait on one another)
  size_t smem_bytes;
};
int launch_sk_i4(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
                 cudaStream_t stream);
int launch_sk_i8(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
                 cudaStream_t stream);

}  // namespace sk

// Host entry: plans and launches the stream-k decode kernel.  `partial` / `flags` are scratch;
// the flags must be zero before the first launch and are left zero by every launch.
// `ar` (may be nullptr): finish the call with the sum over ranks, see sk::ArCtx.
// `grp` (may be nullptr): one expert of the grouped form, see sk::GroupCtx; p.m is then the total
// row count of x / out (at most 32).
int gemv_sk_run(const GemvParams& p, int bits, int zmode, int sm_count, float* partial, size_t partial_bytes,
                unsigned* flags, size_t flag_count, const sk::ArCtx* ar, const sk::GroupCtx* grp, cudaStream_t stream);

}  // namespace rb200
