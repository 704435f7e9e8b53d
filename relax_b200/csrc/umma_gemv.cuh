// Decode-path kernel on the 5th-generation tensor cores (tcgen05 + TMEM), int4 weights, m <= 32.
//
// Why not mma.sync: on B200 the legacy warp MMA issues about once per 32 clocks per SM
// sub-partition, so a 16 x 16 weight fragment costs as many MMAs as there are 8-row batch tiles
// and the decode path turns MMA-bound from m = 9 upward (and latency-bound below).  Here the
// dequantised weights are the A operand of tcgen05.mma and live in tensor memory; the batch is
// the MMA's N (16 or 32), so one instruction covers 128 weight rows x 16 k for the whole batch.
//
//   producer warp  : one bulk async copy per (128-row tile, 256-k chunk): the fragment layout
//                    keeps that 16 KB slice contiguous (the copy engine pays per contiguous
//                    segment; measured: 8 x 2 KB segments per stage halve an SM's streaming rate)
//   loader warp    : x slice and scale / zero tiles with 16-byte cp.async straight into the
//                    layouts their readers want (x: 128B-swizzled K-major tensor-core operand),
//                    completion counted on the stage's mbarrier (cp.async.mbarrier.arrive)
//   8 decode warps : two groups of four warps; group i takes the 64-k blocks i and i + 2 of
//                    every chunk (two blocks per hand-off keep the per-stage bookkeeping small
//                    against the decode arithmetic - the kernel is instruction-issue bound).
//                    thread = one weight row = one TMEM lane; reads its row's packed
//                    nibbles from the fragment-ordered stage, decodes them bit-exactly (lop3 +
//                    exact .rn fp16 ops), writes 64 k of fp16 into its quarter of a TMEM A buffer
//                    with tcgen05.st
//   MMA warp       : one thread waits once per chunk and issues 16 x tcgen05.mma (M=128,
//                    N=16|32, K=16), A from TMEM, B = x tile from shared memory, fp32
//                    accumulators in TMEM; tcgen05.commit recycles A buffers and stages.
//                    A kernel that allocates tensor memory runs one CTA per SM (the occupancy
//                    calculator reports 1 whatever its other resources), so the CTA is sized to
//                    fill the SM: all 512 TMEM columns, ~220 KB of stages.
//   epilogue       : the decode warps read the accumulator with tcgen05.ld, apply bias /
//                    activation / residual, round once to fp16 and store.
//
// Work split (stream-k): the (tile, chunk) iteration space is cut into equal contiguous ranges,
// one per persistent CTA.  A CTA computes first the pieces of tiles it shares with neighbours:
// the tail piece (tile started by an earlier CTA) goes to a global fp32 slot + epoch flag
// straight away; the head piece (tile this CTA owns) stays in TMEM; then all whole tiles; at
// the very end the owner adds the other CTAs' slots - written long before, so the bounded flag
// wait does not block in practice - and stores.  Sum order is fixed (CTA order): deterministic.
//
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at small m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and the reference's GEMV /
// LowBatchGEMV schedules (python/tvm/dlight/gpu/gemv.py:216-530, low_batch_gemv.py:300-613).
#pragma once

#include <cuda.h>

#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace ug {

constexpr int kDecodeWarps = 8;                 // two groups of four (one group = 128 TMEM lanes)
constexpr int kFirstDecodeWarp = 4;             // warps 0..2: producer, MMA, loader; 3 idle; 4.. decode
constexpr int kThreads = (kFirstDecodeWarp + kDecodeWarps) * 32;
constexpr int kTileRows = 128;
constexpr int kKBlock = 64;                     // k per MMA block (4 x K=16) and per fragment tile
constexpr int kBlocksPerChunk = 4;              // 256 k per stage
constexpr int kChunk = kKBlock * kBlocksPerChunk;
constexpr int kWBlockPitch = 2048;              // 16-row block slice of a stage (4 fragment tiles)
constexpr int kWBytes = 8 * kWBlockPitch;
constexpr int kScaleBoxBytes = 2048;
constexpr int kNumA = 3;                        // TMEM A buffers, one whole 256-k chunk each (128 columns)
constexpr int kACols = 32 * kBlocksPerChunk;
constexpr int kNumD = 3;                        // accumulators: two for whole tiles, one for the owned piece
constexpr int kTmemCols = 512;                  // the whole tensor memory (one CTA per SM)

enum ScaleSrc : int { kSrcGlobal = 0, kSrcSmemNK = 1, kSrcSmemKN = 2 };

struct Params {
  GemvParams g;
  float* partial;        // [grid][nb][128] fp32 tail pieces
  unsigned* flags;       // [grid][4] epoch flags, one per lane quadrant
  unsigned epoch;
  int nb;                // MMA N: 16 or 32 (batch rows padded)
  int has_z_tile;
  unsigned s_box_bytes;
};

struct Layout {
  int x_bytes;      // nb * 128 * 4 sub-tiles
  int w_off, s_off, z_off, stage_bytes;
};
inline Layout make_layout(int nb, int src, int zmode) {
  Layout l;
  l.x_bytes = nb * 128 * kBlocksPerChunk;
  l.w_off = l.x_bytes;
  l.s_off = l.w_off + kWBytes;
  l.z_off = l.s_off + (src != kSrcGlobal ? kScaleBoxBytes : 0);
  int end = l.z_off + ((src != kSrcGlobal && zmode == kZeroGeneral) ? kScaleBoxBytes : 0);
  l.stage_bytes = ((end + 1023) / 1024) * 1024;
  return l;
}

#ifdef __CUDACC__

// ---------------------------------------------------------------- PTX wrappers
// 16-byte asynchronous copy global -> shared; bytes beyond src_bytes are written as zero
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
// the mbarrier gets one (pre-counted) arrival once all earlier cp.async of this thread have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]; kind::f16, fp32 accumulate
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ long long range_start(long long cta, long long total, long long grid) {
  return cta * total / grid;
}

// A piece of work: chunks [c0, c1) of `tile`; where the accumulator goes afterwards.
enum PieceKind : int { kWhole = 0, kTail = 1, kHead = 2 };
struct Piece {
  int tile, c0, c1, kind, dbuf;
};

// Enumerates the pieces of CTA `cta` in execution order: tail piece, head piece, whole tiles.
// Returns false when idx is past the end.  All warps of the CTA call this with the same idx.
__device__ __forceinline__ bool get_piece(long long it0, long long it1, int cpt, int idx, Piece* pc) {
  if (it0 >= it1) return false;
  const int first_tile = (int)(it0 / cpt), last_tile = (int)((it1 - 1) / cpt);
  const int fc0 = (int)(it0 % cpt);
  const int lc1 = (int)((it1 - 1) % cpt) + 1;
  // does the range begin mid-tile (tail piece of a tile owned by an earlier CTA)?
  const bool has_tail = fc0 != 0;
  // does it end mid-tile while having started that tile at chunk 0 (head piece of an owned tile)?
  const bool single = first_tile == last_tile;
  const bool has_head = lc1 != cpt && !(single && has_tail);
  int n = 0;
  if (has_tail) {
    if (idx == n) {
      pc->tile = first_tile;
      pc->c0 = fc0;
      pc->c1 = single ? lc1 : cpt;
      pc->kind = kTail;
      pc->dbuf = 0;
      return true;
    }
    ++n;
  }
  if (has_head) {
    if (idx == n) {
      pc->tile = last_tile;
      pc->c0 = 0;
      pc->c1 = lc1;
      pc->kind = kHead;
      pc->dbuf = 2;
      return true;
    }
    ++n;
  }
  const int w0 = first_tile + (has_tail ? 1 : 0);
  const int w1 = last_tile - ((has_head || (single && has_tail)) ? 1 : 0);  // inclusive
  const int wi = idx - n;
  if (w0 + wi <= w1) {
    pc->tile = w0 + wi;
    pc->c0 = 0;
    pc->c1 = cpt;
    pc->kind = kWhole;
    pc->dbuf = wi & 1;
    return true;
  }
  return false;
}

// Decodes one 64-k block (fragment tile KB of the chunk) of this thread's weight row into 32
// packed fp16 pairs.  HI (rows g+8 of the 16-row block: high nibbles) and KB are compile-time so
// that masks, shared-memory offsets and scale selectors fold into immediates.
struct RowCtx {
  const uint8_t* wblk;     // this thread's 16-row block inside the stage
  uint32_t unit_off[4];    // byte offset of unit (g, t) inside a fragment tile
  const uint8_t* s_tile;   // staged scale tile (or nullptr)
  const uint8_t* z_tile;
  uint4 nk_s, nk_z;        // kSrcSmemNK: this row's 8 group scales / zeros of the chunk
  uint32_t s_chan, z_chan; // GROUP == 0
  int row;
  int64_t n_row;
  int kb0;
};

template <int ZMODE, int GROUP, int SRC, int HI, int KB>
__device__ __forceinline__ void decode_block(const GemvParams& p, const Params& pp, const RowCtx& c,
                                             const ZeroConsts& zc, uint32_t zconst_h2, int group,
                                             uint32_t (&regs)[32]) {
  constexpr uint32_t kMagic = 0x64006400u, kSixteenth = 0x2C002C00u;
  constexpr uint32_t kMask = HI ? 0x00f000f0u : 0x000f000fu;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const uint4 u = *reinterpret_cast<const uint4*>(c.wblk + KB * 512 + c.unit_off[t]);
    uint32_t s2, z2 = zconst_h2;
    if (GROUP == 0) {
      s2 = c.s_chan;
      z2 = c.z_chan;
    } else if (SRC == kSrcSmemNK) {
      constexpr int gi = 2 * KB;  // group 32: runs t = 0,1 -> group 2KB, t = 2,3 -> group 2KB + 1
      const uint32_t wsel = (gi >> 1) == 0 ? c.nk_s.x : ((gi >> 1) == 1 ? c.nk_s.y : ((gi >> 1) == 2 ? c.nk_s.z : c.nk_s.w));
      s2 = prmt(wsel, wsel, (t >> 1) ? 0x3232u : 0x1010u);
      if (ZMODE == kZeroGeneral && pp.has_z_tile) {
        const uint32_t zsel = (gi >> 1) == 0 ? c.nk_z.x : ((gi >> 1) == 1 ? c.nk_z.y : ((gi >> 1) == 2 ? c.nk_z.z : c.nk_z.w));
        z2 = prmt(zsel, zsel, (t >> 1) ? 0x3232u : 0x1010u);
      }
    } else if (SRC == kSrcSmemKN) {
      constexpr int kG = GROUP > 0 ? GROUP : 1;
      const int gl = (KB * kKBlock + t * 16) / kG;
      s2 = h2_bcast(reinterpret_cast<const __half*>(c.s_tile)[gl * kTileRows + c.row]);
      if (ZMODE == kZeroGeneral && pp.has_z_tile)
        z2 = h2_bcast(reinterpret_cast<const __half*>(c.z_tile)[gl * kTileRows + c.row]);
    } else {
      const int64_t kk = (int64_t)(c.kb0 + KB) * kKBlock + t * 16;
      const int64_t o = c.n_row * p.s_n + (kk / group) * p.s_g;
      s2 = h2_bcast(p.s[o]);
      if (ZMODE == kZeroGeneral && p.z) z2 = h2_bcast(p.z[o]);
    }
    const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t e0 = and_or(ww[j], kMask, kMagic);
      uint32_t e1 = and_or(ww[j] >> 8, kMask, kMagic);
      if (HI) {
        e0 = h2_fma(e0, kSixteenth, zc.add_hi);
        e1 = h2_fma(e1, kSixteenth, zc.add_hi);
      } else {
        e0 = h2_sub(e0, zc.sub_lo);
        e1 = h2_sub(e1, zc.sub_lo);
      }
      if (ZMODE == kZeroGeneral) {
        e0 = h2_sub(e0, z2);
        e1 = h2_sub(e1, z2);
      }
      regs[8 * t + 2 * j] = h2_mul(e0, s2);
      regs[8 * t + 2 * j + 1] = h2_mul(e1, s2);
    }
  }
}

template <int ZMODE, int GROUP, int SRC, int HI>
__device__ __forceinline__ void decode_block_kb(int kb, const GemvParams& p, const Params& pp, const RowCtx& c,
                                                const ZeroConsts& zc, uint32_t zconst_h2, int group,
                                                uint32_t (&regs)[32]) {
  switch (kb) {
    case 0:
      decode_block<ZMODE, GROUP, SRC, HI, 0>(p, pp, c, zc, zconst_h2, group, regs);
      break;
    case 1:
      decode_block<ZMODE, GROUP, SRC, HI, 1>(p, pp, c, zc, zconst_h2, group, regs);
      break;
    case 2:
      decode_block<ZMODE, GROUP, SRC, HI, 2>(p, pp, c, zc, zconst_h2, group, regs);
      break;
    default:
      decode_block<ZMODE, GROUP, SRC, HI, 3>(p, pp, c, zc, zconst_h2, group, regs);
      break;
  }
}

template <int ZMODE, int GROUP, int SRC>
__global__ void __launch_bounds__(kThreads, 1)
    umma_gemv_kernel(const Params pp) {
  extern __shared__ uint8_t smem_raw[];
  const GemvParams& p = pp.g;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int nb = pp.nb;
  const int stages = p.stages;
  const int x_bytes = nb * 128 * kBlocksPerChunk;
  const int w_off = x_bytes;
  const int s_off = w_off + kWBytes;
  const int z_off = s_off + (SRC != kSrcGlobal ? kScaleBoxBytes : 0);
  const int stage_bytes =
      ((z_off + ((SRC != kSrcGlobal && ZMODE == kZeroGeneral) ? kScaleBoxBytes : 0) + 1023) / 1024) * 1024;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * stage_bytes);
  uint64_t* stage_full = bars;
  uint64_t* stage_empty = stage_full + stages;
  uint64_t* a_full = stage_empty + stages;
  uint64_t* a_empty = a_full + kNumA;
  uint64_t* d_full = a_empty + kNumA;
  uint64_t* d_empty = d_full + kNumD;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_empty + kNumD);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&stage_full[s], 1 + 32);            // producer's expect_tx arrival + 32 loader lanes
      mbar_init(&stage_empty[s], kDecodeWarps + 1);  // decode warps + the MMA thread's commit
    }
    for (int i = 0; i < kNumA; ++i) {
      mbar_init(&a_full[i], kDecodeWarps);
      mbar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < kNumD; ++i) {
      mbar_init(&d_full[i], 1);
      mbar_init(&d_empty[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t a_col0 = tmem_base;                  // kNumA buffers of kACols columns
  const uint32_t d_col0 = tmem_base + kNumA * kACols; // kNumD accumulators of up to 32 columns

  // x rows >= m of every stage are never written by the loader: they must read as zero
  for (int st = 0; st < stages; ++st) {
    uint4* xs = reinterpret_cast<uint4*>(smem + (size_t)st * stage_bytes);
    for (int i = tid; i < x_bytes / 16; i += kThreads) xs[i] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async();
  __syncthreads();

  const long long total = p.total_iters;
  const long long grid = gridDim.x;
#ifdef RB200_ABLATE
  const int ablate = p.ablate;
  unsigned long long* tl = (blockIdx.x == 0 && (ablate & 65536)) ? reinterpret_cast<unsigned long long*>(pp.partial) + (1 << 18) : nullptr;
#define RB200_TL(role, i)                                                          \
  do {                                                                             \
    if (tl && (i) < 256) {                                                         \
      unsigned long long t_;                                                       \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                        \
      tl[(role) * 256 + (i)] = t_;                                                 \
    }                                                                              \
  } while (0)
#else
#define RB200_TL(role, i) do {} while (0)
  constexpr int ablate = 0;
#endif
  const long long it0 = range_start(blockIdx.x, total, grid);
  const long long it1 = (ablate & 8) ? it0 : range_start(blockIdx.x + 1, total, grid);
  const int cpt = p.chunks_per_tile;
  const int kb_total = p.k / kKBlock;
  bool ok = true;

  if (warp == 0) {
    // ============================================================ producer: packed weights
    int tl_i = 0;
    (void)tl_i;
    int stage = 0;
    uint32_t phase = 0;
    Piece pc;
    for (int idx = 0; ok && get_piece(it0, it1, cpt, idx, &pc); ++idx) {
      for (int chunk = pc.c0; chunk < pc.c1; ++chunk) {
        if (!mbar_wait_parked(&stage_empty[stage], phase ^ 1u, p.status)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          RB200_TL(0, tl_i); ++tl_i;
          const int nkb = min(kBlocksPerChunk, kb_total - chunk * kBlocksPerChunk);
          const uint32_t wbytes = (uint32_t)nkb * 8 * 512;  // 8 row blocks x nkb fragment tiles, contiguous
          mbar_arrive_expect_tx(&stage_full[stage], wbytes);
          bulk_g2s(smem + (size_t)stage * stage_bytes + w_off,
                   p.w + frag_stage_offset(pc.tile, chunk, p.n / 16, kb_total), wbytes, &stage_full[stage]);
        }
        __syncwarp();
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 2) {
    // ============================================================ loader: x, scales, zero points
    int stage = 0;
    uint32_t phase = 0;
    Piece pc;
    const int j = lane >> 3, c16 = lane & 7;  // x: 64-k sub-tile and 16-byte chunk handled by this lane
    const int64_t kg = GROUP > 0 ? p.k / GROUP : 0;
    for (int idx = 0; ok && get_piece(it0, it1, cpt, idx, &pc); ++idx) {
      const int64_t n0 = (int64_t)pc.tile * kTileRows;
      for (int chunk = pc.c0; chunk < pc.c1; ++chunk) {
        if (!mbar_wait_parked(&stage_empty[stage], phase ^ 1u, p.status)) {
          ok = false;
          break;
        }
        uint8_t* sbase = smem + (size_t)stage * stage_bytes;
        // x[r, chunk*256 + lane*8 .. +8) -> sub-tile j, row r, 16-byte chunk c16 ^ (r & 7)
        const int64_t kcol = (int64_t)chunk * kChunk + lane * 8;
        const uint32_t xvalid = kcol < p.k ? 16u : 0u;
        const __half* xsrc = p.x + (xvalid ? kcol : 0);
        if (!(ablate & 16))
        for (int r = 0; r < p.m; ++r)
          cp_async16(sbase + j * nb * 128 + r * 128 + ((c16 ^ (r & 7)) << 4), xsrc + (int64_t)r * p.ldx, xvalid);
        if (ablate & 32) {
        } else if (SRC == kSrcSmemNK) {
          // [128 rows][8 groups]: 16 bytes per row, four rows per lane
          const int64_t g0 = (int64_t)chunk * 8;
          const int64_t left = (kg - g0) * 2;
          const uint32_t sv = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = lane + 32 * i;
            const int64_t o = (n0 + row) * kg + (sv ? g0 : 0);
            cp_async16(sbase + s_off + row * 16, p.s + o, sv);
            if (ZMODE == kZeroGeneral && pp.has_z_tile) cp_async16(sbase + z_off + row * 16, p.z + o, sv);
          }
        } else if (SRC == kSrcSmemKN) {
          // [groups of the chunk][128 rows]: 256 bytes per group row
          constexpr int kG = GROUP > 0 ? (kChunk / GROUP) : 1;
          for (int i = lane; i < kG * 16; i += 32) {
            const int gl = i >> 4, cc = i & 15;
            const int64_t grow = (int64_t)chunk * kG + gl;
            const uint32_t sv = grow < kg ? 16u : 0u;
            const int64_t o = (sv ? grow : 0) * p.n + n0 + cc * 8;
            cp_async16(sbase + s_off + gl * 256 + cc * 16, p.s + o, sv);
            if (ZMODE == kZeroGeneral && pp.has_z_tile) cp_async16(sbase + z_off + gl * 256 + cc * 16, p.z + o, sv);
          }
        }
        cp_async_arrive(&stage_full[stage]);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    // drain this thread's copies before the block can retire
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1) {
    // ============================================================ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((uint32_t)(nb >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t q = 0;  // running chunk counter (selects the A buffer)
      uint32_t d_uses[kNumD] = {0, 0, 0};
      Piece pc;
      for (int idx = 0; ok && get_piece(it0, it1, cpt, idx, &pc); ++idx) {
        const int db = pc.dbuf;
        if (!mbar_wait_parked(&d_empty[db], (d_uses[db] & 1u) ^ 1u, p.status)) {
          ok = false;
          break;
        }
        ++d_uses[db];
        tc_fence_after();
        const uint32_t d_tmem = d_col0 + db * 32;
        bool first = true;
        for (int chunk = pc.c0; ok && chunk < pc.c1; ++chunk, ++q) {
          if (!mbar_wait_parked(&stage_full[stage], phase, p.status)) {
            ok = false;
            break;
          }
          if (ablate & 32768) {
            mbar_arrive(&stage_empty[stage]);
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          RB200_TL(4, (int)q);
          // x was written by cp.async (generic proxy): order it before the tensor core's reads
          fence_proxy_async();
          const uint32_t ab = q % kNumA;
          if (!(ablate & 256) && !mbar_wait_parked(&a_full[ab], (q / kNumA) & 1u, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          RB200_TL(5, (int)q);
          const int nkb = min(kBlocksPerChunk, kb_total - chunk * kBlocksPerChunk);
          const uint32_t xbase = smem_u32(smem + (size_t)stage * stage_bytes);
          for (int kb = 0; kb < nkb; ++kb) {
            const uint32_t a_tmem = a_col0 + ab * kACols + kb * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if ((ablate & 4) && !(first && j == 0)) continue;
              const uint64_t bdesc = make_b_desc(xbase + kb * nb * 128 + j * 32);
              if (ablate & 131072) {  // timing probe: independent accumulators (results are not meaningful)
                tc_mma_ts(d_col0 + ((kb * 4 + j) % 6) * 16, a_tmem + j * 8, bdesc, idesc, 1u);
                continue;
              }
              tc_mma_ts(d_tmem, a_tmem + j * 8, bdesc, idesc, (first && j == 0) ? 0u : 1u);
            }
            first = false;
          }
          if (ablate & 64) {
            mbar_arrive(&a_empty[ab]);
            mbar_arrive(&stage_empty[stage]);
          } else {
            tc_commit(&a_empty[ab]);
            tc_commit(&stage_empty[stage]);
          }
          RB200_TL(6, (int)q);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        tc_commit(&d_full[db]);
      }
    }
  } else if (warp >= kFirstDecodeWarp) {
    // ============================================================ decode + epilogue warps
    const int dw = warp - kFirstDecodeWarp;
    const int grp = dw >> 2;             // this warp decodes the 64-k blocks grp and grp + 2 of every chunk
    const int w4 = warp & 3;             // TMEM lane quadrant of this warp
    const int hi = w4 & 1;               // rows g (0) or g+8 (1) of the 16-row blocks
    const int bl = (w4 >> 1) * 4 + (lane >> 3);  // 16-row block inside the tile
    const int g = lane & 7;
    const int row = 16 * bl + g + 8 * hi;       // weight row inside the tile held by this TMEM lane
    const uint32_t lane_taddr = (uint32_t)(32 * w4) << 16;
    const ZeroConsts zc = make_zero_consts(ZMODE, p.zero_const);
    const uint32_t zconst_h2 = h2_bcast(__float2half_rn(p.zero_const));
    const int group = GROUP > 0 ? GROUP : (GROUP == 0 ? p.k : p.group);
    uint32_t unit_off[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) unit_off[t] = (uint32_t)(t * 128 + ((g + 2 * t) & 7) * 16);

    int stage = 0;
    uint32_t phase = 0;
    uint32_t q = 0;
    uint32_t d_uses[kNumD] = {0, 0, 0};
    float owned[32];  // not used: the owned piece stays in TMEM (d buffer 2)
    (void)owned;
    Piece pc;
    bool have_head = false;
    int head_tile = 0;
    for (int idx = 0; ok && get_piece(it0, it1, cpt, idx, &pc); ++idx) {
      const int64_t n_row = (int64_t)pc.tile * kTileRows + row;
      uint32_t s_chan = 0, z_chan = zconst_h2;
      if (GROUP == 0) {
        s_chan = h2_bcast(p.s[n_row * p.s_n]);
        if (ZMODE == kZeroGeneral && p.z) z_chan = h2_bcast(p.z[n_row * p.s_n]);
      }
      for (int chunk = pc.c0; ok && chunk < pc.c1; ++chunk) {
        if (!mbar_wait_parked(&stage_full[stage], phase, p.status)) {
          ok = false;
          break;
        }
        if (ablate & 16384) {
          ++q;
          __syncwarp();
          if (lane == 0) mbar_arrive(&stage_empty[stage]);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
          continue;
        }
        if (warp == kFirstDecodeWarp && lane == 0) RB200_TL(1, (int)q);
        const int kb0 = chunk * kBlocksPerChunk;
        const int nkb = min(kBlocksPerChunk, kb_total - kb0);
        const uint8_t* sbase = smem + (size_t)stage * stage_bytes;
        RowCtx c;
        c.wblk = sbase + w_off + bl * (nkb * 512);
#pragma unroll
        for (int t = 0; t < 4; ++t) c.unit_off[t] = unit_off[t];
        c.s_tile = sbase + s_off;
        c.z_tile = sbase + z_off;
        c.nk_s = make_uint4(0, 0, 0, 0);
        c.nk_z = make_uint4(0, 0, 0, 0);
        if (SRC == kSrcSmemNK) {
          c.nk_s = *reinterpret_cast<const uint4*>(sbase + s_off + row * 16);
          if (ZMODE == kZeroGeneral && pp.has_z_tile) c.nk_z = *reinterpret_cast<const uint4*>(sbase + z_off + row * 16);
        }
        c.s_chan = s_chan;
        c.z_chan = z_chan;
        c.row = row;
        c.n_row = n_row;
        c.kb0 = kb0;
        const int nkb_c = nkb;
        const uint32_t ab = q % kNumA;
        if (!(ablate & 256) && !mbar_wait_parked(&a_empty[ab], ((q / kNumA) & 1u) ^ 1u, p.status)) {
          ok = false;
          break;
        }
        if (warp == kFirstDecodeWarp && lane == 0) RB200_TL(2, (int)q);
        ++q;
        tc_fence_after();
#pragma unroll 1
        for (int kb = grp; kb < nkb_c; kb += 2) {
          uint32_t regs[32];
          if (ablate & 1) {
#pragma unroll
            for (int t = 0; t < 32; ++t) regs[t] = 0x3c003c00u;
          } else if (hi) {
            decode_block_kb<ZMODE, GROUP, SRC, 1>(kb, p, pp, c, zc, zconst_h2, group, regs);
          } else {
            decode_block_kb<ZMODE, GROUP, SRC, 0>(kb, p, pp, c, zc, zconst_h2, group, regs);
          }
          if (!(ablate & 2)) tc_st32(lane_taddr | (a_col0 + ab * kACols + kb * 32), regs);
        }
        if (!(ablate & 2)) tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (warp == kFirstDecodeWarp && lane == 0) RB200_TL(3, (int)q - 1);
        if (lane == 0) {
          if (!(ablate & 256)) mbar_arrive(&a_full[ab]);
          mbar_arrive(&stage_empty[stage]);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      // ---------------------------------------------------------- accumulator hand-over
      const int db = pc.dbuf;
      if (pc.kind == kHead) {  // stays in TMEM until the fix-up at the end
        have_head = true;
        head_tile = pc.tile;
        ++d_uses[db];
        continue;
      }
      // one group drains a given accumulator: whole tiles alternate, tail pieces group 0
      const int drain_grp = (pc.kind == kWhole) ? (db & 1) : 0;
      const uint32_t use = d_uses[db]++;
      if (grp != drain_grp) continue;
      if (!mbar_wait_parked(&d_full[db], use & 1u, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_taddr = lane_taddr | (d_col0 + db * 32);
      const int64_t n_out = (int64_t)pc.tile * kTileRows + row;
      for (int c0 = 0; c0 < nb; c0 += 16) {
        float v[16];
        tc_ld16(d_taddr + c0, v);
        if (pc.kind == kTail) {
          float* dst = pp.partial + ((size_t)blockIdx.x * nb + c0) * kTileRows + row;
#pragma unroll
          for (int i = 0; i < 16; ++i) dst[(size_t)i * kTileRows] = v[i];
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c0 + i;
            if (m < p.m) p.out[(int64_t)m * p.ldo + n_out] = __float2half_rn(apply_epilogue(v[i], p.epi, m, n_out));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&d_empty[db]);
      if (pc.kind == kTail) {
        // publish per warp: the owner's lane quadrant w4 reads exactly the rows this warp wrote
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_u32(pp.flags + blockIdx.x * 4 + w4, pp.epoch);
      }
    }

    // ------------------------------------------------------------ fix-up of the owned tile
    if (ok && have_head && grp == 1) {
      const int db = 2;
      if (mbar_wait_parked(&d_full[db], 0u, p.status)) {
        tc_fence_after();
        // contributors: the CTAs after this one whose range reaches into head_tile
        const long long hi_it = (long long)head_tile * cpt + cpt - 1;
        const int last_cta = (int)(((hi_it + 1) * grid - 1) / total);
        const uint32_t d_taddr = lane_taddr | (d_col0 + db * 32);
        const int64_t n_out = (int64_t)head_tile * kTileRows + row;
        bool flags_ok = true;
        for (int c = blockIdx.x + 1; c <= last_cta && flags_ok; ++c) {
          const long long t0 = clock64();
          while (ld_acquire_u32(pp.flags + c * 4 + w4) != pp.epoch) {
            if (clock64() - t0 > (1ll << 31)) {
              if (p.status) atomicExch(p.status, kStatusWaitTimeout);
              flags_ok = false;
              break;
            }
          }
        }
        if (flags_ok) {
          for (int c0 = 0; c0 < nb; c0 += 16) {
            float v[16];
            tc_ld16(d_taddr + c0, v);
            for (int c = blockIdx.x + 1; c <= last_cta; ++c) {
              const float* src = pp.partial + ((size_t)c * nb + c0) * kTileRows + row;
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] += __ldcg(src + (size_t)i * kTileRows);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int m = c0 + i;
              if (m < p.m) p.out[(int64_t)m * p.ldo + n_out] = __float2half_rn(apply_epilogue(v[i], p.epi, m, n_out));
            }
          }
        }
        tc_fence_before();
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

#endif  // __CUDACC__

}  // namespace ug

// Host entry: plans and launches the tcgen05 decode kernel.  Returns 1 when the problem is
// outside what this kernel covers (caller falls back to the warp-MMA kernel), 0 on launch,
// -1 on error.
int umma_gemv_run(const GemvParams& p, int bits, int zmode, int sm_count, float* partial,
                  size_t partial_bytes, unsigned* flags, size_t flag_count, unsigned epoch,
                  cudaStream_t stream);

}  // namespace rb200
