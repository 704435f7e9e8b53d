// Prefill kernel (m > 32): dense contraction on the 5th-generation tensor cores.
//
//   out^T tile [128 weight rows x up to 256 batch rows] = W_tile [128 x K] * x_tile^T [K x 256]
//
// Measured on B200: one tcgen05.mma (kind::f16, M = 128, K = 16, A from tensor memory) occupies
// the tensor pipe for 108 clocks for any N up to 192 and for 136 clocks at N = 256, so the batch
// is the instruction's N and is made as wide as it goes (256): one instruction then does
// 128 x 256 x 16 MACs.  The dequantised weights are the A operand and never touch shared memory:
// decode warps write them straight into tensor memory (tcgen05.st), the MMA reads A from TMEM and
// B (= x) from a 128B-swizzled K-major tile in shared memory, the fp32 accumulator sits in 256
// TMEM columns.
//
// What bounds it (m 2048 x k 4096 x n 22016, group 128 with zero points; timed by CUDA events):
//  * launched back to back for a second the kernel sits on the 1000 W power cap (sw_power_cap
//    active, SM clock 1.55-1.65 GHz): 395 us per launch; a burst of 20 launches runs 345 us.
//  * with the MMA issuer not waiting for the decode warps (same work, no dependency) a launch
//    takes 7 % less; without decode work at all (x stream + MMA + epilogue) 249 us, without
//    the epilogue too 215 us.
//  * variants measured slower in the burst: N = 192 with two accumulators (the epilogue
//    overlapping the next tile) 874 against 1065 TFLOP/s; a pair of weight tiles per CTA against
//    the same x stages (half the x bytes from L2) 404 us; four decode groups with eight A
//    buffers 358 us; spinning instead of parked waits on the A hand-off 359 us; requesting the
//    accumulator columns of the next epilogue step before working on the current one 345 us
//    (no change).
//
//   warp 0 (producer)  : packed weights, one 16 KB bulk copy per (128-row tile, 4 fragment tiles)
//   warp 1 (MMA)       : one thread, 4 x tcgen05.mma per 64-k block; commits recycle A buffers
//                        and x stages; the commit after the last block hands over the accumulator
//   warp 2 (scales)    : scale / zero tiles of the chunk with 16-byte cp.async (when staged)
//   warp 3 (x)         : one TMA tile load per 64-k block: box 64 k x nb batch rows, 128-byte
//                        swizzle = the tensor core's K-major operand layout; rows past m read zero
//   warps 4..11        : two groups of four warps (128 TMEM lanes each) decode alternate 64-k
//                        blocks; thread = weight row; bit-exact decode, tcgen05.st into one of
//                        four 32-column A buffers.  After the last block the same warps drain
//                        the accumulator (group 0: batch columns [0, nb/2), group 1: the rest),
//                        apply bias / activation / residual, round once to fp16 and store.
// Tiles are walked persistently, batch tiles fastest, so CTAs running together share a weight
// tile in L2.  Every wait is bounded and reports through the device status word.
//
// Stands in for fastertransformer::gemm_fp16_int_bias_act[_residual] at large m
// (python/tvm/contrib/cutlass/gemm_operation.py:441-458) and the reference's tensor-core matmul
// schedule (python/tvm/dlight/gpu/matmul.py:316-535).
#pragma once

#include <cuda.h>

#include "dequant.cuh"
#include "gemv.h"
#include "gemv_cluster.cuh"
#include "umma_common.cuh"

namespace rb200 {
namespace um {

constexpr int kDecodeWarps = 8;
constexpr int kFirstDecodeWarp = 4;
constexpr int kThreads = (kFirstDecodeWarp + kDecodeWarps) * 32;
constexpr int kTileRows = 128;
constexpr int kKBlock = 64;                 // k per MMA block (4 x K=16)
constexpr int kWBytes = 8 * 4 * 512;        // one weight stage: 8 row blocks x 4 fragment tiles
constexpr int kScaleBoxBytes = 2048;
constexpr int kWStageBytes = kWBytes + 2 * kScaleBoxBytes;
constexpr int kWStages = 3;
constexpr int kMaxXStages = 8;
constexpr int kNumA = 4;                    // TMEM A buffers of 32 columns (one 64-k block each)
constexpr int kTmemCols = 512;
constexpr int kDCols = 256;                 // accumulator: columns [0, 256); A buffers follow
constexpr int kMaxNb = 256;
constexpr int kEpiStageBytes = 2 * 2 * 16 * kTileRows * 2;  // per group: two 16 x 128 fp16 buffers

constexpr int kMaxExperts = 64;

struct Params {
  GemvParams g;
  int nb;          // batch rows per tile = MMA N (multiple of 32, <= 256)
  int x_stages;
  int has_z_tile;
  // grouped form: rows [indptr[e-1], indptr[e]) of x / out belong to expert e (indptr: device,
  // end offsets); indptr == nullptr: one group holding all g.m rows
  const int64_t* indptr;
  int indptr_has_prev;      // the first group starts at indptr[-1] (a sub-range of a longer table), not at row 0
  int num_experts;
  int64_t w_expert_bytes;   // bytes between experts' packed weights
  int64_t s_expert_stride;  // elements between experts' scale (and zero) tensors
  // split-k (ungrouped form with fewer tiles than SMs): every tile is cut into k_splits equal k
  // ranges run by different CTAs; fp32 partial tiles meet in `partial`, the group of warps that
  // arrives last (ticket per tile and column half) adds them in split order and stores
  int k_splits;
  float* partial;           // [tiles * k_splits][nb][128] fp32
  int* tickets;             // [tiles * 2], zero at rest
};

inline size_t smem_bytes(int nb, int x_stages) {
  return 1024 + (size_t)x_stages * nb * 128 + (size_t)kWStages * kWStageBytes + kEpiStageBytes +
         (size_t)(2 * kWStages + 2 * kMaxXStages + 2 * kNumA + 4) * 8 + 16 + (3 * kMaxExperts + 4) * sizeof(int);
}

#ifdef __CUDACC__

// hand-offs on the critical path (A buffers, x stages)
__device__ __forceinline__ bool um_wait(uint64_t* bar, uint32_t parity, int* status) {
  return mbar_wait_parked(bar, parity, status);
}

using gc::tma_load_2d;
using ug::cp_async16;
using ug::cp_async_arrive;
using ug::kSrcGlobal;
using ug::kSrcSmemKN;
using ug::kSrcSmemNK;
using ug::make_b_desc;
using ug::RowCtx;
using ug::tc_commit;
using ug::tc_fence_after;
using ug::tc_fence_before;
using ug::tc_ld16;
using ug::tc_mma_ts;
using ug::tc_st32;
using ug::tc_wait_st;
using ug::tmem_alloc;
using ug::tmem_dealloc;
using ug::tmem_relinquish;

// int8: one 64-k MMA block = two 32-k fragment tiles.  Unit (g, t) of a tile holds, for row
// g + 8 HI, the words 2j + HI (j = 0, 1) = k 8t + 4j .. + 3 in byte order.
template <int ZMODE, int GROUP, int HI, int KBM>
__device__ __forceinline__ void decode_block8(const GemvParams& p, const RowCtx& c, const ZeroConsts& zc,
                                              uint32_t zconst_h2, int group, uint32_t (&regs)[32]) {
  constexpr uint32_t kMagicBytes = 0x64646464u;
#pragma unroll
  for (int ti = 0; ti < 2; ++ti) {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const uint4 u = *reinterpret_cast<const uint4*>(c.wblk + (KBM * 2 + ti) * 512 + c.unit_off[t]);
      uint32_t s2, z2 = zconst_h2;
      if (GROUP == 0) {
        s2 = c.s_chan;
        z2 = c.z_chan;
      } else {
        const int64_t kk = (int64_t)(c.kb0 + KBM) * kKBlock + ti * 32 + t * 8;
        const int64_t o = c.n_row * p.s_n + (kk / group) * p.s_g;
        s2 = h2_bcast(p.s[o]);
        if (ZMODE == kZeroGeneral && p.z) z2 = h2_bcast(p.z[o]);
      }
      const uint32_t w0 = HI ? u.y : u.x, w1 = HI ? u.w : u.z;
      const uint32_t ww[2] = {w0, w1};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t e0 = h2_sub(prmt(ww[j], kMagicBytes, 0x4140u), zc.sub_lo);
        uint32_t e1 = h2_sub(prmt(ww[j], kMagicBytes, 0x4342u), zc.sub_lo);
        if (ZMODE == kZeroGeneral) {
          e0 = h2_sub(e0, z2);
          e1 = h2_sub(e1, z2);
        }
        regs[16 * ti + 4 * t + 2 * j] = h2_mul(e0, s2);
        regs[16 * ti + 4 * t + 2 * j + 1] = h2_mul(e1, s2);
      }
    }
  }
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; kind::f16, fp32 accumulate
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

// Work item: one (expert, 128-row weight tile, batch tile).  Items are numbered expert by expert,
// batch tiles fastest; the tables live in shared memory (built once per CTA from indptr).
struct Tile {
  int e, n_tile;
  int m0, m_end;  // first batch row of the tile, end of the expert's rows
};
struct TileTables {
  int base[kMaxExperts + 1];
  int row_begin[kMaxExperts];
  int row_end[kMaxExperts];
};
__device__ __forceinline__ Tile get_tile(const TileTables& tt, int num_experts, int nb, int t) {
  int e = 0;
  while (e + 1 < num_experts && t >= tt.base[e + 1]) ++e;
  const int local = t - tt.base[e];
  const int rows = tt.row_end[e] - tt.row_begin[e];
  const int mt = (rows + nb - 1) / nb;
  Tile tl;
  tl.e = e;
  tl.n_tile = local / mt;
  tl.m0 = tt.row_begin[e] + (local % mt) * nb;
  tl.m_end = tt.row_end[e];
  return tl;
}

template <int BITS, int ZMODE, int GROUP, int SRC, int HI>
__device__ __forceinline__ void decode_any(int kbm, const GemvParams& p, bool has_z_tile, const RowCtx& c,
                                           const ZeroConsts& zc, uint32_t zconst_h2, int group,
                                           uint32_t (&regs)[32]) {
  if constexpr (BITS == 4) {
    ug::decode_block_kb<ZMODE, GROUP, SRC, HI>(kbm, p, has_z_tile, c, zc, zconst_h2, group, regs);
  } else {
    if (kbm == 0) decode_block8<ZMODE, GROUP, HI, 0>(p, c, zc, zconst_h2, group, regs);
    else decode_block8<ZMODE, GROUP, HI, 1>(p, c, zc, zconst_h2, group, regs);
  }
}

// SPLITK: compiled separately so that the unsplit kernel carries none of the reduction code
// (with it, its epilogue was about 1 us per tile slower).
template <int BITS, int ZMODE, int GROUP, int SRC, bool SPLITK>
__global__ void __launch_bounds__(kThreads, 1)
    umma_gemm_kernel(const Params pp, const __grid_constant__ CUtensorMap tmap_x,
                     const __grid_constant__ CUtensorMap tmap_w) {
  // BITS == 16: dense fp16 weights [E, N, K]; a weight stage is one 128 x 64 tile loaded by TMA
  // in the tensor core's swizzled K-major layout and the MMA takes both operands from shared
  // memory; the decode warps only run the epilogue.
  constexpr bool kDense = BITS == 16;
  constexpr int kTilesPerBlock = BITS == 8 ? 2 : 1;       // fragment tiles per 64-k MMA block
  constexpr int kBlocksPerChunk = kDense ? 1 : 4 / kTilesPerBlock;  // MMA blocks per weight stage
  constexpr int kFragK = BITS == 8 ? 32 : 64;
  extern __shared__ uint8_t smem_raw[];
  const GemvParams& p = pp.g;
  // 1 KB alignment as an offset from the array (a pointer rebuilt from an integer would turn
  // every shared-memory access of the decode warps into a generic one)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nb = pp.nb;
  const int x_stages = pp.x_stages;
  const int x_stage_bytes = nb * 128;
  uint8_t* x_ring = smem;
  uint8_t* w_ring = smem + (size_t)x_stages * x_stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(w_ring + (size_t)kWStages * kWStageBytes + kEpiStageBytes);
  uint64_t* w_full = bars;
  uint64_t* w_empty = w_full + kWStages;
  uint64_t* x_full = w_empty + kWStages;
  uint64_t* x_empty = x_full + kMaxXStages;
  uint64_t* a_full = x_empty + kMaxXStages;
  uint64_t* a_empty = a_full + kNumA;
  uint64_t* d_full = a_empty + kNumA;
  uint64_t* d_empty = d_full + 1;
  uint64_t* e_bar = d_empty + 1;  // one per decode group: epilogue staging hand-over
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(e_bar + 2);
  TileTables& tt = *reinterpret_cast<TileTables*>(tmem_holder + 4);
  volatile int* s_last = reinterpret_cast<volatile int*>(tmem_holder + 2);  // split-k: one flag per decode group
  __half* e_stage = reinterpret_cast<__half*>(w_ring + (size_t)kWStages * kWStageBytes);  // [2 groups][2][16][128]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < kWStages; ++s) {
      mbar_init(&w_full[s], 1 + (SRC != kSrcGlobal ? 32 : 0));  // expect_tx arrival (+ scale loader lanes)
      mbar_init(&w_empty[s], kDense ? 1 : kDecodeWarps);
    }
    for (int s = 0; s < x_stages; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 1);
    }
    for (int i = 0; i < kNumA; ++i) {
      mbar_init(&a_full[i], 4);
      mbar_init(&a_empty[i], 1);
    }
    mbar_init(d_full, 1);
    mbar_init(d_empty, kDecodeWarps);
    mbar_init(&e_bar[0], 4);
    mbar_init(&e_bar[1], 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  const int n_tiles = p.n / kTileRows;
  if (tid < pp.num_experts) {
    const int64_t r0 = pp.indptr ? ((tid || pp.indptr_has_prev) ? pp.indptr[tid - 1] : 0) : 0;
    int64_t r1 = pp.indptr ? pp.indptr[tid] : p.m;
    if (r1 > p.m) r1 = p.m;  // never past the rows x / out hold
    tt.row_begin[tid] = (int)r0;
    tt.row_end[tid] = r1 > r0 ? (int)r1 : (int)r0;
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < pp.num_experts; ++e) {
      tt.base[e] = acc;
      acc += n_tiles * ((tt.row_end[e] - tt.row_begin[e] + pp.nb - 1) / pp.nb);
    }
    tt.base[pp.num_experts] = acc;
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t d_col0 = tmem_base;
  const uint32_t a_col0 = tmem_base + kDCols;

  const int kb_total = p.k / kKBlock;             // MMA blocks along k
  const int ft_total = p.k / kFragK;              // fragment tiles along k
  const int chunks = kDense ? kb_total : (ft_total + 3) / 4;  // weight stages per tile
  const int S = SPLITK ? pp.k_splits : 1;                      // 1 unless split-k
  const int total_tiles = tt.base[pp.num_experts] * S;          // work items: (tile, split), split fastest
  const int ne = pp.num_experts;
  // split sp covers the weight stages [sp * chunks / S, (sp + 1) * chunks / S) and their MMA blocks
  auto ch_lo = [&](int sp) { return (int)((long long)sp * chunks / S); };
  auto kb_lo = [&](int sp) { return min(ch_lo(sp) * kBlocksPerChunk, kb_total); };
  bool ok = true;

  if (warp == 0) {
    // ============================================================ producer: packed weights
    int ws = 0;
    uint32_t wph = 0;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const Tile tile = get_tile(tt, ne, nb, t / S);
      const uint8_t* w_e = p.w + (int64_t)tile.e * pp.w_expert_bytes;
      for (int chunk = ch_lo(t % S); chunk < ch_lo(t % S + 1); ++chunk) {
        if (!mbar_wait_parked(&w_empty[ws], wph ^ 1u, p.status)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          if (kDense) {
            mbar_arrive_expect_tx(&w_full[ws], (uint32_t)kWBytes);
            tma_load_3d(w_ring + (size_t)ws * kWStageBytes, &tmap_w, chunk * kKBlock, tile.n_tile * kTileRows, tile.e,
                        &w_full[ws]);
          } else {
            const int nft = min(4, ft_total - chunk * 4);
            const uint32_t wbytes = (uint32_t)nft * 8 * 512;
            mbar_arrive_expect_tx(&w_full[ws], wbytes);
            bulk_g2s(w_ring + (size_t)ws * kWStageBytes, w_e + frag_stage_offset(tile.n_tile, chunk, p.n / 16, ft_total),
                     wbytes, &w_full[ws]);
          }
        }
        __syncwarp();
        if (++ws == kWStages) {
          ws = 0;
          wph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ============================================================ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((uint32_t)(nb >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int xs = 0;
      uint32_t xph = 0;
      uint32_t q = 0;       // running 64-k block counter (selects the A buffer)
      uint32_t tile_i = 0;  // tiles done by this CTA
      int ws = 0;
      uint32_t wph = 0;
      (void)ws;
      (void)wph;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++tile_i) {
        if (!mbar_wait_parked(d_empty, (tile_i & 1u) ^ 1u, p.status)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int kb_first = kb_lo(t % S), kb_end = kb_lo(t % S + 1);
        for (int kb = kb_first; kb < kb_end; ++kb, ++q) {
          if (!um_wait(&x_full[xs], xph, p.status)) {
            ok = false;
            break;
          }
          const uint32_t ab = q % kNumA;
          if (kDense) {
            if (!um_wait(&w_full[ws], wph, p.status)) {
              ok = false;
              break;
            }
          } else if (!um_wait(&a_full[ab], (q / kNumA) & 1u, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t xbase = smem_u32(x_ring + (size_t)xs * x_stage_bytes);
          if (kDense) {
            const uint32_t wbase = smem_u32(w_ring + (size_t)ws * kWStageBytes);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_mma_ss(d_col0, make_b_desc(wbase + j * 32), make_b_desc(xbase + j * 32), idesc,
                        (kb == kb_first && j == 0) ? 0u : 1u);
            tc_commit(&w_empty[ws]);
            if (++ws == kWStages) {
              ws = 0;
              wph ^= 1u;
            }
          } else {
            const uint32_t a_tmem = a_col0 + ab * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              tc_mma_ts(d_col0, a_tmem + j * 8, make_b_desc(xbase + j * 32), idesc, (kb == kb_first && j == 0) ? 0u : 1u);
            tc_commit(&a_empty[ab]);
          }
          tc_commit(&x_empty[xs]);
          if (++xs == x_stages) {
            xs = 0;
            xph ^= 1u;
          }
        }
        if (ok) tc_commit(d_full);
      }
    }
  } else if (warp == 2) {
    // ============================================================ scale / zero tiles of each chunk
    if (SRC != kSrcGlobal && !kDense) {
      int ws = 0;
      uint32_t wph = 0;
      const int64_t kg = GROUP > 0 ? p.k / GROUP : 0;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const Tile tile = get_tile(tt, ne, nb, t / S);
        const int64_t n0 = (int64_t)tile.n_tile * kTileRows;
        const __half* s_e = p.s + (int64_t)tile.e * pp.s_expert_stride;
        const __half* z_e = p.z ? p.z + (int64_t)tile.e * pp.s_expert_stride : nullptr;
        for (int chunk = ch_lo(t % S); chunk < ch_lo(t % S + 1); ++chunk) {
          if (!mbar_wait_parked(&w_empty[ws], wph ^ 1u, p.status)) {
            ok = false;
            break;
          }
          uint8_t* wsb = w_ring + (size_t)ws * kWStageBytes;
          if (SRC == kSrcSmemNK) {
            // [128 rows][8 groups of 32]: 16 bytes per row, four rows per lane
            const int64_t g0 = (int64_t)chunk * 8;
            const int64_t left = (kg - g0) * 2;
            const uint32_t sv = left >= 16 ? 16u : (left > 0 ? (uint32_t)left : 0u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = lane + 32 * i;
              const int64_t o = (n0 + row) * kg + (sv ? g0 : 0);
              cp_async16(wsb + kWBytes + row * 16, s_e + o, sv);
              if (ZMODE == kZeroGeneral && pp.has_z_tile) cp_async16(wsb + kWBytes + kScaleBoxBytes + row * 16, z_e + o, sv);
            }
          } else {
            // [groups of the chunk][128 rows]: 256 bytes per group row
            constexpr int kG = GROUP > 0 ? (256 / GROUP) : 1;
            for (int i = lane; i < kG * 16; i += 32) {
              const int gl = i >> 4, cc = i & 15;
              const int64_t grow = (int64_t)chunk * kG + gl;
              const uint32_t sv = grow < kg ? 16u : 0u;
              const int64_t o = (sv ? grow : 0) * p.n + n0 + cc * 8;
              cp_async16(wsb + kWBytes + gl * 256 + cc * 16, s_e + o, sv);
              if (ZMODE == kZeroGeneral && pp.has_z_tile)
                cp_async16(wsb + kWBytes + kScaleBoxBytes + gl * 256 + cc * 16, z_e + o, sv);
            }
          }
          cp_async_arrive(&w_full[ws]);
          if (++ws == kWStages) {
            ws = 0;
            wph ^= 1u;
          }
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
  } else if (warp == 3) {
    // ============================================================ x tiles (TMA)
    int xs = 0;
    uint32_t xph = 0;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const int m0 = get_tile(tt, ne, nb, t / S).m0;
      for (int kb = kb_lo(t % S); kb < kb_lo(t % S + 1); ++kb) {
        if (!mbar_wait_parked(&x_empty[xs], xph ^ 1u, p.status)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(&x_full[xs], (uint32_t)x_stage_bytes);
          tma_load_2d(x_ring + (size_t)xs * x_stage_bytes, &tmap_x, kb * kKBlock, m0, &x_full[xs]);
        }
        __syncwarp();
        if (++xs == x_stages) {
          xs = 0;
          xph ^= 1u;
        }
      }
    }
  } else {
    // ============================================================ decode + epilogue warps
    const int dw = warp - kFirstDecodeWarp;
    const int grp = dw >> 2;
    const int w4 = warp & 3;             // TMEM lane quadrant of this warp
    const int hi = w4 & 1;               // rows g (0) or g+8 (1) of the 16-row blocks
    const int bl = (w4 >> 1) * 4 + (lane >> 3);
    const int g = lane & 7;
    // weight row held by this thread's TMEM lane: the decode order for packed weights, the
    // natural order when the A operand came from a TMA tile
    const int row = kDense ? 32 * w4 + lane : 16 * bl + g + 8 * hi;
    const uint32_t lane_taddr = (uint32_t)(32 * w4) << 16;
    const ZeroConsts zc = make_zero_consts(ZMODE, p.zero_const);
    const uint32_t zconst_h2 = h2_bcast(__float2half_rn(p.zero_const));
    const int group = GROUP > 0 ? GROUP : (GROUP == 0 ? p.k : p.group);
    uint32_t unit_off[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) unit_off[t] = (uint32_t)(t * 128 + ((g + 2 * t) & 7) * 16);
    const bool has_z_tile = pp.has_z_tile != 0;

    int ws = 0;
    uint32_t wph = 0;
    uint32_t q = 0;
    uint32_t tile_i = 0;
    uint32_t estep = 0;  // epilogue staging steps done by this group
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x, ++tile_i) {
      const Tile tile = get_tile(tt, ne, nb, t / S);
      const int split = t % S;
      const int n_tile = tile.n_tile;
      const int64_t n_row = (int64_t)n_tile * kTileRows + row;
      // row index for scale / zero addressing: the expert's offset folded in (the host checks that
      // the expert stride is a multiple of the row stride)
      const int64_t n_row_s = kDense ? 0 : n_row + (int64_t)tile.e * (pp.s_expert_stride / (p.s_n ? p.s_n : 1));
      uint32_t s_chan = 0, z_chan = zconst_h2;
      if (GROUP == 0 && !kDense) {
        s_chan = h2_bcast(p.s[n_row_s * p.s_n]);
        if (ZMODE == kZeroGeneral && p.z) z_chan = h2_bcast(p.z[n_row_s * p.s_n]);
      }
      for (int chunk = ch_lo(split); chunk < (kDense ? 0 : ch_lo(split + 1)) && ok; ++chunk) {
        if (!mbar_wait_parked(&w_full[ws], wph, p.status)) {
          ok = false;
          break;
        }
        const int nft = min(4, ft_total - chunk * 4);
        const int nblk = nft / kTilesPerBlock;
        const uint8_t* wsb = w_ring + (size_t)ws * kWStageBytes;
        RowCtx c;
        c.wblk = wsb + bl * (nft * 512);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) c.unit_off[tt] = unit_off[tt];
        c.s_tile = wsb + kWBytes;
        c.z_tile = wsb + kWBytes + kScaleBoxBytes;
        c.nk_s = make_uint4(0, 0, 0, 0);
        c.nk_z = make_uint4(0, 0, 0, 0);
        if (SRC == kSrcSmemNK) {
          c.nk_s = *reinterpret_cast<const uint4*>(c.s_tile + row * 16);
          if (ZMODE == kZeroGeneral && pp.has_z_tile) c.nk_z = *reinterpret_cast<const uint4*>(c.z_tile + row * 16);
        }
        c.s_chan = s_chan;
        c.z_chan = z_chan;
        c.row = row;
        c.n_row = n_row_s;
        c.kb0 = chunk * kBlocksPerChunk;
#pragma unroll 1
        for (int kbm = 0; kbm < nblk; ++kbm, ++q) {
          if ((int)(q & 1u) != grp) continue;
          const uint32_t ab = q % kNumA;
          if (!um_wait(&a_empty[ab], ((q / kNumA) & 1u) ^ 1u, p.status)) {
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t regs[32];
          if (hi) decode_any<BITS, ZMODE, GROUP, SRC, 1>(kbm, p, has_z_tile, c, zc, zconst_h2, group, regs);
          else decode_any<BITS, ZMODE, GROUP, SRC, 0>(kbm, p, has_z_tile, c, zc, zconst_h2, group, regs);
          tc_st32(lane_taddr | (a_col0 + ab * 32), regs);
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[ab]);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&w_empty[ws]);
        if (++ws == kWStages) {
          ws = 0;
          wph ^= 1u;
        }
      }
      if (!ok) break;
      // ---------------------------------------------------------- epilogue of this tile
      if (!mbar_wait_parked(d_full, tile_i & 1u, p.status)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int64_t m0 = tile.m0;
      const int64_t m_end = tile.m_end;
      const int c_begin = grp * (nb / 2), c_end = c_begin + nb / 2;
      const int gj = (dw & 3) * 32 + lane;  // thread index inside the group
      const int lrow = 32 * w4 + lane;      // TMEM lane: position of this thread's row in a partial tile
      bool reduce_here = true;
      if (SPLITK && S > 1) {
        // publish this CTA's partial columns, then take a ticket for (tile, column half)
        float* slot = pp.partial + ((size_t)(t / S) * S + split) * (size_t)nb * kTileRows;
        for (int c0 = c_begin; c0 < c_end; c0 += 16) {
          if (m0 + c0 >= m_end) break;
          float v[16];
          tc_ld16(lane_taddr | (d_col0 + c0), v);
#pragma unroll
          for (int i = 0; i < 16; ++i) slot[(size_t)(c0 + i) * kTileRows + lrow] = v[i];
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(&e_bar[grp]);
        if (!mbar_wait_parked(&e_bar[grp], estep & 1u, p.status)) {
          ok = false;
          break;
        }
        ++estep;
        if ((dw & 3) == 0 && lane == 0) {
          const int prev = atomicAdd(&pp.tickets[(t / S) * 2 + grp], 1);
          s_last[grp] = (prev == S - 1) ? 1 : 0;
          if (prev == S - 1) pp.tickets[(t / S) * 2 + grp] = 0;  // at rest again for the next launch
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&e_bar[grp]);
        if (!mbar_wait_parked(&e_bar[grp], estep & 1u, p.status)) {
          ok = false;
          break;
        }
        ++estep;
        reduce_here = s_last[grp] != 0;
        if (reduce_here) __threadfence();
      }
      for (int c0 = c_begin; reduce_here && c0 < c_end; c0 += 16, ++estep) {
        if (m0 + c0 >= m_end) break;
        float v[16];
        tc_ld16(lane_taddr | (d_col0 + c0), v);
        if (SPLITK && S > 1) {
          // all splits in split order, this CTA's own part straight from tensor memory
          float acc[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
          for (int sp = 0; sp < S; ++sp) {
            if (sp == split) {
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] += v[i];
            } else {
              const float* other = pp.partial + ((size_t)(t / S) * S + sp) * (size_t)nb * kTileRows;
#pragma unroll
              for (int i = 0; i < 16; ++i) acc[i] += __ldcg(other + (size_t)(c0 + i) * kTileRows + lrow);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = acc[i];
        }
        // transpose through shared memory: 16 batch rows x 128 weight rows of fp16 (rounded once,
        // after the epilogue), so that global stores are whole 256-byte row segments
        __half* st = e_stage + ((grp * 2 + (estep & 1u)) * 16) * kTileRows;
        apply_epilogue16(v, p.epi, m0 + c0, m_end, n_row);
#pragma unroll
        for (int i = 0; i < 16; ++i) st[i * kTileRows + row] = __float2half_rn(v[i]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&e_bar[grp]);
        if (!mbar_wait_parked(&e_bar[grp], estep & 1u, p.status)) {
          ok = false;
          break;
        }
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int mi = pass * 8 + (gj >> 4), ch = gj & 15;
          const int64_t m = m0 + c0 + mi;
          if (p.epi.act == kActSwiglu) {
            // interleaved repack: 16-byte chunk 2q of a staged row holds gate_f, chunk 2q+1 up_f for
            // the same eight f; the even-chunk threads combine them and store 16 bytes of [m, n/2]
            if (m < m_end && (ch & 1) == 0) {
              const uint4 gv = *reinterpret_cast<const uint4*>(st + mi * kTileRows + ch * 8);
              const uint4 uv = *reinterpret_cast<const uint4*>(st + mi * kTileRows + ch * 8 + 8);
              const __half2* gh = reinterpret_cast<const __half2*>(&gv);
              const __half2* uh = reinterpret_cast<const __half2*>(&uv);
              __half2 res[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 gf = __half22float2(gh[q]), uf = __half22float2(uh[q]);
                res[q] = __floats2half2_rn(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
              }
              *reinterpret_cast<uint4*>(p.out + m * p.ldo + (int64_t)n_tile * (kTileRows / 2) + (ch >> 1) * 8) =
                  *reinterpret_cast<const uint4*>(res);
            }
          } else if (m < m_end) {
            *reinterpret_cast<uint4*>(p.out + m * p.ldo + (int64_t)n_tile * kTileRows + ch * 8) =
                *reinterpret_cast<const uint4*>(st + mi * kTileRows + ch * 8);
          }
        }
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty);
    }
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

#endif  // __CUDACC__

struct Launch {
  int grid;
  size_t smem;
  int group_code;
  int src;
  int zmode;
};
int launch_gemm_i4c(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream);
int launch_gemm_i4g(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream);
int launch_gemm_i8(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream);
int launch_gemm_f16(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& tw, cudaStream_t stream);

}  // namespace um

// Host entry: returns 1 when the problem is outside this kernel's coverage (the caller then runs
// batch slices on the decode kernel), 0 on launch, -1 on error.
int umma_gemm_run(const GemvParams& p, int bits, int zmode, int sm_count, cudaStream_t stream);

// Grouped form (bits 4 / 8: packed weights per expert in the fragment layout; bits 16: dense fp16
// [E, N, K]).  p.m = total rows of x / out; indptr = device int64[num_experts] of end offsets.
// 0 on launch, -1 on error (shapes outside the kernel's coverage are errors here).
int umma_group_gemm_run(const GemvParams& p, int bits, int zmode, int sm_count, const int64_t* indptr,
                        int indptr_has_prev, int num_experts, int64_t w_expert_bytes, int64_t s_expert_stride,
                        cudaStream_t stream);

}  // namespace rb200
