// Tensor-core (tcgen05 + TMEM) building blocks of the prefill / grouped kernel: PTX wrappers for
// tensor-memory allocation, tcgen05.mma / st / ld / commit, the K-major shared-memory operand
// descriptor, and the bit-exact decode of one 64-k block of a weight row into packed fp16 pairs
// (thread = weight row = TMEM lane).
#pragma once

#include <cuda.h>

#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace ug {

constexpr int kTileRows = 128;
constexpr int kKBlock = 64;  // k per MMA block (4 x K=16) and per int4 fragment tile

enum ScaleSrc : int { kSrcGlobal = 0, kSrcSmemNK = 1, kSrcSmemKN = 2 };

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
__device__ __forceinline__ void decode_block(const GemvParams& p, bool has_z_tile, const RowCtx& c,
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
      if (ZMODE == kZeroGeneral && has_z_tile) {
        const uint32_t zsel = (gi >> 1) == 0 ? c.nk_z.x : ((gi >> 1) == 1 ? c.nk_z.y : ((gi >> 1) == 2 ? c.nk_z.z : c.nk_z.w));
        z2 = prmt(zsel, zsel, (t >> 1) ? 0x3232u : 0x1010u);
      }
    } else if (SRC == kSrcSmemKN) {
      constexpr int kG = GROUP > 0 ? GROUP : 1;
      const int gl = (KB * kKBlock + t * 16) / kG;
      s2 = h2_bcast(reinterpret_cast<const __half*>(c.s_tile)[gl * kTileRows + c.row]);
      if (ZMODE == kZeroGeneral && has_z_tile)
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
__device__ __forceinline__ void decode_block_kb(int kb, const GemvParams& p, bool has_z_tile, const RowCtx& c,
                                                const ZeroConsts& zc, uint32_t zconst_h2, int group,
                                                uint32_t (&regs)[32]) {
  switch (kb) {
    case 0:
      decode_block<ZMODE, GROUP, SRC, HI, 0>(p, has_z_tile, c, zc, zconst_h2, group, regs);
      break;
    case 1:
      decode_block<ZMODE, GROUP, SRC, HI, 1>(p, has_z_tile, c, zc, zconst_h2, group, regs);
      break;
    case 2:
      decode_block<ZMODE, GROUP, SRC, HI, 2>(p, has_z_tile, c, zc, zconst_h2, group, regs);
      break;
    default:
      decode_block<ZMODE, GROUP, SRC, HI, 3>(p, has_z_tile, c, zc, zconst_h2, group, regs);
      break;
  }
}

#endif  // __CUDACC__

}  // namespace ug
}  // namespace rb200
