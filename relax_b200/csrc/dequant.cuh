// Bit-exact device decode of packed int4/int8 codes, and the kernel-private fragment layout.
//
// Arithmetic (the reference's decode TIR: tests/python/dlight/test_gpu_gemv.py:193-198,
// tests/python/relax/test_codegen_cutlass.py:1371-1389, :1628, :2041):
//     wq = f16_rn( (f16(u) - z) * s )
// with u an unsigned code, z the zero point and s the fp16 scale.  f16(u) - z is formed exactly
// (magic-number construction of 1024+u, exact subtraction) or, for arbitrary fp16 zero points,
// with one correctly rounded fp16 subtraction; the product is one correctly rounded fp16
// multiply.  Every fp16 op is issued as explicit ".rn" PTX so the compiler cannot contract.
//
// Fragment layout (what rb200_preprocess_weight writes).  The weight of one expert is a set of
// 512-byte fragment tiles; tile (nb, kb) covers 16 output rows (row block nb) x KFRAG reduction
// elements (KFRAG = 64 for int4, 32 for int8; KB = K / KFRAG, NB = N / 16).  Tiles are ordered so
// that everything one pipeline stage of the matmul kernels needs - 8 row blocks (128 rows) x 4
// k-blocks - is ONE contiguous 16 KB run (the copy engine pays per contiguous segment, not per
// byte: eight 2 KB segments per stage halve the streaming rate of an SM):
//     offset(nb, kb) = ((t * 8 * KB) + c * 4 * nblk(t) + b * nkb(c) + j) * 512
//     t = nb / 8, b = nb % 8, c = kb / 4, j = kb % 4,
//     nblk(t) = min(8, NB - 8t)  (last row tile may be short),  nkb(c) = min(4, KB - 4c).
// Inside a tile the 16-byte unit of "lane" L = 4g + t (g = 0..7, t = 0..3) sits at byte
// 16 * unit_pos(L), unit_pos = 8t + ((g + 2t) & 7): all g of one t share a 128-byte line (what a
// quarter-warp of the tensor-core decode kernel reads at once) and the units of lanes 8q..8q+7
// fall in eight different 16-byte bank groups (what a quarter-warp of the warp-MMA kernels
// reads at once), so neither access pattern has shared-memory bank conflicts.  The unit holds
// rows {g, g+8} of the 16-row block and the reduction elements
//   int4: k = 64*kb + 16*t + [0,16)     int8: k = 32*kb + 8*t + [0,8)
//   int4 word j (0..3) covers k4 = 4j..4j+3; nibble p of the word holds
//        p=0:(g,k4+0) p=4:(g,k4+1) p=2:(g,k4+2) p=6:(g,k4+3)
//        p=1:(g+8,k4+0) p=5:(g+8,k4+1) p=3:(g+8,k4+2) p=7:(g+8,k4+3)
//   int8 word 2j+r (j = 0..1, r = 0..1) holds row g+8r, k = 4j..4j+3 in byte order.
// One 128-bit load per lane therefore yields the A fragments of four (int4) or two (int8)
// m16n8k16 MMAs whose k-slots are mapped to 4 consecutive reduction elements per lane, and the
// same 16 bytes are 2 x 16 (int4) / 2 x 8 (int8) row-contiguous elements for the swizzled
// shared-memory tile of the tensor-core kernel.
#pragma once

#include "common.cuh"

namespace rb200 {

// Epilogue operands:  out = unary(binary(act(acc + bias), residual)).
struct Epilogue {
  const __half* bias;      // or nullptr
  int64_t bias_stride;     // 0 or n
  const __half* residual;  // or nullptr
  int64_t ld_res;
  int act, binop, unop;
};

// Byte offset of fragment tile (nb, kb) inside one expert's weight, and of the contiguous run
// that holds all tiles of (row tile t, k-chunk c).
__host__ __device__ __forceinline__ int64_t frag_stage_offset(int64_t t, int64_t c, int64_t NB, int64_t KB) {
  const int64_t nblk = (NB - 8 * t) < 8 ? (NB - 8 * t) : 8;
  return (t * 8 * KB + c * 4 * nblk) * 512;
}
__host__ __device__ __forceinline__ int64_t frag_tile_offset(int64_t nb, int64_t kb, int64_t NB, int64_t KB) {
  const int64_t t = nb >> 3, b = nb & 7, c = kb >> 2, j = kb & 3;
  const int64_t nkb = (KB - 4 * c) < 4 ? (KB - 4 * c) : 4;
  return frag_stage_offset(t, c, NB, KB) + (b * nkb + j) * 512;
}

// Position (in 16-byte units) of lane L's unit inside a 512-byte fragment tile.
__host__ __device__ __forceinline__ int frag_unit_pos(int lane) {
  const int g = lane >> 2, t = lane & 3;
  return 8 * t + ((g + 2 * t) & 7);
}

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// (a & mask) | orv in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t h2_bcast(__half h) {
  uint32_t v = __half_as_ushort(h);
  return v | (v << 16);
}
__device__ __forceinline__ uint32_t f2_to_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Zero-point handling.  kZeroConstInt: z is a kernel-wide integer constant in [0, 255] folded
// into the magic-number subtraction (exact).  kZeroGeneral: z is an arbitrary fp16 value per
// (row, group), subtracted with its own rounding exactly as the reference's fp16 TIR does.
enum ZeroMode : int { kZeroConstInt = 0, kZeroGeneral = 1 };

struct ZeroConsts {
  uint32_t sub_lo;   // f16x2(1024 + z)            (kZeroConstInt)  | f16x2(1024)  (kZeroGeneral)
  uint32_t add_hi;   // f16x2(-(64 + z))           (kZeroConstInt)  | f16x2(-64)   (kZeroGeneral)
};
__device__ __forceinline__ ZeroConsts make_zero_consts(int zmode, float zconst) {
  ZeroConsts c;
  float z = zmode == kZeroConstInt ? zconst : 0.0f;
  c.sub_lo = f2_to_h2(1024.0f + z, 1024.0f + z);
  c.add_hi = f2_to_h2(-(64.0f + z), -(64.0f + z));
  return c;
}

// One int4 word -> A fragment registers of one m16n8k16 MMA:
//   a[0] = (row g;   k4+0, k4+1)   a[1] = (row g+8; k4+0, k4+1)
//   a[2] = (row g;   k4+2, k4+3)   a[3] = (row g+8; k4+2, k4+3)
// s_g / s_g8 (and z_g / z_g8 in kZeroGeneral) are f16x2 broadcasts for rows g and g+8.
template <int ZMODE>
__device__ __forceinline__ void decode_int4_word(uint32_t w, const ZeroConsts& zc, uint32_t s_g,
                                                 uint32_t s_g8, uint32_t z_g, uint32_t z_g8,
                                                 uint32_t (&a)[4]) {
  constexpr uint32_t kMagic = 0x64006400u;      // f16x2(1024, 1024)
  constexpr uint32_t kSixteenth = 0x2C002C00u;  // f16x2(1/16, 1/16)
  const uint32_t w2 = w >> 8;
  uint32_t lo0 = and_or(w, 0x000f000fu, kMagic);   // 1024 + u        rows g
  uint32_t hi0 = and_or(w, 0x00f000f0u, kMagic);   // 1024 + 16 u     rows g+8
  uint32_t lo1 = and_or(w2, 0x000f000fu, kMagic);
  uint32_t hi1 = and_or(w2, 0x00f000f0u, kMagic);
  lo0 = h2_sub(lo0, zc.sub_lo);                 // u - z (or u), exact
  lo1 = h2_sub(lo1, zc.sub_lo);
  hi0 = h2_fma(hi0, kSixteenth, zc.add_hi);     // 64 + u - 64 - z, exact
  hi1 = h2_fma(hi1, kSixteenth, zc.add_hi);
  if (ZMODE == kZeroGeneral) {
    lo0 = h2_sub(lo0, z_g);
    lo1 = h2_sub(lo1, z_g);
    hi0 = h2_sub(hi0, z_g8);
    hi1 = h2_sub(hi1, z_g8);
  }
  a[0] = h2_mul(lo0, s_g);
  a[1] = h2_mul(hi0, s_g8);
  a[2] = h2_mul(lo1, s_g);
  a[3] = h2_mul(hi1, s_g8);
}

// Two int8 words (row g, row g+8; 4 consecutive k each) -> A fragment of one m16n8k16 MMA.
template <int ZMODE>
__device__ __forceinline__ void decode_int8_pair(uint32_t w_g, uint32_t w_g8, const ZeroConsts& zc,
                                                 uint32_t s_g, uint32_t s_g8, uint32_t z_g,
                                                 uint32_t z_g8, uint32_t (&a)[4]) {
  constexpr uint32_t kMagicBytes = 0x64646464u;
  uint32_t g01 = h2_sub(prmt(w_g, kMagicBytes, 0x4140u), zc.sub_lo);
  uint32_t g23 = h2_sub(prmt(w_g, kMagicBytes, 0x4342u), zc.sub_lo);
  uint32_t h01 = h2_sub(prmt(w_g8, kMagicBytes, 0x4140u), zc.sub_lo);
  uint32_t h23 = h2_sub(prmt(w_g8, kMagicBytes, 0x4342u), zc.sub_lo);
  if (ZMODE == kZeroGeneral) {
    g01 = h2_sub(g01, z_g);
    g23 = h2_sub(g23, z_g);
    h01 = h2_sub(h01, z_g8);
    h23 = h2_sub(h23, z_g8);
  }
  a[0] = h2_mul(g01, s_g);
  a[1] = h2_mul(h01, s_g8);
  a[2] = h2_mul(g23, s_g);
  a[3] = h2_mul(h23, s_g8);
}

// ---------------------------------------------------------------- epilogue
constexpr int kActSwiglu = 4;  // fused gated MLP: out = silu(gate) * up, see RB200_ACT_SWIGLU
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case 1:
      return fmaxf(v, 0.0f);
    case 2:
      return v / (1.0f + __expf(-v));
    case 3:
      return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default:
      return v;
  }
}

// out = unary(binary(act(acc + bias), residual)); order as the reference's patterns define it
// (python/tvm/relax/backend/contrib/cutlass.py:296-303, python/tvm/relax/backend/patterns.py:86-131).
__device__ __forceinline__ float apply_epilogue(float v, const Epilogue& e, int64_t m, int64_t n) {
  if (e.bias) v += __half2float(e.bias[m * e.bias_stride + n]);
  v = apply_act(v, e.act);
  if (e.residual) {
    float r = __half2float(e.residual[m * e.ld_res + n]);
    v = e.binop == 2 ? v * r : v + r;
  }
  if (e.unop == 1) v = fmaxf(v, 0.0f);
  return v;
}

// Same, for 16 consecutive batch rows m_base .. m_base + 15 of one output column n (rows >= m_end
// are padding: nothing is loaded for them).  The operand tests sit outside the element loops so
// that the plain case costs one add per element and no transcendental code is ever executed
// speculatively.
__device__ __forceinline__ void apply_epilogue16(float (&v)[16], const Epilogue& e, int64_t m_base, int64_t m_end,
                                                 int64_t n) {
  if (e.bias) {
    if (e.bias_stride == 0) {
      const float b = __half2float(e.bias[n]);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] += b;
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (m_base + i < m_end) v[i] += __half2float(e.bias[(m_base + i) * e.bias_stride + n]);
    }
  }
  if (e.act == 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.0f);
  } else if (e.act == 2) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = v[i] / (1.0f + __expf(-v[i]));
  } else if (e.act == 3) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.5f * v[i] * (1.0f + erff(v[i] * 0.70710678118654752f));
  }
  if (e.residual) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (m_base + i < m_end) {
        const float r = __half2float(e.residual[(m_base + i) * e.ld_res + n]);
        v[i] = e.binop == 2 ? v[i] * r : v[i] + r;
      }
  }
  if (e.unop == 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.0f);
  }
}

#endif  // __CUDACC__
}  // namespace rb200
