// Weight repack into the fragment layout (see dequant.cuh), one 16-byte lane unit per thread.
// Stands in for fastertransformer::preprocess_weights as called by
// cutlass.ft_preprocess_weight (src/runtime/contrib/cutlass/weight_preprocess.cc:38-58): same
// byte size in and out, signed codes biased to unsigned, layout private to the matmul kernels.
#include "dequant.cuh"
#include "preprocess.h"

namespace rb200 {
namespace {

// Unsigned code of logical element (n, k) of one expert in the given source layout.
template <int BITS, int LAYOUT>
__device__ __forceinline__ uint32_t load_code(const uint8_t* src, int64_t n, int64_t k, int64_t K,
                                              int64_t N) {
  if (LAYOUT == 0) {  // FT: int8 container [K, N/2] (int4) or [K, N] (int8), signed
    if (BITS == 4) {
      uint32_t b = src[k * (N / 2) + (n >> 1)];
      return ((b >> ((n & 1) * 4)) & 15u) ^ 8u;  // two's-complement nibble + 8
    }
    return (uint32_t)src[k * N + n] ^ 0x80u;  // signed byte + 128
  }
  if (LAYOUT == 2) {  // AutoGPTQ: uint32 [K/8, N], nibble j of word (k/8, n) = element k = 8*(k/8) + j
    const uint32_t w = reinterpret_cast<const uint32_t*>(src)[(k >> 3) * N + n];
    return (w >> ((k & 7) * 4)) & 15u;
  }
  // q4f16_1: uint32 [N, K/8], nibble j of a word = element 8*word + j, unsigned
  uint32_t b = src[n * (K / 2) + (k >> 1)];
  return (b >> ((k & 1) * 4)) & 15u;
}

// AutoGPTQ zero points: zq uint32 [G, N/8] (nibble j of word (g, n/8) = column 8*(n/8) + j) ->
// fp16 [G, N] holding f16(zq) + f16(1), the value the decode subtracts
// (tests/python/dlight/test_gpu_gemv.py:648).
__global__ void unpack_zeros_autogptq_kernel(const uint32_t* __restrict__ zq, __half* __restrict__ out, int64_t total,
                                             int64_t N) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t g = i / N, n = i % N;
    const uint32_t q = (zq[g * (N / 8) + (n >> 3)] >> ((n & 7) * 4)) & 15u;
    out[i] = __hadd(__int2half_rn((int)q), __float2half_rn(1.0f));
  }
}

// Gate/up interleave: the source holds gate rows [0, N/2) and up rows [N/2, N); fragment row block
// nb then takes gate rows 8nb..8nb+7 as its rows 0..7 and up rows 8nb..8nb+7 as its rows 8..15, so
// that one lane of the warp-MMA kernels (rows g and g+8) owns gate_f and up_f of the same f.
__host__ __device__ __forceinline__ int64_t gate_up_source_row(int64_t j, int64_t N) {
  const int64_t nb = j >> 4, r = j & 15;
  return r < 8 ? 8 * nb + r : N / 2 + 8 * nb + (r - 8);
}

template <int BITS, int LAYOUT>
__global__ void repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                              int64_t K, int64_t N, int64_t units_per_expert, int64_t total_units, int interleave,
                              const int32_t* __restrict__ k_perm) {
  constexpr int kFrag = BITS == 4 ? 64 : 32;
  const int64_t expert_bytes = K * N * BITS / 8;
  for (int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; u < total_units;
       u += (int64_t)gridDim.x * blockDim.x) {
    // unit index -> (expert, row block, k block, lane): 32-bit divisions whenever the unit count
    // fits (64-bit ones are routines of a hundred instructions, three per 16 bytes moved)
    int64_t e, nb, kb;
    int lane;
    const int64_t KB = K / kFrag;
    if (total_units < (1ll << 31)) {
      const uint32_t u32 = (uint32_t)u, upe = (uint32_t)units_per_expert, kb32 = (uint32_t)KB;
      const uint32_t e32 = u32 / upe, r32 = u32 - e32 * upe;
      const uint32_t tile = r32 >> 5, nb32 = tile / kb32;
      e = e32;
      lane = (int)(r32 & 31u);
      nb = nb32;
      kb = tile - nb32 * kb32;
    } else {
      e = u / units_per_expert;
      const int64_t r = u % units_per_expert;
      lane = (int)(r & 31);
      const int64_t tile = r >> 5;
      nb = tile / KB;
      kb = tile % KB;
    }
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* s = src + e * expert_bytes;
    uint32_t words[4];
    if (BITS == 4 && LAYOUT == 1) {
      // q4f16_1 source: the unit's 16 k of a row are two consecutive 32-bit words of that row
      // (8 nibbles each, k ascending from the low nibble): two 8-byte loads per unit, then bit moves
      const int64_t k0 = kb * 64 + t * 16;
      int64_t r_lo = nb * 16 + g, r_hi = r_lo + 8;
      if (interleave) {
        r_lo = gate_up_source_row(r_lo, N);
        r_hi = gate_up_source_row(r_hi, N);
      }
      const uint2 lo = *reinterpret_cast<const uint2*>(s + (r_lo * (K / 8) + k0 / 8) * 4);
      const uint2 hi = *reinterpret_cast<const uint2*>(s + (r_hi * (K / 8) + k0 / 8) * 4);
      const uint32_t lw[2] = {lo.x, lo.y}, hw[2] = {hi.x, hi.y};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // word j covers k4 = 4j .. 4j+3: nibbles (j & 1) * 4 .. + 3 of source word j >> 1
        const uint32_t a = (lw[j >> 1] >> ((j & 1) * 16)) & 0xffffu;  // row g:   k4+0..3 in nibbles 0..3
        const uint32_t b = (hw[j >> 1] >> ((j & 1) * 16)) & 0xffffu;  // row g+8
        // slots: p0 (g,k4) p4 (g,k4+1) p2 (g,k4+2) p6 (g,k4+3); p1 p5 p3 p7 the same for g+8
        const uint32_t ga = (a & 0xfu) | ((a & 0xf0u) << 12) | ((a & 0xf00u)) | ((a & 0xf000u) << 12);
        const uint32_t gb = (b & 0xfu) | ((b & 0xf0u) << 12) | ((b & 0xf00u)) | ((b & 0xf000u) << 12);
        words[j] = ga | (gb << 4);
      }
    } else if (BITS == 4) {
      const int64_t k0 = kb * 64 + t * 16;
      // nibble slot p of a word <- (row offset, k offset inside the word's 4 k)
      const int row_of[8] = {0, 8, 0, 8, 0, 8, 0, 8};
      const int k_of[8] = {0, 0, 2, 2, 1, 1, 3, 3};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w = 0;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          int64_t srow = nb * 16 + g + row_of[p];
          if (interleave) srow = gate_up_source_row(srow, N);
          int64_t ks = k0 + 4 * j + k_of[p];
          if (LAYOUT == 2 && k_perm) ks = k_perm[ks];  // act-order: k position -> source row
          uint32_t c = load_code<BITS, LAYOUT>(s, srow, ks, K, N);
          w |= c << (4 * p);
        }
        words[j] = w;
      }
    } else {
      const int64_t k0 = kb * 32 + t * 8;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int r8 = 0; r8 < 2; ++r8) {
          uint32_t w = 0;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            int64_t srow = nb * 16 + g + 8 * r8;
            if (interleave) srow = gate_up_source_row(srow, N);
            w |= load_code<BITS, LAYOUT>(s, srow, k0 + 4 * j + c4, K, N) << (8 * c4);
          }
          words[2 * j + r8] = w;
        }
    }
    reinterpret_cast<uint4*>(dst + e * expert_bytes + frag_tile_offset(nb, kb, N / 16, KB))[frag_unit_pos(lane)] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// FT source ([K, N] bytes for int8, [K, N/2] bytes for int4, both contiguous along n) without the
// gate/up interleave: the fragment layout gathers along k, the source is contiguous along n, so
// a byte gather straight from global memory wastes 15 of every 16 bytes of each sector it
// touches.  Here a CTA stages one panel - the kFrag k-rows of one fragment k-block x 512 output
// columns (16 KB) - in shared memory with 16-byte (int8) / 8-byte (int4) loads that are coalesced
// along n, and every lane then gathers its 16-byte unit from shared memory; the 32 units of a
// fragment tile leave as one 512-byte segment.  The 16-byte chunks of panel row k are stored at
// chunk ^ (row quarter), so that the four lane groups of a warp, which read rows a quarter of
// the block apart, hit different banks.
template <int BITS>
__global__ void __launch_bounds__(256) repack_ft_panel_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                              int64_t K, int64_t N, int64_t panels_per_kb,
                                                              int64_t total_panels) {
  constexpr int kFrag = BITS == 4 ? 64 : 32;         // k rows of a panel
  constexpr int kRowBytes = BITS == 4 ? 256 : 512;   // 512 output columns
  constexpr int kChunks = kRowBytes / 16;
  constexpr int kQuarter = kFrag / 4;                // k rows per lane group t
  __shared__ __align__(16) uint8_t panel[kFrag * kRowBytes];
  const int64_t KB = K / kFrag, NB = N / 16;
  const int64_t row_bytes = N * BITS / 8;
  const int64_t expert_bytes = K * row_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  for (int64_t pi = blockIdx.x; pi < total_panels; pi += gridDim.x) {
    const int64_t e = pi / (KB * panels_per_kb);
    const int64_t rem = pi % (KB * panels_per_kb);
    const int64_t kb = rem / panels_per_kb, pn = rem % panels_per_kb;
    const int64_t byte0 = pn * kRowBytes;                       // first byte of the panel inside a source row
    const int64_t valid = min((int64_t)kRowBytes, row_bytes - byte0);
    const uint8_t* s = src + e * expert_bytes + kb * kFrag * row_bytes + byte0;
    __syncthreads();  // the previous panel has been read
    if (BITS == 8) {
      for (int i = tid; i < kFrag * kChunks; i += 256) {
        const int r = i / kChunks, c = i % kChunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (c * 16 < valid) v = *reinterpret_cast<const uint4*>(s + r * row_bytes + c * 16);
        *reinterpret_cast<uint4*>(panel + r * kRowBytes + ((c ^ ((r / kQuarter) & 3)) << 4)) = v;
      }
    } else {
      for (int i = tid; i < kFrag * kChunks * 2; i += 256) {
        const int r = i / (kChunks * 2), h = i % (kChunks * 2);  // 8-byte halves: rows are only 8-byte aligned
        uint2 v = make_uint2(0u, 0u);
        if (h * 8 < valid) v = *reinterpret_cast<const uint2*>(s + r * row_bytes + h * 8);
        *reinterpret_cast<uint2*>(panel + r * kRowBytes + (((h >> 1) ^ ((r / kQuarter) & 3)) << 4) + (h & 1) * 8) = v;
      }
    }
    __syncthreads();
    // 32 fragment tiles (16 output rows each) per panel, four per warp
    for (int bi = warp; bi < 32; bi += 8) {
      const int64_t nb = pn * 32 + bi;
      if (nb >= NB) break;
      uint32_t words[4];
      if (BITS == 8) {
        // unit: rows g, g + 8; k = 8 t .. 8 t + 7; word 2 j + r8 = row g + 8 r8, k 4 j .. 4 j + 3
        const uint8_t* base = panel + ((bi ^ t) << 4) + g;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int r8 = 0; r8 < 2; ++r8) {
            uint32_t w = 0;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              w |= ((uint32_t)base[(t * 8 + 4 * j + c4) * kRowBytes + 8 * r8] ^ 0x80u) << (8 * c4);
            words[2 * j + r8] = w;
          }
      } else {
        // unit: rows g, g + 8; k = 16 t .. 16 t + 15; word j covers k4 = 4 j .. 4 j + 3 with nibble
        // slots p0 (g,k4) p4 (g,k4+1) p2 (g,k4+2) p6 (g,k4+3), p1 p5 p3 p7 the same for g + 8
        // The eight bytes at `base` of a panel row hold the tile's 16 output rows of that k: one
        // 8-byte load (the same address for the eight lanes of a t: a broadcast) brings row g in
        // its low word and row g + 8 in its high word, nibble g & 1 of byte g >> 1.
        const uint8_t* base = panel + (((bi >> 1) ^ t) << 4) + (bi & 1) * 8;
        const int sh = (g >> 1) * 8 + (g & 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t w = 0;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint2 v = *reinterpret_cast<const uint2*>(base + (t * 16 + 4 * j + kk) * kRowBytes);
            const uint32_t pair = (((v.x >> sh) & 15u) | (((v.y >> sh) & 15u) << 4)) ^ 0x88u;  // rows g, g + 8
            const int slot = kk == 0 ? 0 : (kk == 1 ? 4 : (kk == 2 ? 2 : 6));
            w |= pair << (4 * slot);
          }
          words[j] = w;
        }
      }
      reinterpret_cast<uint4*>(dst + e * expert_bytes + frag_tile_offset(nb, kb, NB, KB))[frag_unit_pos(lane)] =
          make_uint4(words[0], words[1], words[2], words[3]);
    }
  }
}

// Act-order AutoGPTQ weights (tests/python/dlight/test_gpu_gemv.py:639-649 reads scale and zero
// of element k through g_idx[k]): perm lists the k rows group by group, in their original order
// inside a group, so that the weight repacked through perm has its groups contiguous along k and
// the matmul of x gathered through the same perm equals the reference's.  One CTA; every thread
// owns groups g = tid, tid + blockDim, ... and scans g_idx twice (count, then place).
// status: 0 = fine, 1 = some group does not have exactly K / G members or an index is out of range.
__global__ void gptq_act_order_kernel(const int32_t* __restrict__ g_idx, int K, int G, int32_t* __restrict__ perm,
                                      int* __restrict__ status) {
  extern __shared__ int s_start[];  // [G + 1]
  const int per = K / G;
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    int c = 0;
    for (int k = 0; k < K; ++k) c += g_idx[k] == g;
    if (c != per) bad = 1;
    s_start[g] = g * per;  // groups of equal size, or the result is rejected
  }
  __syncthreads();
  if (threadIdx.x == 0) *status = bad;
  if (bad) return;
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    int pos = s_start[g];
    for (int k = 0; k < K; ++k)
      if (g_idx[k] == g) perm[pos++] = k;
  }
}

// out[m, j] = x[m, perm[j]] over fp16
__global__ void gather_columns_kernel(const __half* __restrict__ x, const int32_t* __restrict__ perm,
                                      __half* __restrict__ out, int64_t M, int64_t K, int64_t ldx, int64_t ldo) {
  const int64_t total = M * K;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / K, j = i % K;
    out[m * ldo + j] = x[m * ldx + perm[j]];
  }
}

}  // namespace

// dst[o][j][i] = src[o][gate_up_source_row(j)][i] over fp16 elements: the row permutation of the
// interleaved repack applied to a scale / zero-point tensor viewed as [outer][n][inner]
__global__ void interleave_rows_kernel(const __half* __restrict__ src, __half* __restrict__ dst, int64_t outer,
                                       int64_t N, int64_t inner) {
  const int64_t total = outer * N * inner;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t in = i % inner, j = (i / inner) % N, o = i / (inner * N);
    dst[i] = src[(o * N + gate_up_source_row(j, N)) * inner + in];
  }
}

int preprocess_launch(const void* src, void* dst, int64_t experts, int64_t k, int64_t n, int bits,
                      int layout_flags, const int32_t* k_perm, cudaStream_t stream) {
  const int interleave = (layout_flags & 0x100) ? 1 : 0;
  const int layout = layout_flags & 0xff;
  RB200_CHECK(!k_perm || layout == 2, "a k permutation goes with the AutoGPTQ source layout only");
  const int64_t units = k * n * bits / 8 / 16;
  const int64_t total = units * experts;
  const int threads = 256;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > (int64_t)sm_count_current() * 32) blocks = (int64_t)sm_count_current() * 32;
  if (blocks == 0) return 0;
  const uint8_t* s = static_cast<const uint8_t*>(src);
  uint8_t* d = static_cast<uint8_t*>(dst);
  if (layout == 0 && !interleave && (reinterpret_cast<uintptr_t>(src) & (bits == 8 ? 15u : 7u)) == 0) {
    // FT source: staged through shared memory, coalesced both ways
    const int64_t panels_per_kb = (n + 511) / 512;
    const int64_t total_panels = experts * (k / (bits == 4 ? 64 : 32)) * panels_per_kb;
    int64_t grid = total_panels;
    if (grid > (int64_t)sm_count_current() * 32) grid = (int64_t)sm_count_current() * 32;
    if (bits == 4) repack_ft_panel_kernel<4><<<(int)grid, 256, 0, stream>>>(s, d, k, n, panels_per_kb, total_panels);
    else repack_ft_panel_kernel<8><<<(int)grid, 256, 0, stream>>>(s, d, k, n, panels_per_kb, total_panels);
    RB200_CUDA(cudaGetLastError());
    return 0;
  }
  if (bits == 4 && layout == 0)
    repack_kernel<4, 0><<<(int)blocks, threads, 0, stream>>>(s, d, k, n, units, total, interleave, k_perm);
  else if (bits == 4 && layout == 1)
    repack_kernel<4, 1><<<(int)blocks, threads, 0, stream>>>(s, d, k, n, units, total, interleave, k_perm);
  else if (bits == 4 && layout == 2)
    repack_kernel<4, 2><<<(int)blocks, threads, 0, stream>>>(s, d, k, n, units, total, interleave, k_perm);
  else if (bits == 8 && layout == 0)
    repack_kernel<8, 0><<<(int)blocks, threads, 0, stream>>>(s, d, k, n, units, total, interleave, k_perm);
  else
    RB200_CHECK(false, "unsupported preprocess combination bits=%d layout=%d", bits, layout);

  RB200_CUDA(cudaGetLastError());
  return 0;
}

int interleave_rows_launch(const void* src, void* dst, int64_t outer, int64_t n, int64_t inner, cudaStream_t stream) {
  const int64_t total = outer * n * inner;
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sm_count_current() * 16) blocks = (int64_t)sm_count_current() * 16;
  interleave_rows_kernel<<<(int)blocks, 256, 0, stream>>>(static_cast<const __half*>(src), static_cast<__half*>(dst),
                                                         outer, n, inner);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

int gptq_act_order_launch(const int32_t* g_idx, int64_t k, int64_t groups, int32_t* perm, int* status,
                          cudaStream_t stream) {
  gptq_act_order_kernel<<<1, 1024, (size_t)(groups + 1) * sizeof(int), stream>>>(g_idx, (int)k, (int)groups, perm, status);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

int gather_columns_launch(const void* x, const int32_t* perm, void* out, int64_t m, int64_t k, int64_t ldx,
                          int64_t ldo, cudaStream_t stream) {
  const int64_t total = m * k;
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sm_count_current() * 16) blocks = (int64_t)sm_count_current() * 16;
  gather_columns_kernel<<<(int)blocks, 256, 0, stream>>>(static_cast<const __half*>(x), perm, static_cast<__half*>(out),
                                                        m, k, ldx, ldo);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

int unpack_zeros_autogptq_launch(const void* zq, void* out, int64_t groups, int64_t n, cudaStream_t stream) {
  const int64_t total = groups * n;
  if (total == 0) return 0;
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sm_count_current() * 16) blocks = (int64_t)sm_count_current() * 16;
  unpack_zeros_autogptq_kernel<<<(int)blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(zq),
                                                               static_cast<__half*>(out), total, n);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace rb200
