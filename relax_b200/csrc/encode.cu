// Quantiser on the GPU: the reference tests' encode TIR
// (tests/python/relax/test_codegen_cutlass.py:1391-1457 int4 per-row, :1630-1676 int8 per-row,
// :2043-2109 int8 in groups of 64) - the transform_params stage that the reference runs on the
// CPU before ft_preprocess_weight.
//   absmax over the row (or the row's group) in fp16;
//   scale = max(f32(absmax), 1e-4) * (1/8 | 1/128) in fp32;
//   code  = clamp(round_half_away(f32(a) / scale), -8..7 | -128..127);
//   packed int8 [K, N/2] (low nibble = even n) or [K, N]; scales fp16 [N] or [K/g, N].
// One CTA per 32 rows x one group: the tile is read once (coalesced along k), kept in shared
// memory, reduced per row, quantised and written transposed (coalesced along n).
#include "../../include/relax_b200.h"
#include "common.cuh"

namespace rb200 {
namespace {

constexpr int kRows = 32;     // n per CTA
constexpr int kMaxSpan = 512;  // k per pass through shared memory

template <int BITS>
__global__ void __launch_bounds__(256) encode_ft_kernel(const __half* __restrict__ A, int8_t* __restrict__ packed,
                                                        __half* __restrict__ scales, int64_t N, int64_t K,
                                                        int64_t group, int per_row) {
  __shared__ __half tile[kRows][kMaxSpan + 8];
  __shared__ float s_scale[kRows];
  const int64_t n0 = (int64_t)blockIdx.x * kRows;
  const int64_t g = blockIdx.y;  // group index (0 when one scale per row)
  const int64_t k_begin = g * group, k_end = k_begin + group;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float mul = BITS == 4 ? 0.125f : 0.0078125f;
  const float qlo = BITS == 4 ? -8.0f : -128.0f, qhi = BITS == 4 ? 7.0f : 127.0f;

  // pass 1: absmax of every row over [k_begin, k_end)
  float amax[kRows / 8];
#pragma unroll
  for (int i = 0; i < kRows / 8; ++i) amax[i] = 0.0f;
  for (int64_t k = k_begin + lane; k < k_end; k += 32) {
#pragma unroll
    for (int i = 0; i < kRows / 8; ++i) {
      const int64_t n = n0 + warp + 8 * i;
      if (n < N) amax[i] = fmaxf(amax[i], fabsf(__half2float(A[n * K + k])));
    }
  }
#pragma unroll
  for (int i = 0; i < kRows / 8; ++i) {
    float v = amax[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) s_scale[warp + 8 * i] = fmaxf(v, 1e-4f) * mul;  // |a| is exact in fp16, so is its max
  }
  __syncthreads();
  if (tid < kRows && n0 + tid < N)
    scales[(per_row ? 0 : g * N) + n0 + tid] = __float2half_rn(s_scale[tid]);

  // pass 2: quantise spans of k, transposing through shared memory
  for (int64_t ks = k_begin; ks < k_end; ks += kMaxSpan) {
    const int span = (int)min((int64_t)kMaxSpan, k_end - ks);
    __syncthreads();
    for (int i = tid; i < kRows * span; i += 256) {
      const int r = i / span, c = i % span;
      tile[r][c] = (n0 + r < N) ? A[(n0 + r) * K + ks + c] : __float2half_rn(0.0f);
    }
    __syncthreads();
    if (BITS == 4) {
      // thread -> (k, pair of rows): 16 byte columns per k
      for (int i = tid; i < span * (kRows / 2); i += 256) {
        const int c = i / (kRows / 2), pr = i % (kRows / 2);
        const int r0 = 2 * pr, r1 = r0 + 1;
        if (n0 + r0 >= N) continue;
        const float q0 = fminf(fmaxf(roundf(__fdiv_rn(__half2float(tile[r0][c]), s_scale[r0])), qlo), qhi);
        const float q1 = (n0 + r1 < N)
                             ? fminf(fmaxf(roundf(__fdiv_rn(__half2float(tile[r1][c]), s_scale[r1])), qlo), qhi)
                             : 0.0f;
        const int b = ((int)q0 & 15) | (((int)q1 & 15) << 4);
        packed[(ks + c) * (N / 2) + (n0 >> 1) + pr] = (int8_t)b;
      }
    } else {
      for (int i = tid; i < span * kRows; i += 256) {
        const int c = i / kRows, r = i % kRows;
        if (n0 + r >= N) continue;
        const float q = fminf(fmaxf(roundf(__fdiv_rn(__half2float(tile[r][c]), s_scale[r])), qlo), qhi);
        packed[(ks + c) * N + n0 + r] = (int8_t)(int)q;
      }
    }
  }
}

}  // namespace
}  // namespace rb200

using namespace rb200;

extern "C" int rb200_encode_ft(const void* a, void* packed, void* scales, int64_t n, int64_t k, int weight_bits,
                               int64_t group_size, void* stream) {
  RB200_CHECK(a && packed && scales, "a, packed and scales must be non-NULL");
  RB200_CHECK(weight_bits == 4 || weight_bits == 8, "weight_bits must be 4 or 8");
  RB200_CHECK(n > 0 && k > 0 && (weight_bits == 8 || n % 2 == 0), "bad shape n=%lld k=%lld", (long long)n, (long long)k);
  const bool per_row = group_size <= 0 || group_size >= k;
  const int64_t group = per_row ? k : group_size;
  RB200_CHECK(k % group == 0, "group_size=%lld must divide k=%lld", (long long)group, (long long)k);
  RB200_CHECK(k / group <= 65535, "too many groups");
  dim3 grid((unsigned)((n + kRows - 1) / kRows), (unsigned)(k / group), 1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (weight_bits == 4)
    encode_ft_kernel<4><<<grid, 256, 0, s>>>(static_cast<const __half*>(a), static_cast<int8_t*>(packed),
                                             static_cast<__half*>(scales), n, k, group, per_row ? 1 : 0);
  else
    encode_ft_kernel<8><<<grid, 256, 0, s>>>(static_cast<const __half*>(a), static_cast<int8_t*>(packed),
                                             static_cast<__half*>(scales), n, k, group, per_row ? 1 : 0);
  RB200_CUDA(cudaGetLastError());
  return 0;
}
