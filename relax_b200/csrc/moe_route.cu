// Mixture-of-experts routing around the grouped matmul: softmax + top-k, rows sorted by expert,
// indptr, gather of the tokens' activations and the gated combine of the experts' outputs.
// The reference has no fused operator for this, only the building blocks its models compose
// (stable sort by key and scan: src/runtime/contrib/thrust/thrust.cu:215,325); the output
// convention is the one its grouped GEMM consumes (src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64:
// x rows sorted by expert, indptr = end row of each expert).
//
//   route   : logits fp32 [T, E] -> for every token its top_k experts by softmax probability
//             (ties: lower expert index first) with their probabilities; assignments are numbered
//             token-major (flat = t * top_k + j); rows = the assignments stably sorted by expert.
//             Outputs: indptr int64 [E], token_of_row int32 [R], gate_of_row fp32 [R],
//             row_of_flat int32 [R]  (R = T * top_k).
//   gather  : xg[row] = x[token_of_row[row]]                         (fp16 rows, 16-byte vectors)
//   combine : out[t] = f16( sum_j gate[t, j] * y[row_of_flat[t, j]] )  fp32 sum in j order.
// All three are streaming kernels; nothing is allocated, the caller passes a small int workspace.
#include "../../include/relax_b200.h"
#include "common.cuh"

namespace rb200 {
namespace {

constexpr int kMaxE = 64;
constexpr int kMaxTopK = 8;

// one warp per token
__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ logits, int T, int E, int top_k,
                                                         int* __restrict__ expert_of_flat,
                                                         float* __restrict__ gate_of_flat, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + (size_t)warp * E;
  float v0 = lane < E ? row[lane] : -INFINITY;
  float v1 = lane + 32 < E ? row[lane + 32] : -INFINITY;
  float mx = fmaxf(v0, v1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  // probabilities as exp(l - max) / sum with the sum taken in expert order by one lane (fixed order)
  float e0 = lane < E ? expf(v0 - mx) : 0.0f;
  float e1 = lane + 32 < E ? expf(v1 - mx) : 0.0f;
  float sum = 0.0f;
  for (int i = 0; i < E; ++i) sum += __shfl_sync(0xffffffffu, i < 32 ? e0 : e1, i & 31);
  float p0 = lane < E ? e0 / sum : -1.0f;
  float p1 = lane + 32 < E ? e1 / sum : -1.0f;
  for (int j = 0; j < top_k; ++j) {
    // arg max over (p, -index): larger p wins, equal p -> lower index
    float bp = p0;
    int bi = lane;
    if (p1 > bp) {
      bp = p1;
      bi = lane + 32;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float op = __shfl_xor_sync(0xffffffffu, bp, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (op > bp || (op == bp && oi < bi)) {
        bp = op;
        bi = oi;
      }
    }
    if (lane == 0) {
      expert_of_flat[warp * top_k + j] = bi;
      gate_of_flat[warp * top_k + j] = bp;
      atomicAdd(&counts[bi], 1);
    }
    if (bi == lane) p0 = -1.0f;
    if (bi == lane + 32) p1 = -1.0f;
  }
}

// one CTA per expert: the expert's assignments in flat order -> consecutive rows
__global__ void __launch_bounds__(256) route_place_kernel(const int* __restrict__ expert_of_flat,
                                                          const float* __restrict__ gate_of_flat,
                                                          const int* __restrict__ counts, int R, int E, int top_k,
                                                          int64_t* __restrict__ indptr, int* __restrict__ token_of_row,
                                                          float* __restrict__ gate_of_row,
                                                          int* __restrict__ row_of_flat) {
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ int s_warp[8];
  __shared__ int s_base;
  int begin = 0;
  for (int i = 0; i < e; ++i) begin += counts[i];
  if (tid == 0) {
    indptr[e] = (int64_t)begin + counts[e];
    s_base = begin;
  }
  __syncthreads();
  for (int i0 = 0; i0 < R; i0 += 256) {
    const int i = i0 + tid;
    const bool mine = i < R && expert_of_flat[i] == e;
    const unsigned bal = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += s_warp[w];
      total += s_warp[w];
    }
    if (mine) {
      const int row = s_base + before + __popc(bal & ((1u << lane) - 1u));
      token_of_row[row] = i / top_k;
      gate_of_row[row] = gate_of_flat[i];
      row_of_flat[i] = row;
    }
    __syncthreads();
    if (tid == 0) s_base += total;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ token_of_row,
                                                          uint4* __restrict__ out, int64_t R, int64_t vec_per_row) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < R * vec_per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i % vec_per_row;
    out[i] = x[(int64_t)token_of_row[r] * vec_per_row + c];
  }
}

__global__ void __launch_bounds__(256) combine_kernel(const __half* __restrict__ y, const int* __restrict__ row_of_flat,
                                                      const float* __restrict__ gate_of_flat_rows, int top_k,
                                                      __half* __restrict__ out, int64_t T, int64_t N) {
  // gate_of_flat_rows: gate indexed by ROW (gate_of_row); thread -> (token, 8 consecutive n)
  const int64_t vec_per_row = N / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < T * vec_per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec_per_row, c = i % vec_per_row;
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
    for (int j = 0; j < top_k; ++j) {
      const int row = row_of_flat[t * top_k + j];
      const float g = gate_of_flat_rows[row];
      const uint4 v = *reinterpret_cast<const uint4*>(y + (int64_t)row * N + c * 8);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(h[q]);
        acc[2 * q] = fmaf(g, f.x, acc[2 * q]);
        acc[2 * q + 1] = fmaf(g, f.y, acc[2 * q + 1]);
      }
    }
    __half res[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) res[q] = __float2half_rn(acc[q]);
    *reinterpret_cast<uint4*>(out + t * N + c * 8) = *reinterpret_cast<uint4*>(res);
  }
}

int blocks_for(int64_t work, int threads) {
  int64_t b = (work + threads - 1) / threads;
  if (b > (int64_t)sm_count_current() * 16) b = (int64_t)sm_count_current() * 16;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace
}  // namespace rb200

using namespace rb200;

extern "C" {

size_t rb200_moe_route_workspace_bytes(int64_t tokens, int64_t top_k) {
  // [counts: 64 ints | expert_of_flat: R ints | gate_of_flat: R floats]
  return (size_t)(kMaxE + 2 * tokens * top_k) * 4;
}

int rb200_moe_route(const void* logits, int64_t tokens, int64_t num_experts, int64_t top_k, int64_t* indptr,
                    int32_t* token_of_row, float* gate_of_row, int32_t* row_of_flat, void* workspace,
                    size_t workspace_bytes, void* stream) {
  RB200_CHECK(logits && indptr && token_of_row && gate_of_row && row_of_flat && workspace, "NULL argument");
  RB200_CHECK(num_experts >= 1 && num_experts <= kMaxE, "num_experts=%lld outside [1, %d]", (long long)num_experts, kMaxE);
  RB200_CHECK(top_k >= 1 && top_k <= kMaxTopK && top_k <= num_experts, "top_k=%lld outside [1, min(%d, experts)]",
              (long long)top_k, kMaxTopK);
  RB200_CHECK(tokens >= 0 && tokens * top_k < (1ll << 30), "bad token count");
  RB200_CHECK(workspace_bytes >= rb200_moe_route_workspace_bytes(tokens, top_k), "workspace too small");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* counts = static_cast<int*>(workspace);
  int* expert_of_flat = counts + kMaxE;
  float* gate_of_flat = reinterpret_cast<float*>(expert_of_flat + tokens * top_k);
  RB200_CUDA(cudaMemsetAsync(counts, 0, kMaxE * sizeof(int), s));
  const int R = (int)(tokens * top_k);
  if (tokens > 0) {
    route_topk_kernel<<<(int)((tokens * 32 + 255) / 256), 256, 0, s>>>(static_cast<const float*>(logits), (int)tokens,
                                                                      (int)num_experts, (int)top_k, expert_of_flat,
                                                                      gate_of_flat, counts);
    RB200_CUDA(cudaGetLastError());
  }
  route_place_kernel<<<(int)num_experts, 256, 0, s>>>(expert_of_flat, gate_of_flat, counts, R, (int)num_experts,
                                                      (int)top_k, indptr, token_of_row, gate_of_row, row_of_flat);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

int rb200_moe_gather(const void* x, const int32_t* token_of_row, void* out, int64_t rows, int64_t k, void* stream) {
  RB200_CHECK(x && token_of_row && out, "NULL argument");
  RB200_CHECK(k > 0 && k % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
                  (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
              "k must be a multiple of 8 and the tensors 16-byte aligned");
  if (rows == 0) return 0;
  gather_rows_kernel<<<blocks_for(rows * (k / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), token_of_row, static_cast<uint4*>(out), rows, k / 8);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

int rb200_moe_combine(const void* y, const int32_t* row_of_flat, const float* gate_of_row, void* out, int64_t tokens,
                      int64_t top_k, int64_t n, void* stream) {
  RB200_CHECK(y && row_of_flat && gate_of_row && out, "NULL argument");
  RB200_CHECK(n > 0 && n % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0 &&
                  (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
              "n must be a multiple of 8 and the tensors 16-byte aligned");
  RB200_CHECK(top_k >= 1 && top_k <= kMaxTopK, "top_k outside [1, %d]", kMaxTopK);
  if (tokens == 0) return 0;
  combine_kernel<<<blocks_for(tokens * (n / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(y), row_of_flat, gate_of_row, (int)top_k, static_cast<__half*>(out), tokens, n);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
