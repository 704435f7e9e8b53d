// Host-visible declarations of the decode-path (m <= 32) kernel.
#pragma once

#include "common.cuh"
#include "dequant.cuh"

namespace rb200 {

struct GemvParams {
  const __half* x;      // [m, k], row stride ldx
  int64_t ldx;
  const uint8_t* w;     // fragment layout
  const __half* s;      // scales, element (n, grp) at n*s_n + grp*s_g
  const __half* z;      // zero points with the same addressing, or nullptr
  int64_t s_n, s_g;
  __half* out;          // [m, n], row stride ldo
  int64_t ldo;
  Epilogue epi;
  float* partial;       // split-k scratch: [grid*2][8 warps][MT][4][32] fp32
  int* counters;        // one self-resetting ticket per 16-row block
  int* status;          // device status word (bounded waits), may be nullptr
  int m, n, k;
  int group;            // run-time group size (used when not one of the compiled sizes)
  float zero_const;
  int stages;
  int chunks_per_tile;
  long long total_iters;
};

struct GemvPlan {
  int mt;               // m-tiles of 8 rows: 1, 2 or 4
  int stages;
  int grid;
  int n_tiles;
  int chunks_per_tile;
  long long total_iters;
  size_t smem_bytes;
  size_t partial_bytes;
  size_t counter_ints;
};

int gemv_plan(int bits, int m, int n, int k, int sm_count, int ctas_per_sm_hint, int stages_hint,
              GemvPlan* plan);
int gemv_launch(const GemvParams& p, const GemvPlan& plan, int bits, int zmode, cudaStream_t stream);

}  // namespace rb200
