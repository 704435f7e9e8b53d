// Host-visible declaration of the tensor-core (m > 32) kernel.
#pragma once
#include "../../include/relax_b200.h"
#include "common.cuh"
#include "dequant.cuh"
namespace rb200 {
// ldx / ldo: the row pitches the entry point resolved (defaults applied, the fused gate/up form
// halving the output width).
int gemm_tc_launch(const rb200_gemm_desc* d, const Epilogue& epi, int group, int zmode, int64_t ldx, int64_t ldo,
                   cudaStream_t stream);
}
