// Host-visible declaration of the tensor-core (m > 32) kernel.
#pragma once
#include "../../include/relax_b200.h"
#include "common.cuh"
#include "dequant.cuh"
namespace rb200 {
int gemm_tc_launch(const rb200_gemm_desc* d, const Epilogue& epi, int group, int zmode,
                   cudaStream_t stream);
}
