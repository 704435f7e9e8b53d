#pragma once
#include "common.cuh"
namespace rb200 {
int preprocess_launch(const void* src, void* dst, int64_t experts, int64_t k, int64_t n, int bits,
                      int layout, cudaStream_t stream);
int interleave_rows_launch(const void* src, void* dst, int64_t outer, int64_t n, int64_t inner, cudaStream_t stream);
int unpack_zeros_autogptq_launch(const void* zq, void* out, int64_t groups, int64_t n, cudaStream_t stream);
}
