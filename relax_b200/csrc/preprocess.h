#pragma once
#include "common.cuh"
namespace rb200 {
int preprocess_launch(const void* src, void* dst, int64_t experts, int64_t k, int64_t n, int bits,
                      int layout, const int32_t* k_perm, cudaStream_t stream);
int gptq_act_order_launch(const int32_t* g_idx, int64_t k, int64_t groups, int32_t* perm, int* status,
                          cudaStream_t stream);
int gather_columns_launch(const void* x, const int32_t* perm, void* out, int64_t m, int64_t k, int64_t ldx,
                          int64_t ldo, cudaStream_t stream);
int interleave_rows_launch(const void* src, void* dst, int64_t outer, int64_t n, int64_t inner, cudaStream_t stream);
int unpack_zeros_autogptq_launch(const void* zq, void* out, int64_t groups, int64_t n, cudaStream_t stream);
}
