#include "tensormap.h"

#include <mutex>

namespace rb200 {
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;
}  // namespace

int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype,
                       unsigned long long dim0, unsigned long long dim1,
                       unsigned long long stride1_bytes, unsigned box0, unsigned box1,
                       CUtensorMapSwizzle swizzle) {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeFn>(fn);
  });
  RB200_CHECK(g_encode != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  RB200_CHECK((reinterpret_cast<uintptr_t>(base) & 15u) == 0 && stride1_bytes % 16 == 0,
              "tensor map needs a 16-byte aligned base and row pitch (pitch %llu)", stride1_bytes);
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {stride1_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RB200_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}
}  // namespace rb200
