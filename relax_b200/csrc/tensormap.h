// Host helper: build TMA tensor maps without linking libcuda (the driver entry point is
// resolved through the runtime).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace rb200 {
// 2-D row-major tensor of `elem_bytes`-wide elements: dim0 = inner extent, dim1 = rows, row pitch
// `stride1_bytes` (multiple of 16); box = {box0, box1} elements.  Returns 0 / -1 (last error set).
int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype,
                       unsigned long long dim0, unsigned long long dim1,
                       unsigned long long stride1_bytes, unsigned box0, unsigned box1,
                       CUtensorMapSwizzle swizzle);
// General form: rank 1..5, dims[0] innermost, strides_bytes[i] = pitch of dims[i+1].
int make_tensor_map(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int rank,
                    const unsigned long long* dims, const unsigned long long* strides_bytes,
                    const unsigned* box, CUtensorMapSwizzle swizzle);
}  // namespace rb200
