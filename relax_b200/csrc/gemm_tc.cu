// m > 32: batch-sliced execution on the tensor-core decode kernel.
//
// The decode kernel takes the batch as the MMA's N dimension (up to 32 rows per pass).  Larger
// batches are run as consecutive 32-row slices, each a full pass over the packed weight; the
// weight (tens of MB) stays L2-resident between passes for the layer sizes of the benchmark
// configurations.  A dedicated prefill kernel with a 256-row batch tile replaces this path;
// until then this keeps every entry point correct for any m.
#include "gemm_tc.h"

namespace rb200 {

int gemm_tc_launch(const rb200_gemm_desc* d, const Epilogue&, int, int, cudaStream_t stream) {
  rb200_gemm_desc s = *d;
  const int64_t ldx = d->ldx > 0 ? d->ldx : d->k;
  const int64_t ldo = d->ldo > 0 ? d->ldo : d->n;
  for (int64_t m0 = 0; m0 < d->m; m0 += 32) {
    s.m = (d->m - m0) < 32 ? (d->m - m0) : 32;
    s.x = static_cast<const char*>(d->x) + m0 * ldx * 2;
    s.out = static_cast<char*>(d->out) + m0 * ldo * 2;
    s.ldx = ldx;
    s.ldo = ldo;
    if (d->bias && d->bias_stride != 0) s.bias = static_cast<const char*>(d->bias) + m0 * d->bias_stride * 2;
    if (d->residual) s.residual = static_cast<const char*>(d->residual) + m0 * d->n * 2;
    if (rb200_gemm_fp16_intx(&s, stream) != 0) return -1;
  }
  return 0;
}

}  // namespace rb200
