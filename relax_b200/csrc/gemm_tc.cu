// Tensor-core (tcgen05 / TMEM) prefill kernel - placeholder until the kernel lands: reports an
// error instead of computing anything on another path.
#include "gemm_tc.h"
namespace rb200 {
int gemm_tc_launch(const rb200_gemm_desc* d, const Epilogue&, int, int, cudaStream_t) {
  RB200_CHECK(false, "m=%lld > 32: the tensor-core kernel is not built into this library yet",
              (long long)d->m);
  return -1;
}
}  // namespace rb200
