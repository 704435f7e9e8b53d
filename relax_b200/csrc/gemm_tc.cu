// m > 32: the tcgen05 prefill kernel (256-row batch tiles, weights decoded into tensor memory);
// shapes it does not cover (n not a multiple of 128, k not a multiple of 64, unaligned x) run as
// consecutive 32-row batch slices on the decode kernel, each a full pass over the packed weight.
#include "gemm_tc.h"

#include <cstdlib>
#include <cstring>

#include "umma_gemm.cuh"

namespace rb200 {

int gemm_tc_launch(const rb200_gemm_desc* d, const Epilogue& epi, int group, int zmode, int64_t ldx, int64_t ldo,
                   cudaStream_t stream) {
  DeviceScratch* sc = device_scratch(0, 0);
  if (!sc) return -1;
  {
    GemvParams p;
    memset(&p, 0, sizeof(p));
    p.status = sc->status;
    p.x = static_cast<const __half*>(d->x);
    p.ldx = ldx;
    p.w = static_cast<const uint8_t*>(d->w);
    p.s = static_cast<const __half*>(d->scales);
    p.z = static_cast<const __half*>(d->zeros);
    p.s_n = d->scale_stride_n;
    p.s_g = d->scale_stride_g;
    p.out = static_cast<__half*>(d->out);
    p.ldo = ldo;
    p.epi = epi;
    p.m = (int)d->m;
    p.n = (int)d->n;
    p.k = (int)d->k;
    p.group = group;
    p.zero_const = d->zero_const;
    const int rc = umma_gemm_run(p, d->weight_bits, zmode, sc->sm_count, stream);
    if (rc <= 0) return rc;
  }
  rb200_gemm_desc s = *d;
  for (int64_t m0 = 0; m0 < d->m; m0 += 32) {
    s.m = (d->m - m0) < 32 ? (d->m - m0) : 32;
    s.x = static_cast<const char*>(d->x) + m0 * ldx * 2;
    s.out = static_cast<char*>(d->out) + m0 * ldo * 2;
    s.ldx = ldx;
    s.ldo = ldo;
    if (d->bias && d->bias_stride != 0) s.bias = static_cast<const char*>(d->bias) + m0 * d->bias_stride * 2;
    if (d->residual) s.residual = static_cast<const char*>(d->residual) + m0 * d->n * 2;  // residual rows are n wide
    if (rb200_gemm_fp16_intx(&s, stream) != 0) return -1;
  }
  return 0;
}

}  // namespace rb200
