// Instantiation + dispatch of gemv_sk_kernel for one weight width.
#pragma once
#include <cstring>

#include "gemv_sk.cuh"

namespace rb200 {
namespace sk {

template <int BITS, int MT, int ZMODE, int GROUP, int SRC, bool AR = false>
int launch_inst(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
                cudaStream_t stream) {
  auto kern = gemv_sk_kernel<BITS, MT, ZMODE, GROUP, SRC, AR>;
  static thread_local int configured_device = -1;
  int dev = 0;
  RB200_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    RB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)l.grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = l.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (l.cooperative) {
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
  } else {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = launch_overlap_enabled() ? 1 : 0;
  }
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RB200_CUDA(cudaLaunchKernelEx(&cfg, kern, pp, tx, ts, tz));
  return 0;
}

template <int BITS, int MT, int ZMODE>
int launch_gs(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
              cudaStream_t stream) {
  if (pp.ar.world > 1) {
    // the all-reduce epilogue is compiled for the forms sharded layers use: symmetric codes with
    // group-32 [N, K/32] scales (int4) or one scale per output channel
    if constexpr (ZMODE == kZeroConstInt) {
      if constexpr (BITS == 4) {
        if (l.group_code == 32 && l.src == kSrcSmemNK)
          return launch_inst<4, MT, kZeroConstInt, 32, kSrcSmemNK, true>(pp, l, tx, ts, tz, stream);
        // a K-shard whose scale rows are not 16-byte multiples cannot be staged by TMA
        if (l.group_code == 32 && l.src == kSrcGlobal)
          return launch_inst<4, MT, kZeroConstInt, 32, kSrcGlobal, true>(pp, l, tx, ts, tz, stream);
      }
      if (l.group_code == 0 && l.src == kSrcGlobal)
        return launch_inst<BITS, MT, kZeroConstInt, 0, kSrcGlobal, true>(pp, l, tx, ts, tz, stream);
    }
    RB200_CHECK(false, "the fused all-reduce epilogue covers symmetric weights with group-32 scales (int4) or "
                "per-channel scales; got group code %d, scale source %d, zero mode %d", l.group_code, l.src, ZMODE);
  }
#define RB200_CASE(G, S) \
  if (l.group_code == (G) && l.src == (S)) return launch_inst<BITS, MT, ZMODE, G, S>(pp, l, tx, ts, tz, stream)
  RB200_CASE(32, kSrcGlobal);
  RB200_CASE(64, kSrcGlobal);
  RB200_CASE(128, kSrcGlobal);
  RB200_CASE(0, kSrcGlobal);
  RB200_CASE(-1, kSrcGlobal);
  if (BITS == 4) RB200_CASE(32, kSrcSmemNK);
  RB200_CASE(32, kSrcSmemKN);
  RB200_CASE(64, kSrcSmemKN);
  RB200_CASE(128, kSrcSmemKN);
#undef RB200_CASE
  RB200_CHECK(false, "no decode kernel for group code %d with scale source %d", l.group_code, l.src);
  return -1;
}

template <int BITS>
int launch_bits(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& ts, const CUtensorMap& tz,
                cudaStream_t stream) {
#define RB200_MZ(M, Z) \
  if (l.mt == (M) && l.zmode == (Z)) return launch_gs<BITS, M, Z>(pp, l, tx, ts, tz, stream)
  RB200_MZ(1, kZeroConstInt);
  RB200_MZ(2, kZeroConstInt);
  RB200_MZ(4, kZeroConstInt);
  RB200_MZ(1, kZeroGeneral);
  RB200_MZ(2, kZeroGeneral);
  RB200_MZ(4, kZeroGeneral);
#undef RB200_MZ
  RB200_CHECK(false, "bad m-tile count %d / zero mode %d", l.mt, l.zmode);
  return -1;
}

}  // namespace sk
}  // namespace rb200
