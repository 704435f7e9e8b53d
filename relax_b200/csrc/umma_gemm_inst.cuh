// Instantiation + dispatch of umma_gemm_kernel for one weight width and zero-point mode.
#pragma once
#include "umma_gemm.cuh"

namespace rb200 {
namespace um {

template <int BITS, int ZMODE, int GROUP, int SRC, bool SPLITK>
int launch_inst2(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& tw, cudaStream_t stream) {
  auto kern = umma_gemm_kernel<BITS, ZMODE, GROUP, SRC, SPLITK>;
  static thread_local int configured_device = -1;
  int dev = 0;
  RB200_CUDA(cudaGetDevice(&dev));
  if (configured_device != dev) {
    RB200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_device = dev;
  }
  kern<<<l.grid, kThreads, l.smem, stream>>>(pp, tx, tw);
  RB200_CUDA(cudaGetLastError());
  return 0;
}

template <int BITS, int ZMODE, int GROUP, int SRC>
int launch_inst(const Params& pp, const Launch& l, const CUtensorMap& tx, const CUtensorMap& tw, cudaStream_t stream) {
  if (pp.k_splits > 1) return launch_inst2<BITS, ZMODE, GROUP, SRC, true>(pp, l, tx, tw, stream);
  return launch_inst2<BITS, ZMODE, GROUP, SRC, false>(pp, l, tx, tw, stream);
}

template <int BITS, int ZMODE>
int launch_gs(const Params& pp, const Launch& l, const CUtensorMap& tx, cudaStream_t stream) {
#define RB200_CASE(G, S) \
  if (l.group_code == (G) && l.src == (S)) return launch_inst<BITS, ZMODE, G, S>(pp, l, tx, tx, stream)
  RB200_CASE(0, kSrcGlobal);
  RB200_CASE(-1, kSrcGlobal);
  if constexpr (BITS == 4) {
    RB200_CASE(32, kSrcGlobal);
    RB200_CASE(64, kSrcGlobal);
    RB200_CASE(128, kSrcGlobal);
    RB200_CASE(32, kSrcSmemNK);
    RB200_CASE(32, kSrcSmemKN);
    RB200_CASE(64, kSrcSmemKN);
    RB200_CASE(128, kSrcSmemKN);
  }
#undef RB200_CASE
  RB200_CHECK(false, "no prefill kernel for group code %d with scale source %d", l.group_code, l.src);
  return -1;
}

}  // namespace um
}  // namespace rb200
