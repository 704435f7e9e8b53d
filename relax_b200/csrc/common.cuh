// Shared host/device helpers: thread-local error string, CUDA checks, PTX wrappers for
// mbarrier / bulk async copies / legacy warp MMA, and bounded waits.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

namespace rb200 {

// ---------------------------------------------------------------- host-side error plumbing
void set_last_error(const char* fmt, ...);

#define RB200_CHECK(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      ::rb200::set_last_error(__VA_ARGS__); \
      return -1;                          \
    }                                     \
  } while (0)

#define RB200_CUDA(expr)                                                                  \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      ::rb200::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                              __FILE__, __LINE__);                                        \
      return -1;                                                                          \
    }                                                                                     \
  } while (0)

// Per-device library-owned state (scratch for split-K partials, tile counters, status word).
struct DeviceScratch {
  void* base = nullptr;     // one cudaMalloc: [status word | counters | partials]
  size_t bytes = 0;
  int* status = nullptr;    // device int, set by bounded waits that gave up
  int* counters = nullptr;  // zero-initialised tickets, self-resetting
  size_t counter_ints = 0;
  float* partials = nullptr;
  size_t partial_bytes = 0;
  int sm_count = 0;
};
// Returns the current device's scratch, allocating it on first use (never inside a capture:
// call once during warm-up).  nullptr + last error set on failure.
DeviceScratch* device_scratch(size_t min_partial_bytes, size_t min_counter_ints);
// The current device's scratch if some earlier call created it, else nullptr; never allocates.
DeviceScratch* device_scratch_if_any();
// Status word of the no-alloc entry point's static array on the current device (0 when that
// entry has not been used on it); reads and clears it without allocating anything.
int noalloc_read_status(int* status_out);
// Upper bound, in milliseconds, of the waits on flags written by other CTAs or other GPUs
// (split-k fix-up, all-reduce); 0 = the default of about two seconds.  See rb200_set_wait_limit_ms.
unsigned wait_limit_ms();

// Launch overlap (programmatic dependent launch): when the host enabled it, matmul kernels are
// launched so that they may start - and stream their weights - while the previous kernel on the
// stream is still finishing.  See rb200_set_launch_overlap in the public header.
bool launch_overlap_enabled();

// Number of SMs of the current device (queried once per device, no allocation).
int sm_count_current();

// Status codes written to the device status word.
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadConfig = 2 };

// ---------------------------------------------------------------- device-side PTX helpers
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after ~2^31 clock ticks (about a second), records the failure in the
// global status word and returns false; callers then skip their work and fall through to the
// end of the kernel so the context stays usable.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > (1ll << 31)) {
      if (status) atomicExch(status, kStatusWaitTimeout);
      return false;
    }
  }
}

// try_wait with a suspend-time hint: the hardware parks the thread until the phase completes or
// the hint (ns) expires, so a waiting warp neither burns issue slots nor wakes late.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, int* status) {
  // each try parks the thread for up to ~10 us; 200k tries bound the wait to about two seconds
#pragma unroll 1
  for (int i = 0; i < 200000; ++i)
    if (mbar_try_wait_hint(bar, parity, 10000u)) return true;
  if (status) atomicExch(status, kStatusWaitTimeout);
  return false;
}

// Same, for roles with slack (producer, MMA issuer): sleeps between polls so the waiting warp
// does not take issue slots from the warps doing the arithmetic.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(40);
    }
    if (clock64() - t0 > (1ll << 31)) {
      if (status) atomicExch(status, kStatusWaitTimeout);
      return false;
    }
  }
}

// 1-D bulk async copy global -> shared, completion counted on an mbarrier (both addresses and
// the size must be multiples of 16 bytes).
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Programmatic dependent launch.  launch_dependents: the next kernel on the stream may begin
// once every CTA of this grid has executed it (or exited).  wait: blocks until the kernels this
// grid depends on have completed and their memory is visible; returns at once for an ordinary
// launch.  Everything the previous kernel may have produced (activations) is read after wait,
// and every global write of this grid (outputs, scratch) comes after it too.
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_nc_u16(const __half* p) {
  unsigned short v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

#endif  // __CUDACC__

}  // namespace rb200
