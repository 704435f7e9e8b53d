// Low-latency sum all-reduce for the row-parallel decode outputs (messages of a few KB to a few
// hundred KB): one kernel per rank, one exchange of flags, partial sums pulled from the peers'
// memory over NVLink with ordinary loads.  Stands in for the one-shot strategy of the reference's
// customized all-reduce (src/runtime/disco/cuda_ipc/custom_allreduce.cc:65-105,
// 3rdparty/tensorrt_llm/custom_allreduce_kernels.cu:120-264); larger messages stay on NCCL, as
// the reference falls back to ncclAllReduce (custom_allreduce.cc:69-76).
//
// Every rank owns a workspace that its peers can address (CUDA IPC, mapped at set-up):
//     [ call counters: 64 x u32 | flags: 8 ranks x 64 CTAs x u32 | pad to 4 KB | data 0 | data 1 ]
// CTA c of rank r: copies slice c of its input into its own data region (parity of the call
// number), then stores the call number into flag [r][c] of EVERY rank's workspace
// (st.release.sys), waits - bounded - until flag [p][c] of its own workspace shows the call
// number for every peer p, then sums slice c over all ranks in rank order (fp32, one rounding to
// fp16: every rank computes bit-identical results) and writes its output.  Synchronisation is per
// slice: CTA c only ever needs the peers' CTA c.  The call number lives on the device (one
// counter per CTA index), so a CUDA graph that replays the same launch keeps working; the two
// data regions alternate because a peer may still be reading call i while this rank has moved on
// to call i + 1 (it cannot have reached call i + 2: that needs the peer's flag of call i + 1,
// which the peer writes after it finished call i).  Every call runs the same 32 CTAs so that all
// counters advance together.  No multicast objects, no collective library.
#include <cooperative_groups.h>

#include <cstring>

#include "../../include/relax_b200.h"
#include "common.cuh"

namespace rb200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 64;
constexpr int kArThreads = 256;
constexpr size_t kHeaderBytes = 4096;

struct ArParams {
  uint8_t* ws[kMaxRanks];        // every rank's workspace, addressed from this GPU
  const __half* in[kMaxRanks];   // used entries: [rank_base .. rank_base + gridDim.y)
  __half* out[kMaxRanks];
  int world;
  int rank_base;                 // real launch: this rank; self-test: 0 with gridDim.y = world
  long long count;               // fp16 elements
  long long region_bytes;        // size of one data region
  unsigned long long wait_limit_ns;
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
  const int r = p.rank_base + blockIdx.y;
  const int c = blockIdx.x;
  const int nct = gridDim.x;
  const int tid = threadIdx.x;
  __shared__ uint32_t s_call;
  __shared__ int s_fail;

  // Launch overlap: the next kernel on the stream (usually the next layer's matmul) may become
  // resident next to these 32 small CTAs and stream its weights while the exchange runs; this
  // kernel itself touches nothing - not even its call counters, which the previous all-reduce
  // may still be updating - before everything ahead of it on the stream has completed.
  griddep_launch_dependents();
  griddep_wait();
  uint32_t* counters = reinterpret_cast<uint32_t*>(p.ws[r]);
  uint32_t* my_flags = counters + kMaxCtas;
  if (tid == 0) {
    s_call = counters[c] + 1u;
    s_fail = 0;
  }
  __syncthreads();
  const uint32_t call = s_call;

  // slice of this CTA, in 8-element (16-byte) units
  const long long units = (p.count + 7) / 8;
  const long long per = (units + nct - 1) / nct;
  const long long u0 = per * c, u1 = min(units, per * (c + 1));
  const size_t region = kHeaderBytes + (size_t)(call & 1u) * (size_t)p.region_bytes;

  // 1. publish this rank's slice in its own workspace
  {
    uint4* dst = reinterpret_cast<uint4*>(p.ws[r] + region);
    const __half* src = p.in[r];
    for (long long u = u0 + tid; u < u1; u += kArThreads) {
      uint4 v;
      if (u * 8 + 8 <= p.count) {
        v = *reinterpret_cast<const uint4*>(src + u * 8);
      } else {  // ragged end: zero-padded
        __half tmp[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) tmp[i] = (u * 8 + i < p.count) ? src[u * 8 + i] : __float2half_rn(0.0f);
        v = *reinterpret_cast<uint4*>(tmp);
      }
      dst[u] = v;
    }
  }
  __syncthreads();
  // 2. tell every rank (this one included) that slice c of rank r is there; wait for the peers.
  // One system-scope fence per signalling thread: the block barrier orders the other threads'
  // stores before it (a fence in every thread costs several microseconds per call).
  if (tid < p.world) {
    __threadfence_system();
    uint32_t* peer_flags = reinterpret_cast<uint32_t*>(p.ws[tid]) + kMaxCtas;
    st_release_sys(peer_flags + r * kMaxCtas + c, call);
  }
  if (tid < p.world) {
    const uint32_t* f = my_flags + tid * kMaxCtas + c;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    // flags only grow: a peer may already be one call ahead
    while ((int32_t)(ld_acquire_sys(f) - call) < 0) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > p.wait_limit_ns) {  // give up, report, leave the output unwritten
        if (p.status) atomicExch(p.status, kStatusWaitTimeout);
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_fail) {
    // 3. pull slice c from every rank, fixed order, fp32 sum, one rounding
    __half* out = p.out[r];
    for (long long u = u0 + tid; u < u1; u += kArThreads) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      for (int q = 0; q < p.world; ++q) {
        const uint4 v = ld_volatile_v4(p.ws[q] + region + (size_t)u * 16);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
      __half res[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = __float2half_rn(acc[i]);
      if (u * 8 + 8 <= p.count) {
        *reinterpret_cast<uint4*>(out + u * 8) = *reinterpret_cast<uint4*>(res);
      } else {
        for (int i = 0; i < 8 && u * 8 + i < p.count; ++i) out[u * 8 + i] = res[i];
      }
    }
  }
  __syncthreads();
  if (tid == 0) counters[c] = call;
}

// Every call uses the same number of CTAs whatever the message size: the per-CTA call counters of
// all ranks then advance in lockstep, which is what makes the two alternating data regions safe
// (a rank cannot start call i + 2 before every CTA of every peer has finished reading call i).
constexpr int kArCtas = 32;
int grid_for(long long) { return kArCtas; }

int check_common(int world, long long count, long long max_count, const void* in, const void* out) {
  RB200_CHECK(world >= 1 && world <= kMaxRanks, "world=%d outside [1, %d]", world, kMaxRanks);
  RB200_CHECK(count >= 0 && count <= max_count, "count=%lld exceeds the workspace's max_count=%lld", count, max_count);
  RB200_CHECK((reinterpret_cast<uintptr_t>(in) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
              "in and out must be 16-byte aligned");
  return 0;
}

long long region_bytes_for(long long max_count) { return ((max_count * 2 + 255) / 256) * 256; }

}  // namespace
}  // namespace rb200

using namespace rb200;

extern "C" {

size_t rb200_allreduce_workspace_bytes(int64_t max_count) {
  if (max_count < 0) return 0;
  return kHeaderBytes + 2 * (size_t)region_bytes_for(max_count);
}

int rb200_allreduce_oneshot(void* const* workspaces, int rank, int world, const void* in, void* out, int64_t count,
                            int64_t max_count, void* stream) {
  RB200_CHECK(workspaces != nullptr && in && out, "workspaces, in and out must be non-NULL");
  if (check_common(world, count, max_count, in, out) != 0) return -1;
  RB200_CHECK(rank >= 0 && rank < world, "rank=%d outside [0, %d)", rank, world);
  if (count == 0) return 0;
  DeviceScratch* sc = device_scratch(0, 0);
  if (!sc) return -1;
  ArParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < world; ++i) {
    RB200_CHECK(workspaces[i] != nullptr, "workspace of rank %d is NULL", i);
    p.ws[i] = static_cast<uint8_t*>(workspaces[i]);
  }
  p.in[rank] = static_cast<const __half*>(in);
  p.out[rank] = static_cast<__half*>(out);
  p.world = world;
  p.rank_base = rank;
  p.count = count;
  p.region_bytes = region_bytes_for(max_count);
  p.status = sc->status;
  p.wait_limit_ns = (wait_limit_ms() ? (unsigned long long)wait_limit_ms() : 2000ull) * 1000000ull;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid_for(count), 1, 1);
  cfg.blockDim = dim3(kArThreads, 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = launch_overlap_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RB200_CUDA(cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel, p));
  return 0;
}

int rb200_allreduce_oneshot_selftest(void* const* workspaces, const void* const* ins, void* const* outs, int world,
                                     int64_t count, int64_t max_count, void* stream) {
  RB200_CHECK(workspaces && ins && outs, "workspaces, ins and outs must be non-NULL");
  if (check_common(world, count, max_count, ins[0], outs[0]) != 0) return -1;
  if (count == 0) return 0;
  DeviceScratch* sc = device_scratch(0, 0);
  if (!sc) return -1;
  ArParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < world; ++i) {
    RB200_CHECK(workspaces[i] && ins[i] && outs[i], "NULL pointer for rank %d", i);
    p.ws[i] = static_cast<uint8_t*>(workspaces[i]);
    p.in[i] = static_cast<const __half*>(ins[i]);
    p.out[i] = static_cast<__half*>(outs[i]);
  }
  p.world = world;
  p.rank_base = 0;
  p.count = count;
  p.region_bytes = region_bytes_for(max_count);
  p.status = sc->status;
  p.wait_limit_ns = (wait_limit_ms() ? (unsigned long long)wait_limit_ms() : 2000ull) * 1000000ull;
  // all ranks' CTAs wait on one another: a cooperative launch guarantees they are co-resident
  void* args[] = {&p};
  RB200_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_oneshot_kernel),
                                         dim3(grid_for(count), world, 1), dim3(kArThreads, 1, 1), args, 0,
                                         static_cast<cudaStream_t>(stream)));
  return 0;
}

int rb200_peer_alloc(size_t bytes, void** ptr) {
  RB200_CHECK(ptr != nullptr && bytes > 0, "bad arguments");
  RB200_CUDA(cudaMalloc(ptr, bytes));
  RB200_CUDA(cudaMemset(*ptr, 0, bytes));
  RB200_CUDA(cudaDeviceSynchronize());
  return 0;
}
int rb200_peer_free(void* ptr) {
  if (ptr) RB200_CUDA(cudaFree(ptr));
  return 0;
}
int rb200_peer_export(void* ptr, void* handle_out) {
  RB200_CHECK(ptr && handle_out, "bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == RB200_PEER_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  RB200_CUDA(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int rb200_peer_import(const void* handle, void** ptr) {
  RB200_CHECK(handle && ptr, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  RB200_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int rb200_peer_close(void* ptr) {
  if (ptr) RB200_CUDA(cudaIpcCloseMemHandle(ptr));
  return 0;
}

}  // extern "C"
