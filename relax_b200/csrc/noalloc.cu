// Decode-path entry point for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot let it call cudaMalloc: runtimes that reserve the whole
// device for their own pool at start-up (a later driver allocation simply fails with
// out-of-memory), and serving loops that ban driver allocation calls on the hot thread because
// such a call stalls every stream of the device.  For them the split-k scratch of the decode
// kernel (fp32 partial fragments, per-row-block tickets, the status word) lives in a fixed
// array that is part of the library image instead of in the lazily allocated per-device block
// that rb200_gemm_fp16_intx uses.  The price is a size limit and 5 MiB + 64.25 KiB of device
// memory held by every GPU that loads the library, until the process exits.
#include <cstring>
#include <mutex>

#include "../../include/relax_b200.h"
#include "dequant.cuh"
#include "gemv.h"

namespace rb200 {
namespace {

constexpr size_t kHeaderBytes = 256;                       // status word
constexpr size_t kCounterInts = 16384;                     // one ticket per 16 rows: n <= 262144
constexpr size_t kCounterBytes = kCounterInts * sizeof(int);
constexpr size_t kPartialBytes = 5u << 20;                 // fp32 partials: enough for m <= 16 on 148 SMs
constexpr size_t kScratchBytes = kHeaderBytes + kCounterBytes + kPartialBytes;
constexpr int kMaxRows = 16;

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table,
// not a device address; the address a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct PerDevice {
  unsigned char* base = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
PerDevice g_per_device[kMaxDevices];
std::mutex g_setup_mutex;

// Once per device, with that device current: resolve the array's device address.
int setup_current_device(PerDevice** out) {
  int dev = -1;
  RB200_CUDA(cudaGetDevice(&dev));
  RB200_CHECK(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  PerDevice& pd = g_per_device[dev];
  if (!pd.base) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    RB200_CHECK(e == cudaSuccess && ptr != nullptr,
                "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev,
                cudaGetErrorString(e));
    int sms = 0;
    RB200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    pd.sm_count = sms;
    pd.base = static_cast<unsigned char*>(ptr);
  }
  *out = &pd;
  return 0;
}

bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// The status word of the static array on the current device, for rb200_check_async_error: read
// (and cleared when set) with plain copies, so asking never allocates.  0 when the no-alloc entry
// has not run on this device.
int noalloc_read_status(int* status_out) {
  *status_out = 0;
  int dev = -1;
  RB200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return 0;
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    base = g_per_device[dev].base;
  }
  if (!base) return 0;
  int v = 0;
  RB200_CUDA(cudaMemcpy(&v, base, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) RB200_CUDA(cudaMemset(base, 0, sizeof(int)));
  *status_out = v;
  return 0;
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200_gemm_fp16_intx_noalloc(const rb200_gemm_desc* d, void* stream_v) {
  RB200_CHECK(d != nullptr, "descriptor is NULL");
  RB200_CHECK(d->struct_size == sizeof(rb200_gemm_desc), "descriptor struct_size %u != %zu",
              d->struct_size, sizeof(rb200_gemm_desc));
  RB200_CHECK(d->weight_bits == 4 || d->weight_bits == 8, "weight_bits must be 4 or 8, got %d",
              d->weight_bits);
  const int frag = d->weight_bits == 4 ? 64 : 32;
  RB200_CHECK(d->m >= 0, "m must be >= 0");
  if (d->m == 0) return 0;
  RB200_CHECK(d->m <= kMaxRows,
              "rb200_gemm_fp16_intx_noalloc handles m <= %d (its fixed scratch holds no more); got m=%lld",
              kMaxRows, (long long)d->m);
  RB200_CHECK(d->x && d->w && d->scales && d->out, "x, w, scales and out must be non-NULL");
  RB200_CHECK(d->n > 0 && d->k > 0 && d->n % 16 == 0 && d->k % frag == 0,
              "need n %% 16 == 0 and k %% %d == 0 (n=%lld, k=%lld)", frag, (long long)d->n,
              (long long)d->k);
  RB200_CHECK(d->n / 16 <= (int64_t)kCounterInts && d->k < (1ll << 31),
              "n=%lld exceeds the fixed scratch limit of %zu rows", (long long)d->n,
              kCounterInts * 16);
  const int64_t ldx = d->ldx > 0 ? d->ldx : d->k;
  const int64_t ldo = d->ldo > 0 ? d->ldo : d->n;
  RB200_CHECK(is_aligned16(d->x) && is_aligned16(d->w) && ldx % 8 == 0,
              "x and w must be 16-byte aligned with ldx %% 8 == 0");
  RB200_CHECK(d->activation != RB200_ACT_SWIGLU,
              "rb200_gemm_fp16_intx_noalloc has no fused gate/up form: run the plain matmul and gate afterwards, "
              "or use rb200_gemm_fp16_intx");
  RB200_CHECK(d->activation >= RB200_ACT_IDENTITY && d->activation <= RB200_ACT_GELU, "unknown activation code %d",
              d->activation);
  RB200_CHECK(d->binary_op >= RB200_BIN_NONE && d->binary_op <= RB200_BIN_MULTIPLY, "unknown binary_op code %d",
              d->binary_op);
  RB200_CHECK(d->unary_op >= RB200_UN_IDENTITY && d->unary_op <= RB200_UN_RELU, "unknown unary_op code %d",
              d->unary_op);
  RB200_CHECK(d->binary_op == RB200_BIN_NONE || d->residual, "binary_op needs a residual tensor");
  RB200_CHECK(d->bias_stride == 0 || d->bias_stride == d->n, "bias_stride must be 0 or n");
  const int group = (d->group_size <= 0 || d->group_size >= d->k) ? 0 : (int)d->group_size;
  if (group) {
    RB200_CHECK(d->k % group == 0 && group % (frag / 4) == 0,
                "group_size=%d must divide k=%lld and be a multiple of %d", group, (long long)d->k,
                frag / 4);
  }

  PerDevice* pd = nullptr;
  if (setup_current_device(&pd) != 0) return -1;

  GemvPlan plan;
  if (gemv_plan(d->weight_bits, (int)d->m, (int)d->n, (int)d->k, pd->sm_count, 0, 0, &plan) != 0)
    return -1;
  RB200_CHECK(plan.partial_bytes <= kPartialBytes && plan.counter_ints <= kCounterInts,
              "problem needs %zu bytes of split-k scratch, the fixed array holds %zu",
              plan.partial_bytes, kPartialBytes);

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // The array keeps whatever the previous call left: the tickets must start at zero.  The status
  // word is left alone - a wait that gave up in an earlier call stays visible until
  // rb200_check_async_error reads and clears it.
  RB200_CUDA(cudaMemsetAsync(pd->base + kHeaderBytes, 0, kCounterBytes, stream));

  int zmode = kZeroGeneral;
  if (!d->zeros) {
    const float z = d->zero_const;
    if (z >= 0.0f && z <= 255.0f && z == (float)(int)z) zmode = kZeroConstInt;
  }
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.status = reinterpret_cast<int*>(pd->base);
  p.counters = reinterpret_cast<int*>(pd->base + kHeaderBytes);
  p.partial = reinterpret_cast<float*>(pd->base + kHeaderBytes + kCounterBytes);
  p.x = static_cast<const __half*>(d->x);
  p.ldx = ldx;
  p.w = static_cast<const uint8_t*>(d->w);
  p.s = static_cast<const __half*>(d->scales);
  p.z = static_cast<const __half*>(d->zeros);
  p.s_n = d->scale_stride_n;
  p.s_g = d->scale_stride_g;
  p.out = static_cast<__half*>(d->out);
  p.ldo = ldo;
  p.epi.bias = static_cast<const __half*>(d->bias);
  p.epi.bias_stride = d->bias_stride;
  p.epi.residual = d->binary_op == RB200_BIN_NONE ? nullptr : static_cast<const __half*>(d->residual);
  p.epi.ld_res = d->n;
  p.epi.act = d->activation;
  p.epi.binop = d->binary_op;
  p.epi.unop = d->unary_op;
  p.m = (int)d->m;
  p.n = (int)d->n;
  p.k = (int)d->k;
  p.group = group;
  p.zero_const = d->zero_const;
  return gemv_launch(p, plan, d->weight_bits, zmode, stream);
}
