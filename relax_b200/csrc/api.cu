// C ABI entry points: argument validation, per-device scratch, kernel selection.
// No entry point here allocates after its first call on a device, synchronises, or falls back
// to a host computation.
#include <cstring>
#include <atomic>
#include <mutex>

#include "../../include/relax_b200.h"
#include "dequant.cuh"
#include "gemv.h"
#include "gemv_cluster.cuh"
#include "umma_gemm.cuh"
#include "gemv_sk.cuh"
#include "gemm_tc.h"
#include "preprocess.h"

namespace rb200 {

// ---------------------------------------------------------------- errors
static thread_local std::string g_last_error;
static thread_local cudaStream_t g_stream = nullptr;

void set_last_error(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

// ---------------------------------------------------------------- per-device scratch
namespace {
constexpr int kMaxDevices = 64;
// split-k flags of the stream-k decode kernel: inside the ticket area of the scratch block
constexpr size_t kSkFlagOffset = 49152, kSkFlagCount = 16384;
DeviceScratch g_scratch[kMaxDevices];
std::mutex g_scratch_mutex;
}  // namespace

int sm_count_current() {
  static std::atomic<int> cached[kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int v = cached[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  cached[dev].store(v, std::memory_order_relaxed);
  return v;
}

// The current device's scratch if it has been created, else nullptr: never allocates.
DeviceScratch* device_scratch_if_any() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  return g_scratch[dev].base ? &g_scratch[dev] : nullptr;
}

DeviceScratch* device_scratch(size_t min_partial_bytes, size_t min_counter_ints) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_last_error("cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  DeviceScratch& s = g_scratch[dev];
  if (s.base && s.partial_bytes >= min_partial_bytes && s.counter_ints >= min_counter_ints) return &s;
  if (s.base) {
    // growing: the old block may still be in use by queued kernels, so drain the device first
    cudaDeviceSynchronize();
    cudaFree(s.base);
    s.base = nullptr;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    set_last_error("cudaGetDeviceProperties failed");
    return nullptr;
  }
  s.sm_count = prop.multiProcessorCount;
  // generous defaults so ordinary use never grows: partials for 2 CTAs/SM at m <= 32
  size_t partial = (size_t)s.sm_count * 2 * 2 * 8 * 4 * 128 * sizeof(float);
  // and for the split-k form of the prefill kernel: one 128 x 256 fp32 partial tile per SM
  if (partial < (size_t)s.sm_count * 128 * 256 * sizeof(float)) partial = (size_t)s.sm_count * 128 * 256 * sizeof(float);
  if (partial < min_partial_bytes) partial = min_partial_bytes;
  size_t counters = 1u << 16;
  if (counters < min_counter_ints) counters = min_counter_ints;
  const size_t header = 256;
  const size_t counter_bytes = ((counters * sizeof(int) + 255) / 256) * 256;
  s.bytes = header + counter_bytes + partial;
  cudaError_t e = cudaMalloc(&s.base, s.bytes);
  if (e != cudaSuccess) {
    set_last_error("cudaMalloc(%zu) for library scratch failed: %s", s.bytes, cudaGetErrorString(e));
    s.base = nullptr;
    return nullptr;
  }
  cudaMemset(s.base, 0, header + counter_bytes);
  s.status = static_cast<int*>(s.base);
  s.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(s.base) + header);
  s.counter_ints = counters;
  s.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(s.base) + header + counter_bytes);
  s.partial_bytes = partial;
  return &s;
}

// ---------------------------------------------------------------- dequantize (debug) kernel
namespace {

template <int BITS, int ZMODE>
__global__ void dequantize_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ s,
                                  const __half* __restrict__ z, int64_t s_n, int64_t s_g, int group,
                                  float zero_const, int64_t N, int64_t K, __half* __restrict__ wq) {
  constexpr int kFrag = BITS == 4 ? 64 : 32;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int64_t KB = K / kFrag;
  const int64_t tiles = (N / 16) * KB;
  const ZeroConsts zc = make_zero_consts(ZMODE, zero_const);
  const uint32_t zconst_h2 = h2_bcast(__float2half_rn(zero_const));
  for (int64_t tile = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5); tile < tiles;
       tile += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t nb = tile / KB, kb = tile % KB;
    const uint4 wv = reinterpret_cast<const uint4*>(w + frag_tile_offset(nb, kb, N / 16, KB))[frag_unit_pos(lane)];
    const int64_t n_g = nb * 16 + g;
    const int64_t k0 = kb * kFrag + t * (kFrag / 4);
    const int64_t grp = k0 / group;
    const int64_t o_g = n_g * s_n + grp * s_g, o_g8 = o_g + 8 * s_n;
    const uint32_t s_gv = h2_bcast(s[o_g]), s_g8v = h2_bcast(s[o_g8]);
    uint32_t z_g = zconst_h2, z_g8 = zconst_h2;
    if (ZMODE == kZeroGeneral && z) {
      z_g = h2_bcast(z[o_g]);
      z_g8 = h2_bcast(z[o_g8]);
    }
    uint32_t* row_g = reinterpret_cast<uint32_t*>(wq + n_g * K + k0);
    uint32_t* row_g8 = reinterpret_cast<uint32_t*>(wq + (n_g + 8) * K + k0);
    if (BITS == 4) {
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a[4];
        decode_int4_word<ZMODE>(ww[j], zc, s_gv, s_g8v, z_g, z_g8, a);
        row_g[2 * j] = a[0];
        row_g[2 * j + 1] = a[2];
        row_g8[2 * j] = a[1];
        row_g8[2 * j + 1] = a[3];
      }
    } else {
      uint32_t a[4];
      decode_int8_pair<ZMODE>(wv.x, wv.y, zc, s_gv, s_g8v, z_g, z_g8, a);
      row_g[0] = a[0];
      row_g[1] = a[2];
      row_g8[0] = a[1];
      row_g8[1] = a[3];
      decode_int8_pair<ZMODE>(wv.z, wv.w, zc, s_gv, s_g8v, z_g, z_g8, a);
      row_g[2] = a[0];
      row_g[3] = a[2];
      row_g8[2] = a[1];
      row_g8[3] = a[3];
    }
  }
}

int parse_act(const char* s, int* out) {
  if (!s || !*s || !strcmp(s, "identity")) return *out = RB200_ACT_IDENTITY, 0;
  if (!strcmp(s, "relu")) return *out = RB200_ACT_RELU, 0;
  if (!strcmp(s, "silu")) return *out = RB200_ACT_SILU, 0;
  if (!strcmp(s, "gelu")) return *out = RB200_ACT_GELU, 0;
  if (!strcmp(s, "swiglu")) return *out = RB200_ACT_SWIGLU, 0;
  set_last_error("unknown activation '%s'", s);
  return -1;
}
int parse_bin(const char* s, int* out) {
  if (!s || !*s || !strcmp(s, "none")) return *out = RB200_BIN_NONE, 0;
  if (!strcmp(s, "plus")) return *out = RB200_BIN_PLUS, 0;
  if (!strcmp(s, "multiply")) return *out = RB200_BIN_MULTIPLY, 0;
  set_last_error("unknown binary_op '%s'", s);
  return -1;
}
int parse_un(const char* s, int* out) {
  if (!s || !*s || !strcmp(s, "identity")) return *out = RB200_UN_IDENTITY, 0;
  if (!strcmp(s, "relu")) return *out = RB200_UN_RELU, 0;
  set_last_error("unknown unary_op '%s'", s);
  return -1;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// zero-point mode for a descriptor: integer constants in [0, 255] fold into the exact path
int zero_mode(const rb200_gemm_desc* d) {
  if (d->zeros) return kZeroGeneral;
  float z = d->zero_const;
  if (z >= 0.0f && z <= 255.0f && z == (float)(int)z) return kZeroConstInt;
  return kZeroGeneral;
}

int validate_common(const rb200_gemm_desc* d) {
  RB200_CHECK(d != nullptr, "descriptor is NULL");
  RB200_CHECK(d->struct_size == sizeof(rb200_gemm_desc), "descriptor struct_size %u != %zu",
              d->struct_size, sizeof(rb200_gemm_desc));
  RB200_CHECK(d->weight_bits == 4 || d->weight_bits == 8, "weight_bits must be 4 or 8, got %d",
              d->weight_bits);
  RB200_CHECK(d->w && d->scales, "weight and scales must be non-NULL");
  RB200_CHECK(d->n > 0 && d->k > 0, "n and k must be positive (n=%lld k=%lld)", (long long)d->n,
              (long long)d->k);
  RB200_CHECK(d->n % 16 == 0, "n=%lld must be a multiple of 16", (long long)d->n);
  const int frag = d->weight_bits == 4 ? 64 : 32;
  RB200_CHECK(d->k % frag == 0, "k=%lld must be a multiple of %d for %d-bit weights",
              (long long)d->k, frag, d->weight_bits);
  RB200_CHECK(d->n < (1ll << 31) && d->k < (1ll << 31), "n and k must fit in 31 bits");
  RB200_CHECK(aligned16(d->w), "weight pointer must be 16-byte aligned");
  if (d->group_size > 0 && d->group_size < d->k) {
    RB200_CHECK(d->k % d->group_size == 0 && d->group_size % (frag / 4) == 0,
                "group_size=%lld must divide k=%lld and be a multiple of %d",
                (long long)d->group_size, (long long)d->k, frag / 4);
  }
  return 0;
}

}  // namespace
}  // namespace rb200

using namespace rb200;

namespace rb200 {
static std::atomic<int> g_launch_overlap{0};
static std::atomic<unsigned> g_wait_limit_ms{0};
bool launch_overlap_enabled() { return g_launch_overlap.load(std::memory_order_relaxed) != 0; }
unsigned wait_limit_ms() { return g_wait_limit_ms.load(std::memory_order_relaxed); }
}  // namespace rb200

extern "C" {

int rb200_set_launch_overlap(int enabled) {
  g_launch_overlap.store(enabled ? 1 : 0, std::memory_order_relaxed);
  return 0;
}
int rb200_get_launch_overlap(void) { return launch_overlap_enabled() ? 1 : 0; }

const char* rb200_last_error(void) { return g_last_error.c_str(); }

int rb200_set_stream(void* stream) {
  g_stream = static_cast<cudaStream_t>(stream);
  return 0;
}
void* rb200_get_stream(void) { return g_stream; }

int rb200_check_async_error(void* stream, int* status_out) {
  // Two status words can exist on a device: the one in the library's lazily allocated scratch
  // block (every entry point but the no-alloc one) and the one in the no-alloc entry's static
  // array.  Neither is created here: a host that only ever used the no-alloc entry must be
  // able to ask without triggering a device allocation.
  int st = 0;
  RB200_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  if (DeviceScratch* sc = device_scratch_if_any()) {
    int v = 0;
    RB200_CUDA(cudaMemcpy(&v, sc->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v != 0) {
      // a wait that gave up may have left split-k flags and tickets behind: back to rest
      RB200_CUDA(cudaMemset(sc->base, 0, (size_t)(reinterpret_cast<uint8_t*>(sc->partials) - static_cast<uint8_t*>(sc->base))));
      st = v;
    }
  }
  int v2 = 0;
  if (noalloc_read_status(&v2) != 0) return -1;
  if (st == 0) st = v2;
  if (status_out) *status_out = st;
  return 0;
}

int rb200_set_wait_limit_ms(unsigned limit_ms) {
  g_wait_limit_ms.store(limit_ms, std::memory_order_relaxed);
  return 0;
}

int rb200_preprocess_weight(const void* src, void* dst, int64_t num_experts, int64_t k, int64_t n,
                            int is_int4, int src_layout, void* stream) {
  RB200_CHECK(src && dst, "src and dst must be non-NULL");
  RB200_CHECK(src != dst, "preprocess cannot run in place");
  RB200_CHECK(num_experts >= 1, "num_experts must be >= 1");
  const int bits = is_int4 ? 4 : 8;
  const int frag = is_int4 ? 64 : 32;
  RB200_CHECK(n > 0 && k > 0 && n % 16 == 0 && k % frag == 0,
              "preprocess needs n %% 16 == 0 and k %% %d == 0 (n=%lld, k=%lld)", frag, (long long)n,
              (long long)k);
  const int base_layout = src_layout & ~RB200_LAYOUT_GATE_UP_INTERLEAVE;
  RB200_CHECK(base_layout == RB200_LAYOUT_FT_KN ||
                  ((base_layout == RB200_LAYOUT_Q4_NK || base_layout == RB200_LAYOUT_AUTOGPTQ_KN) && is_int4),
              "unsupported source layout %d for %d-bit weights", src_layout, bits);
  RB200_CHECK(!(src_layout & RB200_LAYOUT_GATE_UP_INTERLEAVE) || n % 32 == 0,
              "the gate/up interleave needs n %% 32 == 0 (n=%lld)", (long long)n);
  RB200_CHECK(aligned16(dst), "dst must be 16-byte aligned");
  RB200_CHECK(base_layout != RB200_LAYOUT_Q4_NK || (reinterpret_cast<uintptr_t>(src) & 7u) == 0,
              "a q4f16_1 source must be 8-byte aligned");
  return preprocess_launch(src, dst, num_experts, k, n, bits, src_layout, nullptr,
                           static_cast<cudaStream_t>(stream));
}

int rb200_gptq_act_order(const int32_t* g_idx, int64_t k, int64_t groups, int32_t* perm_out, void* stream) {
  RB200_CHECK(g_idx && perm_out, "g_idx and perm_out must be non-NULL");
  RB200_CHECK(k > 0 && groups > 0 && k % groups == 0 && k < (1ll << 30) && groups <= 8192,
              "need groups dividing k, at most 8192 groups (k=%lld, groups=%lld)", (long long)k, (long long)groups);
  // set-up time routine (once per weight): a status word of its own, read back before returning
  int* d_status = nullptr;
  RB200_CUDA(cudaMalloc(&d_status, sizeof(int)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = gptq_act_order_launch(g_idx, k, groups, perm_out, d_status, st);
  int h_status = -1;
  cudaError_t e = cudaSuccess;
  if (rc == 0) e = cudaMemcpyAsync(&h_status, d_status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (rc == 0 && e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(d_status);
  RB200_CUDA(e);
  if (rc != 0) return rc;
  RB200_CHECK(h_status == 0, "g_idx must give every one of the %lld groups exactly %lld rows", (long long)groups,
              (long long)(k / groups));
  return 0;
}

int rb200_preprocess_weight_autogptq_perm(const void* qweight, void* dst, int64_t k, int64_t n, const int32_t* perm,
                                          void* stream) {
  RB200_CHECK(qweight && dst && perm, "qweight, dst and perm must be non-NULL");
  RB200_CHECK(qweight != dst, "preprocess cannot run in place");
  RB200_CHECK(n > 0 && k > 0 && n % 16 == 0 && k % 64 == 0, "preprocess needs n %% 16 == 0 and k %% 64 == 0 (n=%lld, k=%lld)",
              (long long)n, (long long)k);
  RB200_CHECK(aligned16(dst), "dst must be 16-byte aligned");
  return preprocess_launch(qweight, dst, 1, k, n, 4, RB200_LAYOUT_AUTOGPTQ_KN, perm, static_cast<cudaStream_t>(stream));
}

int rb200_gather_columns(const void* x, const int32_t* perm, void* out, int64_t m, int64_t k, int64_t ldx, int64_t ldo,
                         void* stream) {
  RB200_CHECK(x && perm && out, "x, perm and out must be non-NULL");
  RB200_CHECK(x != out, "gather cannot run in place");
  RB200_CHECK(m >= 0 && k > 0 && ldx >= k && ldo >= k, "need ldx >= k and ldo >= k (k=%lld)", (long long)k);
  return gather_columns_launch(x, perm, out, m, k, ldx, ldo, static_cast<cudaStream_t>(stream));
}

int rb200_unpack_zeros_autogptq(const void* zq, void* zeros_out, int64_t groups, int64_t n, void* stream) {
  RB200_CHECK(zq && zeros_out, "zq and zeros_out must be non-NULL");
  RB200_CHECK(groups >= 1 && n >= 8 && n % 8 == 0, "need groups >= 1 and n %% 8 == 0 (groups=%lld, n=%lld)",
              (long long)groups, (long long)n);
  return unpack_zeros_autogptq_launch(zq, zeros_out, groups, n, static_cast<cudaStream_t>(stream));
}

int rb200_interleave_gate_up(const void* src, void* dst, int64_t outer, int64_t n, int64_t inner, void* stream) {
  RB200_CHECK(src && dst && src != dst, "src and dst must be distinct non-NULL tensors");
  RB200_CHECK(outer >= 1 && inner >= 1 && n > 0 && n % 32 == 0, "need outer, inner >= 1 and n %% 32 == 0 (n=%lld)",
              (long long)n);
  return interleave_rows_launch(src, dst, outer, n, inner, static_cast<cudaStream_t>(stream));
}

size_t rb200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int weight_bits) {
  if (m > 32) return 0;
  DeviceScratch* sc = device_scratch(0, 0);
  if (!sc) return 0;
  GemvPlan plan;
  if (gemv_plan(weight_bits, (int)m, (int)n, (int)k, sc->sm_count, 0, 0, &plan) != 0) return 0;
  return plan.partial_bytes + ((plan.counter_ints * sizeof(int) + 255) / 256) * 256 + 256;
}

// rb200_gemm_fp16_intx and its row-parallel form share one body; `ar` is nullptr for the former.
static int gemm_impl(const rb200_gemm_desc* d, const sk::ArCtx* ar, void* stream_v) {
  if (validate_common(d) != 0) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  RB200_CHECK(d->m >= 0, "m must be >= 0");
  if (d->m == 0) return 0;  // empty batch: nothing to launch (pointers of empty tensors may be NULL)
  RB200_CHECK(d->x && d->out, "x and out must be non-NULL");
  const int64_t ldx = d->ldx > 0 ? d->ldx : d->k;
  const bool swiglu = d->activation == RB200_ACT_SWIGLU;
  const int64_t ldo = d->ldo > 0 ? d->ldo : (swiglu ? d->n / 2 : d->n);
  RB200_CHECK(aligned16(d->x) && ldx % 8 == 0, "x must be 16-byte aligned with ldx %% 8 == 0");
  RB200_CHECK(d->activation >= RB200_ACT_IDENTITY && d->activation <= RB200_ACT_SWIGLU, "unknown activation code %d",
              d->activation);
  RB200_CHECK(d->binary_op >= RB200_BIN_NONE && d->binary_op <= RB200_BIN_MULTIPLY, "unknown binary_op code %d",
              d->binary_op);
  RB200_CHECK(d->unary_op >= RB200_UN_IDENTITY && d->unary_op <= RB200_UN_RELU, "unknown unary_op code %d",
              d->unary_op);
  RB200_CHECK(d->binary_op == RB200_BIN_NONE || d->residual, "binary_op needs a residual tensor");
  if (swiglu) {
    RB200_CHECK(!d->bias && d->binary_op == RB200_BIN_NONE && d->unary_op == RB200_UN_IDENTITY && !d->workspace,
                "the fused gate/up activation takes no bias, residual, unary op or caller workspace");
    RB200_CHECK(d->n % 32 == 0, "the fused gate/up activation needs n %% 32 == 0");
  }
  RB200_CHECK(d->bias_stride == 0 || d->bias_stride == d->n, "bias_stride must be 0 or n");

  Epilogue epi;
  epi.bias = static_cast<const __half*>(d->bias);
  epi.bias_stride = d->bias_stride;
  epi.residual = d->binary_op == RB200_BIN_NONE ? nullptr : static_cast<const __half*>(d->residual);
  epi.ld_res = d->n;
  epi.act = d->activation;
  epi.binop = d->binary_op;
  epi.unop = d->unary_op;
  const int group = (d->group_size <= 0 || d->group_size >= d->k) ? 0 : (int)d->group_size;

  if (ar) {
    RB200_CHECK(d->m <= 32, "the fused all-reduce form covers the decode path (m <= 32); reduce larger batches with "
                "a collective library after rb200_gemm_fp16_intx (m=%lld)", (long long)d->m);
    RB200_CHECK(!d->workspace && !swiglu && d->k % 64 == 0,
                "the fused all-reduce form takes no caller workspace, no gate/up activation, and needs k %% 64 == 0");
  }
  if (d->m <= 32 && !d->workspace) {
    DeviceScratch* sc = device_scratch(0, 0);
    if (!sc) return -1;
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
    // Which decode kernel: the stream-k kernel whenever x can be fetched as TMA tiles of whole
    // 64-k blocks (always for int4); the cluster kernel - split-k partials meeting in distributed
    // shared memory - for the remaining int8 shapes (k a multiple of 32 only).  Measured on B200
    // with launch overlap: stream-k is ahead at every size, 8.3 against 9.3 us at k = n = 4096.
    if (p.k % 64 == 0) {
      unsigned* flags = reinterpret_cast<unsigned*>(sc->counters) + kSkFlagOffset;
      return gemv_sk_run(p, d->weight_bits, zero_mode(d), sc->sm_count, sc->partials, sc->partial_bytes, flags,
                         kSkFlagCount, ar, nullptr, stream);
    }
    return gemv_cluster_run(p, d->weight_bits, zero_mode(d), sc->sm_count, stream);
  }
  if (d->m <= 32) {
    // caller-provided workspace: the ticket-based split-k kernel, partials in the caller's memory
    DeviceScratch* sc = device_scratch(0, 0);
    if (!sc) return -1;
    GemvPlan plan;
    if (gemv_plan(d->weight_bits, (int)d->m, (int)d->n, (int)d->k, sc->sm_count, 0, 0, &plan) != 0) return -1;
    GemvParams p;
    memset(&p, 0, sizeof(p));
    if (d->workspace) {
      // caller scratch: [counters (zeroed by the caller once, self-resetting) | partials]
      const size_t cbytes = ((plan.counter_ints * sizeof(int) + 255) / 256) * 256;
      RB200_CHECK(d->workspace_bytes >= cbytes + plan.partial_bytes && aligned16(d->workspace),
                  "workspace too small: need %zu bytes", cbytes + plan.partial_bytes);
      p.counters = static_cast<int*>(d->workspace);
      p.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(d->workspace) + cbytes);
    } else {
      if (sc->partial_bytes < plan.partial_bytes || sc->counter_ints < plan.counter_ints) {
        sc = device_scratch(plan.partial_bytes, plan.counter_ints);
        if (!sc) return -1;
      }
      p.counters = sc->counters;
      p.partial = sc->partials;
    }
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
    return gemv_launch(p, plan, d->weight_bits, zero_mode(d), stream);
  }
  return gemm_tc_launch(d, epi, group, zero_mode(d), ldx, ldo, stream);
}

int rb200_gemm_fp16_intx(const rb200_gemm_desc* d, void* stream_v) { return gemm_impl(d, nullptr, stream_v); }

size_t rb200_gemm_allreduce_workspace_bytes(int64_t max_n) {
  if (max_n <= 0) return 0;
  return sk::ar_workspace_bytes((unsigned)((max_n + 15) / 16));
}

int rb200_gemm_fp16_intx_allreduce(const rb200_gemm_desc* d, void* const* workspaces, int rank, int world,
                                   int64_t max_n, void* stream_v) {
  RB200_CHECK(world >= 1 && world <= sk::kArMaxRanks, "world=%d outside [1, %d]", world, sk::kArMaxRanks);
  RB200_CHECK(rank >= 0 && rank < world, "rank=%d outside [0, %d)", rank, world);
  if (world == 1) return gemm_impl(d, nullptr, stream_v);
  RB200_CHECK(workspaces != nullptr && max_n > 0, "workspaces must be non-NULL and max_n positive");
  sk::ArCtx ar;
  memset(&ar, 0, sizeof(ar));
  for (int i = 0; i < world; ++i) {
    RB200_CHECK(workspaces[i] != nullptr, "workspace of rank %d is NULL", i);
    ar.ws[i] = static_cast<uint8_t*>(workspaces[i]);
  }
  ar.rank = rank;
  ar.world = world;
  ar.max_blocks = (unsigned)((max_n + 15) / 16);
  return gemm_impl(d, &ar, stream_v);
}

int rb200_gemm_fp16_intx_allreduce_selftest(const rb200_gemm_desc* d, void* const* workspaces, int world,
                                            int64_t max_n, void* stream_v) {
  RB200_CHECK(world >= 2 && world <= sk::kArMaxRanks, "world=%d outside [2, %d]", world, sk::kArMaxRanks);
  RB200_CHECK(workspaces != nullptr && max_n > 0, "workspaces must be non-NULL and max_n positive");
  sk::ArCtx ar;
  memset(&ar, 0, sizeof(ar));
  for (int i = 0; i < world; ++i) {
    RB200_CHECK(workspaces[i] != nullptr, "workspace of rank %d is NULL", i);
    ar.ws[i] = static_cast<uint8_t*>(workspaces[i]);
  }
  ar.rank = 0;
  ar.world = world;
  ar.emulate = world;
  ar.max_blocks = (unsigned)((max_n + 15) / 16);
  return gemm_impl(d, &ar, stream_v);
}

static int fill_ft_desc(rb200_gemm_desc* d, const void* A, const void* B, const void* scales,
                        const void* bias, const void* residual, void* out, int m, int n, int k,
                        int group_size, int bias_stride, int weight_bits, void* workspace,
                        size_t workspace_bytes) {
  memset(d, 0, sizeof(*d));
  d->struct_size = sizeof(*d);
  d->weight_bits = weight_bits;
  d->x = A;
  d->w = B;
  d->scales = scales;
  d->bias = bias;
  d->residual = residual;
  d->out = out;
  d->m = m;
  d->n = n;
  d->k = k;
  d->ldx = k;
  d->ldo = 0;  // the entry point's default: n, or n / 2 for the fused gate/up activation
  const bool per_col = group_size <= 0 || group_size >= k;
  d->group_size = per_col ? k : group_size;
  d->scale_stride_n = 1;               // FT scales: [n] or [k/g, n]
  d->scale_stride_g = per_col ? 0 : n;
  d->bias_stride = bias_stride;
  d->zero_const = weight_bits == 4 ? 8.0f : 128.0f;  // preprocess biased the signed codes
  d->workspace = workspace;
  d->workspace_bytes = workspace_bytes;
  return 0;
}

int rb200_gemm_fp16_int_bias_act(const void* A, const void* B, const void* scales, const void* bias,
                                 void* out, const char* activation, int m, int n, int k,
                                 int group_size, int bias_stride, int weight_bits, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  rb200_gemm_desc d;
  fill_ft_desc(&d, A, B, scales, bias, nullptr, out, m, n, k, group_size, bias_stride, weight_bits,
               workspace, workspace_bytes);
  if (parse_act(activation, &d.activation) != 0) return -1;
  return rb200_gemm_fp16_intx(&d, stream);
}

int rb200_gemm_fp16_int_bias_act_residual(const void* A, const void* B, const void* scales,
                                          const void* bias, const void* residual, void* out,
                                          const char* activation, const char* binary_op,
                                          const char* unary_op, int m, int n, int k, int group_size,
                                          int weight_bits, void* workspace, size_t workspace_bytes,
                                          void* stream) {
  rb200_gemm_desc d;
  // the residual form of the reference call has no bias_stride argument: bias is a row vector
  fill_ft_desc(&d, A, B, scales, bias, residual, out, m, n, k, group_size, 0, weight_bits, workspace,
               workspace_bytes);
  if (parse_act(activation, &d.activation) != 0) return -1;
  if (parse_bin(binary_op, &d.binary_op) != 0) return -1;
  if (parse_un(unary_op, &d.unary_op) != 0) return -1;
  RB200_CHECK(residual != nullptr, "residual must be non-NULL");
  if (d.binary_op == RB200_BIN_NONE) d.binary_op = RB200_BIN_PLUS;
  return rb200_gemm_fp16_intx(&d, stream);
}

int rb200_group_gemm(const rb200_group_gemm_desc* d, void* stream_v) {
  RB200_CHECK(d != nullptr, "descriptor is NULL");
  RB200_CHECK(d->struct_size == sizeof(rb200_group_gemm_desc), "descriptor struct_size %u != %zu", d->struct_size,
              sizeof(rb200_group_gemm_desc));
  RB200_CHECK(d->weight_bits == 4 || d->weight_bits == 8 || d->weight_bits == 16,
              "weight_bits must be 4, 8 or 16, got %d", d->weight_bits);
  RB200_CHECK(d->num_experts >= 1, "num_experts must be >= 1");
  RB200_CHECK(d->n > 0 && d->k > 0 && d->n < (1ll << 31) && d->k < (1ll << 31), "bad n=%lld / k=%lld",
              (long long)d->n, (long long)d->k);
  RB200_CHECK(d->total_rows >= 0 && d->total_rows < (1ll << 31), "bad total_rows=%lld", (long long)d->total_rows);
  if (d->total_rows == 0) return 0;
  RB200_CHECK(d->x && d->w && d->indptr && d->out, "x, w, indptr and out must be non-NULL");
  RB200_CHECK(aligned16(d->w), "weight pointer must be 16-byte aligned");
  const bool packed = d->weight_bits != 16;
  RB200_CHECK(!packed || d->scales, "packed weights need scales");
  DeviceScratch* sc = device_scratch(0, 0);
  if (!sc) return -1;
  GemvParams p;
  memset(&p, 0, sizeof(p));
  p.status = sc->status;
  p.x = static_cast<const __half*>(d->x);
  p.ldx = d->k;
  p.w = static_cast<const uint8_t*>(d->w);
  p.s = static_cast<const __half*>(d->scales);
  p.z = static_cast<const __half*>(d->zeros);
  p.s_n = packed ? d->scale_stride_n : 1;
  p.s_g = d->scale_stride_g;
  p.out = static_cast<__half*>(d->out);
  p.ldo = d->n;
  memset(&p.epi, 0, sizeof(p.epi));
  p.m = (int)d->total_rows;
  p.n = (int)d->n;
  p.k = (int)d->k;
  p.group = (d->group_size <= 0 || d->group_size >= d->k) ? 0 : (int)d->group_size;
  p.zero_const = d->zero_const;
  const bool int_zero = d->zero_const >= 0.0f && d->zero_const <= 255.0f && d->zero_const == (float)(int)d->zero_const;
  const int zmode = (packed && (d->zeros || !int_zero)) ? kZeroGeneral : kZeroConstInt;
  const int64_t w_expert_bytes = d->n * d->k * d->weight_bits / 8;
  if (packed && d->total_rows <= 32 && d->k % 64 == 0 && d->n % 16 == 0 && aligned16(d->x) && aligned16(d->out)) {
    // Decode-size batch: the weights of an expert with rows are streamed once by the decode
    // kernel (one launch per expert; a launch whose expert has no rows returns at once), instead
    // of padding a handful of rows to a tensor-core tile of 192.
    unsigned* flags = reinterpret_cast<unsigned*>(sc->counters) + kSkFlagOffset;
    for (int e = 0; e < (int)d->num_experts; ++e) {
      GemvParams pe = p;
      pe.w = p.w + (int64_t)e * w_expert_bytes;
      pe.s = p.s + (int64_t)e * d->scale_stride_e;
      if (p.z) pe.z = p.z + (int64_t)e * d->scale_stride_e;
      sk::GroupCtx g;
      g.indptr = d->indptr;
      g.expert = e;
      g.has_prev = d->indptr_has_prev ? 1 : 0;
      if (gemv_sk_run(pe, d->weight_bits, zmode, sc->sm_count, sc->partials, sc->partial_bytes, flags, kSkFlagCount,
                      nullptr, &g, static_cast<cudaStream_t>(stream_v)) != 0)
        return -1;
    }
    return 0;
  }
  return umma_group_gemm_run(p, d->weight_bits, zmode, sc->sm_count, d->indptr, d->indptr_has_prev ? 1 : 0,
                             (int)d->num_experts, w_expert_bytes,
                             packed ? d->scale_stride_e : 0, static_cast<cudaStream_t>(stream_v));
}

int rb200_dequantize(const rb200_gemm_desc* d, void* wq_out, void* stream_v) {
  if (validate_common(d) != 0) return -1;
  RB200_CHECK(wq_out != nullptr, "wq_out must be non-NULL");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int group = (d->group_size <= 0 || d->group_size >= d->k) ? (int)d->k : (int)d->group_size;
  const int zmode = zero_mode(d);
  const int frag = d->weight_bits == 4 ? 64 : 32;
  int64_t tiles = (d->n / 16) * (d->k / frag);
  int64_t blocks = (tiles + 7) / 8;
  const int64_t max_blocks = (int64_t)sm_count_current() * 16;
  if (blocks > max_blocks) blocks = max_blocks;
  const uint8_t* w = static_cast<const uint8_t*>(d->w);
  const __half* s = static_cast<const __half*>(d->scales);
  const __half* z = static_cast<const __half*>(d->zeros);
  __half* o = static_cast<__half*>(wq_out);
#define RB200_DQ(BITS, ZM)                                                                       \
  dequantize_kernel<BITS, ZM><<<(int)blocks, 256, 0, stream>>>(w, s, z, d->scale_stride_n,       \
                                                               d->scale_stride_g, group,          \
                                                               d->zero_const, d->n, d->k, o)
  if (d->weight_bits == 4 && zmode == kZeroConstInt) RB200_DQ(4, kZeroConstInt);
  if (d->weight_bits == 4 && zmode == kZeroGeneral) RB200_DQ(4, kZeroGeneral);
  if (d->weight_bits == 8 && zmode == kZeroConstInt) RB200_DQ(8, kZeroConstInt);
  if (d->weight_bits == 8 && zmode == kZeroGeneral) RB200_DQ(8, kZeroGeneral);
#undef RB200_DQ
  RB200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
