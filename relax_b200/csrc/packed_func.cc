// PackedFunc-style registry and the operator shims registered in it.  Host C++ only: every
// shim unpacks DLTensor arguments, validates them, and calls the plain C ABI of relax_b200.h.
//
// Mirrors: global registry (src/runtime/registry.cc, include/tvm/runtime/c_runtime_api.h:385-486),
// the packed wrapper the reference's C-source codegen emits around each offloaded operator
// (src/relay/backend/contrib/codegen_c/codegen_c.h:100-131,163-235), and the contrib function
// src/runtime/contrib/cutlass/weight_preprocess.cc:38-58.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/relax_b200_packed.h"

namespace rb200 {
void set_last_error(const char* fmt, ...);
}

namespace {

struct Entry {
  RB200PackedCFunc fn;
  void* resource;
  std::string name;
};

std::mutex& reg_mutex() {
  static std::mutex m;
  return m;
}
std::map<std::string, Entry*>& registry() {
  static std::map<std::string, Entry*> r;
  return r;
}

#define PF_CHECK(cond, ...)               \
  do {                                    \
    if (!(cond)) {                        \
      rb200::set_last_error(__VA_ARGS__); \
      return -1;                          \
    }                                     \
  } while (0)

struct Args {
  RB200Value* v;
  int* tc;
  int n;
  const char* fname;

  bool is_null(int i) const { return tc[i] == (int)RB200_ARG_NULL || (is_tensor_code(i) && v[i].v_handle == nullptr); }
  bool is_tensor_code(int i) const {
    return tc[i] == (int)RB200_ARG_DLTENSOR || tc[i] == (int)RB200_ARG_NDARRAY;
  }
  int tensor(int i, const DLTensor** out, bool optional = false) const {
    *out = nullptr;
    PF_CHECK(i < n, "%s: missing argument %d", fname, i);
    if (optional && is_null(i)) return 0;
    PF_CHECK(is_tensor_code(i) && v[i].v_handle, "%s: argument %d must be a tensor (type code %d)",
             fname, i, tc[i]);
    *out = static_cast<const DLTensor*>(v[i].v_handle);
    return 0;
  }
  int integer(int i, int64_t* out) const {
    PF_CHECK(i < n && tc[i] == (int)RB200_ARG_INT, "%s: argument %d must be an int", fname, i);
    *out = v[i].v_int64;
    return 0;
  }
  int real(int i, double* out) const {
    PF_CHECK(i < n && (tc[i] == (int)RB200_ARG_FLOAT || tc[i] == (int)RB200_ARG_INT),
             "%s: argument %d must be a number", fname, i);
    *out = tc[i] == (int)RB200_ARG_FLOAT ? v[i].v_float64 : (double)v[i].v_int64;
    return 0;
  }
  int str(int i, const char** out) const {
    PF_CHECK(i < n && (tc[i] == (int)RB200_ARG_STR || tc[i] == (int)RB200_ARG_NULL),
             "%s: argument %d must be a string", fname, i);
    *out = tc[i] == (int)RB200_ARG_STR ? v[i].v_str : "";
    return 0;
  }
};

bool compact(const DLTensor* t) {
  if (!t->strides) return true;
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->strides[i] != expect) return false;
    expect *= t->shape[i];
  }
  return true;
}
void* data_of(const DLTensor* t) { return static_cast<char*>(t->data) + t->byte_offset; }
int64_t numel(const DLTensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->shape[i];
  return n;
}
bool is_dtype(const DLTensor* t, int code, int bits) {
  return t->dtype.code == code && t->dtype.bits == bits && t->dtype.lanes == 1;
}

int check_tensor(const char* fn, const char* what, const DLTensor* t, int code, int bits,
                 bool need_cuda = true) {
  PF_CHECK(is_dtype(t, code, bits), "%s: %s has dtype (code %d, bits %d), expected (code %d, bits %d)",
           fn, what, t->dtype.code, t->dtype.bits, code, bits);
  PF_CHECK(compact(t), "%s: %s must be compact row-major", fn, what);
  if (need_cuda) {
    PF_CHECK(t->device.device_type == kDLCUDA, "%s: %s must live on a CUDA device (device type %d)",
             fn, what, (int)t->device.device_type);
    int dev = -1;
    cudaGetDevice(&dev);
    PF_CHECK(dev == t->device.device_id, "%s: %s is on cuda:%d but the current device is cuda:%d", fn,
             what, t->device.device_id, dev);
  }
  return 0;
}
bool is_f16(const DLTensor* t) { return is_dtype(t, kDLFloat, 16); }

// ------------------------------------------------------------------ preprocess
int preprocess_common(const char* fn, const DLTensor* w, const DLTensor* out, bool is_int4,
                      int layout) {
  PF_CHECK(w->ndim == 2 || w->ndim == 3, "%s: weight must be 2-D or 3-D, got %d-D", fn, w->ndim);
  PF_CHECK(out->ndim == w->ndim, "%s: out rank differs from input", fn);
  for (int i = 0; i < w->ndim; ++i)
    PF_CHECK(out->shape[i] == w->shape[i], "%s: out shape differs from input at dim %d", fn, i);
  PF_CHECK(out->dtype.code == w->dtype.code && out->dtype.bits == w->dtype.bits,
           "%s: out dtype differs from input", fn);
  PF_CHECK(compact(w) && compact(out), "%s: tensors must be compact", fn);
  PF_CHECK(w->device.device_type == out->device.device_type &&
               w->device.device_id == out->device.device_id,
           "%s: out must be on the input's device", fn);
  const bool is_2d = w->ndim == 2;
  const int64_t experts = is_2d ? 1 : w->shape[0];
  const int64_t rows = w->shape[is_2d ? 0 : 1];
  const int64_t cols = w->shape[is_2d ? 1 : 2];
  const int64_t elem_bytes = w->dtype.bits / 8;
  int64_t k, n;
  const int base_layout = layout & 0xff;  // without the gate/up interleave flag
  if (base_layout == RB200_LAYOUT_FT_KN) {
    PF_CHECK(w->dtype.bits == 8 && (w->dtype.code == kDLInt || w->dtype.code == kDLUInt),
             "%s: FT weights must be int8", fn);
    k = rows;
    n = cols * (is_int4 ? 2 : 1);
  } else if (base_layout == RB200_LAYOUT_AUTOGPTQ_KN) {
    PF_CHECK(is_dtype(w, kDLUInt, 32) || is_dtype(w, kDLInt, 32), "%s: AutoGPTQ weights must be uint32 [K/8, N]", fn);
    k = rows * 8;
    n = cols;
  } else {
    PF_CHECK(is_dtype(w, kDLUInt, 32) || is_dtype(w, kDLInt, 32), "%s: q4f16 weights must be uint32", fn);
    n = rows;
    k = cols * 8;
  }
  const size_t bytes = (size_t)(experts * rows * cols * elem_bytes);
  cudaStream_t stream = static_cast<cudaStream_t>(rb200_get_stream());
  if (w->device.device_type == kDLCUDA) {
    return rb200_preprocess_weight(data_of(w), data_of(out), experts, k, n, is_int4 ? 1 : 0, layout,
                                   stream);
  }
  PF_CHECK(w->device.device_type == kDLCPU || w->device.device_type == kDLCUDAHost,
           "%s: unsupported device type %d", fn, (int)w->device.device_type);
  // Host tensors: the repack itself always runs on the GPU; stage through device memory.
  void* d_in = nullptr;
  void* d_out = nullptr;
  cudaError_t e = cudaMalloc(&d_in, bytes);
  if (e == cudaSuccess) e = cudaMalloc(&d_out, bytes);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_in, data_of(w), bytes, cudaMemcpyHostToDevice, stream);
  int rc = -1;
  if (e == cudaSuccess) {
    rc = rb200_preprocess_weight(d_in, d_out, experts, k, n, is_int4 ? 1 : 0, layout, stream);
    if (rc == 0) {
      e = cudaMemcpyAsync(data_of(out), d_out, bytes, cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
  }
  if (d_in) cudaFree(d_in);
  if (d_out) cudaFree(d_out);
  if (e != cudaSuccess) {
    rb200::set_last_error("%s: staging a host tensor through the device failed: %s", fn,
                          cudaGetErrorString(e));
    return -1;
  }
  return rc;
}

// A tensor this library allocated for a caller: DLPack's managed form, freed through its deleter.
struct OwnedTensor {
  DLManagedTensor mt;
  int64_t shape[8];
};
void owned_tensor_deleter(DLManagedTensor* self) {
  if (!self) return;
  OwnedTensor* o = static_cast<OwnedTensor*>(self->manager_ctx);
  if (o->mt.dl_tensor.device.device_type == kDLCUDA) cudaFree(o->mt.dl_tensor.data);
  else free(o->mt.dl_tensor.data);
  delete o;
}
// New compact tensor with the shape, dtype and device of `like` (CUDA: cudaMalloc on that device,
// which must be current; CPU: malloc).
int alloc_like(const char* fn, const DLTensor* like, OwnedTensor** out) {
  PF_CHECK(like->ndim >= 1 && like->ndim <= 8, "%s: rank %d not supported", fn, like->ndim);
  OwnedTensor* o = new OwnedTensor();
  memset(&o->mt, 0, sizeof(o->mt));
  size_t bytes = (size_t)((like->dtype.bits * like->dtype.lanes + 7) / 8);
  for (int i = 0; i < like->ndim; ++i) {
    o->shape[i] = like->shape[i];
    bytes *= (size_t)like->shape[i];
  }
  void* data = nullptr;
  if (like->device.device_type == kDLCUDA) {
    cudaError_t e = cudaMalloc(&data, bytes ? bytes : 1);
    if (e != cudaSuccess) {
      delete o;
      rb200::set_last_error("%s: cudaMalloc(%zu) for the result failed: %s", fn, bytes, cudaGetErrorString(e));
      return -1;
    }
  } else {
    data = malloc(bytes ? bytes : 1);
    if (!data) {
      delete o;
      rb200::set_last_error("%s: malloc(%zu) for the result failed", fn, bytes);
      return -1;
    }
  }
  o->mt.dl_tensor.data = data;
  o->mt.dl_tensor.device = like->device;
  o->mt.dl_tensor.ndim = like->ndim;
  o->mt.dl_tensor.dtype = like->dtype;
  o->mt.dl_tensor.shape = o->shape;
  o->mt.dl_tensor.strides = nullptr;
  o->mt.dl_tensor.byte_offset = 0;
  o->mt.manager_ctx = o;
  o->mt.deleter = owned_tensor_deleter;
  *out = o;
  return 0;
}

// Two calling forms.  (packed_weight, sm, is_int4): the reference's own argument list
// (src/runtime/contrib/cutlass/weight_preprocess.cc:38-39); the result is allocated here on the
// input's device and returned as a DLManagedTensor* (type code: opaque handle) that the caller
// releases through its deleter - a standalone library cannot mint the reference runtime's NDArray
// object, DLPack's managed tensor is the form every such runtime can adopt without a copy.
// (packed_weight, sm, is_int4, out): destination-passing, nothing allocated, nothing returned.
int pf_ft_preprocess_weight(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "cutlass.ft_preprocess_weight"};
  const DLTensor *w, *out;
  int64_t sm, is_int4;
  PF_CHECK(n == 3 || n == 4, "%s expects (packed_weight, sm, is_int4[, out]), got %d arguments", a.fname, n);
  if (a.tensor(0, &w) || a.integer(1, &sm) || a.integer(2, &is_int4)) return -1;
  PF_CHECK(sm >= 70 && sm <= 120, "%s: implausible sm=%lld", a.fname, (long long)sm);
  if (n == 4) {
    if (a.tensor(3, &out)) return -1;
    if (ret_tc) *ret_tc = RB200_ARG_NULL;
    return preprocess_common(a.fname, w, out, is_int4 != 0, RB200_LAYOUT_FT_KN);
  }
  if (w->device.device_type == kDLCUDA) {
    int dev = -1;
    cudaGetDevice(&dev);
    PF_CHECK(dev == w->device.device_id, "%s: packed_weight is on cuda:%d but the current device is cuda:%d", a.fname,
             w->device.device_id, dev);
  }
  OwnedTensor* o = nullptr;
  if (alloc_like(a.fname, w, &o)) return -1;
  if (preprocess_common(a.fname, w, &o->mt.dl_tensor, is_int4 != 0, RB200_LAYOUT_FT_KN) != 0) {
    owned_tensor_deleter(&o->mt);
    return -1;
  }
  if (ret) ret->v_handle = &o->mt;
  if (ret_tc) *ret_tc = RB200_ARG_HANDLE;
  return 0;
}

int pf_preprocess_q4f16(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.preprocess_weight_q4f16"};
  const DLTensor *w, *out;
  PF_CHECK(n == 2, "%s expects (packed_weight, out), got %d arguments", a.fname, n);
  if (a.tensor(0, &w) || a.tensor(1, &out)) return -1;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return preprocess_common(a.fname, w, out, true, RB200_LAYOUT_Q4_NK);
}

int pf_preprocess_autogptq(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.preprocess_weight_autogptq"};
  const DLTensor *w, *out;
  PF_CHECK(n == 2 || n == 3, "%s expects (qweight, out[, perm]), got %d arguments", a.fname, n);
  if (a.tensor(0, &w) || a.tensor(1, &out)) return -1;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  if (n == 2 || a.is_null(2)) return preprocess_common(a.fname, w, out, true, RB200_LAYOUT_AUTOGPTQ_KN);
  // act-order: the reduction axis permuted through perm (from relax_b200.gptq_act_order)
  const DLTensor* perm;
  if (a.tensor(2, &perm)) return -1;
  PF_CHECK(w->ndim == 2 && (is_dtype(w, kDLUInt, 32) || is_dtype(w, kDLInt, 32)) && compact(w) &&
               w->device.device_type == kDLCUDA,
           "%s: with perm, qweight must be a compact uint32 [K/8, N] CUDA tensor", a.fname);
  PF_CHECK(out->ndim == 2 && out->shape[0] == w->shape[0] && out->shape[1] == w->shape[1] &&
               out->dtype.bits == 32 && compact(out) && out->device.device_type == kDLCUDA,
           "%s: out must match qweight", a.fname);
  if (check_tensor(a.fname, "perm", perm, kDLInt, 32)) return -1;
  PF_CHECK(perm->ndim == 1 && perm->shape[0] == w->shape[0] * 8, "%s: perm must be int32 [K]", a.fname);
  return rb200_preprocess_weight_autogptq_perm(data_of(w), data_of(out), w->shape[0] * 8, w->shape[1],
                                               static_cast<const int32_t*>(data_of(perm)), rb200_get_stream());
}
// (g_idx i32 [K], groups:int, perm_out i32 [K])
int pf_gptq_act_order(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.gptq_act_order"};
  const DLTensor *g_idx, *perm;
  int64_t groups = 0;
  PF_CHECK(n == 3, "%s expects (g_idx, groups, perm_out), got %d arguments", a.fname, n);
  if (a.tensor(0, &g_idx) || a.integer(1, &groups) || a.tensor(2, &perm)) return -1;
  if (check_tensor(a.fname, "g_idx", g_idx, kDLInt, 32) || check_tensor(a.fname, "perm_out", perm, kDLInt, 32)) return -1;
  PF_CHECK(g_idx->ndim == 1 && perm->ndim == 1 && perm->shape[0] == g_idx->shape[0], "%s: g_idx and perm_out must be int32 [K]",
           a.fname);
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_gptq_act_order(static_cast<const int32_t*>(data_of(g_idx)), g_idx->shape[0], groups,
                              static_cast<int32_t*>(data_of(perm)), rb200_get_stream());
}
// (x f16 [..., K], perm i32 [K], out f16 like x): out[..., j] = x[..., perm[j]]
int pf_gather_columns(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.gather_columns"};
  const DLTensor *x, *perm, *out;
  PF_CHECK(n == 3, "%s expects (x, perm, out), got %d arguments", a.fname, n);
  if (a.tensor(0, &x) || a.tensor(1, &perm) || a.tensor(2, &out)) return -1;
  if (check_tensor(a.fname, "x", x, kDLFloat, 16) || check_tensor(a.fname, "perm", perm, kDLInt, 32) ||
      check_tensor(a.fname, "out", out, kDLFloat, 16))
    return -1;
  PF_CHECK(x->ndim >= 1 && perm->ndim == 1 && perm->shape[0] == x->shape[x->ndim - 1], "%s: perm must be int32 [K]", a.fname);
  PF_CHECK(out->ndim == x->ndim, "%s: out must have the shape of x", a.fname);
  int64_t m = 1;
  for (int i = 0; i < x->ndim; ++i) {
    PF_CHECK(out->shape[i] == x->shape[i], "%s: out must have the shape of x", a.fname);
    if (i + 1 < x->ndim) m *= x->shape[i];
  }
  const int64_t k = perm->shape[0];
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_gather_columns(data_of(x), static_cast<const int32_t*>(data_of(perm)), data_of(out), m, k, k, k,
                              rb200_get_stream());
}
// (qzeros u32 [G, N/8], out f16 [G, N])
int pf_unpack_zeros_autogptq(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.unpack_zeros_autogptq"};
  const DLTensor *zq, *out;
  PF_CHECK(n == 2, "%s expects (qzeros, out), got %d arguments", a.fname, n);
  if (a.tensor(0, &zq) || a.tensor(1, &out)) return -1;
  PF_CHECK(zq->ndim == 2 && (is_dtype(zq, kDLUInt, 32) || is_dtype(zq, kDLInt, 32)) && compact(zq) &&
               zq->device.device_type == kDLCUDA,
           "%s: qzeros must be a compact uint32 [G, N/8] CUDA tensor", a.fname);
  if (check_tensor(a.fname, "out", out, kDLFloat, 16)) return -1;
  PF_CHECK(out->ndim == 2 && out->shape[0] == zq->shape[0] && out->shape[1] == zq->shape[1] * 8,
           "%s: out must be fp16 [G, N]", a.fname);
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_unpack_zeros_autogptq(data_of(zq), data_of(out), zq->shape[0], out->shape[1], rb200_get_stream());
}

// (packed_weight, layout:int (RB200_LAYOUT_*), is_int4:int, out): repack with the gate/up row interleave
int pf_preprocess_gate_up(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.preprocess_weight_gate_up"};
  const DLTensor *w, *out;
  int64_t layout, is_int4;
  PF_CHECK(n == 4, "%s expects (packed_weight, layout, is_int4, out), got %d arguments", a.fname, n);
  if (a.tensor(0, &w) || a.integer(1, &layout) || a.integer(2, &is_int4) || a.tensor(3, &out)) return -1;
  PF_CHECK(layout == RB200_LAYOUT_FT_KN || layout == RB200_LAYOUT_Q4_NK, "%s: layout must be FT_KN or Q4_NK", a.fname);
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return preprocess_common(a.fname, w, out, is_int4 != 0, (int)layout | RB200_LAYOUT_GATE_UP_INTERLEAVE);
}
// (src f16, n_axis:int, out f16): the same row permutation for scales / zero points along axis n_axis
int pf_interleave_gate_up(RB200Value* v, int* tc, int n, RB200Value* ret, int* ret_tc, void*) {
  Args a{v, tc, n, "relax_b200.interleave_gate_up"};
  const DLTensor *src, *out;
  int64_t axis;
  PF_CHECK(n == 3, "%s expects (tensor, n_axis, out), got %d arguments", a.fname, n);
  if (a.tensor(0, &src) || a.integer(1, &axis) || a.tensor(2, &out)) return -1;
  if (check_tensor(a.fname, "tensor", src, kDLFloat, 16) || check_tensor(a.fname, "out", out, kDLFloat, 16)) return -1;
  PF_CHECK(axis >= 0 && axis < src->ndim && numel(src) == numel(out), "%s: bad axis or out size", a.fname);
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < axis; ++i) outer *= src->shape[i];
  for (int i = (int)axis + 1; i < src->ndim; ++i) inner *= src->shape[i];
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_interleave_gate_up(data_of(src), data_of(out), outer, src->shape[axis], inner, rb200_get_stream());
}

// ------------------------------------------------------------------ GEMM shims
int parse_names(const char* fn, const char* act, const char* bin, const char* un, rb200_gemm_desc* d) {
  struct {
    const char* s;
    int v;
  } acts[] = {{"", 0}, {"identity", 0}, {"relu", 1}, {"silu", 2}, {"gelu", 3}, {"swiglu", 4}},
    bins[] = {{"", 0}, {"none", 0}, {"plus", 1}, {"multiply", 2}},
    uns[] = {{"", 0}, {"identity", 0}, {"relu", 1}};
  bool ok = false;
  for (auto& e : acts)
    if (!strcmp(act, e.s)) d->activation = e.v, ok = true;
  PF_CHECK(ok, "%s: unknown activation '%s'", fn, act);
  ok = false;
  for (auto& e : bins)
    if (!strcmp(bin, e.s)) d->binary_op = e.v, ok = true;
  PF_CHECK(ok, "%s: unknown binary_op '%s'", fn, bin);
  ok = false;
  for (auto& e : uns)
    if (!strcmp(un, e.s)) d->unary_op = e.v, ok = true;
  PF_CHECK(ok, "%s: unknown unary_op '%s'", fn, un);
  return 0;
}

int64_t lead_rows(const DLTensor* t) {  // product of all dims but the last
  int64_t m = 1;
  for (int i = 0; i + 1 < t->ndim; ++i) m *= t->shape[i];
  return m;
}

// (x, w_pre, scales, bias|null, residual|null, activation, binary_op, unary_op, m, n, k,
//  group_size, bias_stride, out)
int ft_gemm(const char* fname, int bits, RB200Value* v, int* tc, int n_args, int* ret_tc) {
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 14, "%s expects 14 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *s, *bias, *res, *out;
  const char *act, *bin, *un;
  int64_t m, n, k, group, bias_stride;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &s) || a.tensor(3, &bias, true) ||
      a.tensor(4, &res, true) || a.str(5, &act) || a.str(6, &bin) || a.str(7, &un) ||
      a.integer(8, &m) || a.integer(9, &n) || a.integer(10, &k) || a.integer(11, &group) ||
      a.integer(12, &bias_stride) || a.tensor(13, &out))
    return -1;
  if (check_tensor(fname, "x", x, kDLFloat, 16) || check_tensor(fname, "scales", s, kDLFloat, 16) ||
      check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  PF_CHECK(w->dtype.bits == 8 && compact(w) && w->device.device_type == kDLCUDA,
           "%s: weight must be a compact int8 CUDA tensor", fname);
  PF_CHECK(w->ndim == 2 && w->shape[0] == k && w->shape[1] * (bits == 4 ? 2 : 1) == n,
           "%s: weight shape [%lld, %lld] does not match k=%lld, n=%lld", fname,
           (long long)w->shape[0], (long long)(w->ndim > 1 ? w->shape[1] : 0), (long long)k, (long long)n);
  PF_CHECK(x->ndim >= 1 && x->shape[x->ndim - 1] == k && lead_rows(x) == m,
           "%s: x shape does not match m=%lld, k=%lld", fname, (long long)m, (long long)k);
  const int64_t n_out = !strcmp(act, "swiglu") ? n / 2 : n;  // the fused gate/up form halves the width
  PF_CHECK(numel(out) == m * n_out, "%s: out has %lld elements, expected %lld", fname, (long long)numel(out),
           (long long)(m * n_out));
  const bool per_col = group <= 0 || group >= k;
  // the shapes the reference's pattern check admits (python/tvm/relax/backend/contrib/cutlass.py:255-257):
  // (N,), (1, N) or (K / group_size, N)
  PF_CHECK(s->ndim >= 1 && s->ndim <= 2 && s->shape[s->ndim - 1] == n,
           "%s: scales must be [n], [1, n] or [k / group_size, n]", fname);
  PF_CHECK(s->ndim == 1 || s->shape[0] == (per_col ? 1 : k / group),
           "%s: scales have %lld rows, expected %lld", fname, (long long)s->shape[0],
           (long long)(per_col ? 1 : k / group));
  const char* a_name = act;
  rb200_gemm_desc d;
  memset(&d, 0, sizeof(d));
  if (parse_names(fname, a_name, bin, un, &d)) return -1;
  if (bias) {
    if (check_tensor(fname, "bias", bias, kDLFloat, 16)) return -1;
    PF_CHECK(numel(bias) == (bias_stride == 0 ? n : m * n), "%s: bias size does not match bias_stride",
             fname);
  }
  if (res) {
    if (check_tensor(fname, "residual", res, kDLFloat, 16)) return -1;
    PF_CHECK(numel(res) == m * n, "%s: residual must have m*n elements", fname);
  }
  void* stream = rb200_get_stream();
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  if (res) {
    PF_CHECK(bias_stride == 0, "%s: the residual form takes a row-vector bias (bias_stride 0)", fname);
    return rb200_gemm_fp16_int_bias_act_residual(
        data_of(x), data_of(w), data_of(s), bias ? data_of(bias) : nullptr, data_of(res), data_of(out),
        act, bin[0] ? bin : "plus", un, (int)m, (int)n, (int)k, (int)group, bits, nullptr, 0, stream);
  }
  return rb200_gemm_fp16_int_bias_act(data_of(x), data_of(w), data_of(s),
                                      bias ? data_of(bias) : nullptr, data_of(out), act, (int)m, (int)n,
                                      (int)k, (int)group, (int)bias_stride, bits, nullptr, 0, stream);
}
int pf_ft_gemm_int4(RB200Value* v, int* tc, int n, RB200Value*, int* ret_tc, void*) {
  return ft_gemm("cutlass.ft_gemm_fp16_int4", 4, v, tc, n, ret_tc);
}
int pf_ft_gemm_int8(RB200Value* v, int* tc, int n, RB200Value*, int* ret_tc, void*) {
  return ft_gemm("cutlass.ft_gemm_fp16_int8", 8, v, tc, n, ret_tc);
}

// (x, w_pre, scales, zeros|null, bias|null, residual|null, activation, binary_op, unary_op,
//  group_size, zero_const, out)
int pf_gemm_q4f16(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "relax_b200.gemm_fp16_q4f16";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 12, "%s expects 12 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *s, *z, *bias, *res, *out;
  const char *act, *bin, *un;
  int64_t group;
  double zconst;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &s) || a.tensor(3, &z, true) ||
      a.tensor(4, &bias, true) || a.tensor(5, &res, true) || a.str(6, &act) || a.str(7, &bin) ||
      a.str(8, &un) || a.integer(9, &group) || a.real(10, &zconst) || a.tensor(11, &out))
    return -1;
  if (check_tensor(fname, "x", x, kDLFloat, 16) || check_tensor(fname, "scales", s, kDLFloat, 16) ||
      check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  PF_CHECK(w->ndim == 2 && w->dtype.bits == 32 && compact(w) && w->device.device_type == kDLCUDA,
           "%s: weight must be a compact uint32 [N, K/8] CUDA tensor", fname);
  const int64_t n = w->shape[0], k = w->shape[1] * 8;
  PF_CHECK(x->ndim >= 1 && x->shape[x->ndim - 1] == k, "%s: x inner extent %lld != k=%lld", fname,
           (long long)x->shape[x->ndim - 1], (long long)k);
  const int64_t m = lead_rows(x);
  const int64_t n_out = !strcmp(act, "swiglu") ? n / 2 : n;  // the fused gate/up form halves the width
  PF_CHECK(numel(out) == m * n_out, "%s: out has %lld elements, expected %lld", fname,
           (long long)numel(out), (long long)(m * n_out));
  PF_CHECK(group > 0 && k % group == 0, "%s: group_size=%lld must divide k=%lld", fname,
           (long long)group, (long long)k);
  PF_CHECK(numel(s) == n * (k / group), "%s: scales must be [N, K/group]", fname);
  rb200_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  if (parse_names(fname, act, bin, un, &d)) return -1;
  d.weight_bits = 4;
  d.x = data_of(x);
  d.w = data_of(w);
  d.scales = data_of(s);
  if (z) {
    if (check_tensor(fname, "zeros", z, kDLFloat, 16)) return -1;
    PF_CHECK(numel(z) == numel(s), "%s: zeros must have the shape of scales", fname);
    d.zeros = data_of(z);
  }
  if (bias) {
    if (check_tensor(fname, "bias", bias, kDLFloat, 16)) return -1;
    PF_CHECK(numel(bias) == n || numel(bias) == m * n, "%s: bias must be [n] or [m, n]", fname);
    d.bias = data_of(bias);
    d.bias_stride = (numel(bias) == n) ? 0 : n;
  }
  if (res) {
    if (check_tensor(fname, "residual", res, kDLFloat, 16)) return -1;
    PF_CHECK(numel(res) == m * n, "%s: residual must have m*n elements", fname);
    d.residual = data_of(res);
    if (d.binary_op == RB200_BIN_NONE) d.binary_op = RB200_BIN_PLUS;
  }
  d.out = data_of(out);
  d.m = m;
  d.n = n;
  d.k = k;
  d.ldx = k;
  d.ldo = n_out;
  d.group_size = group;
  d.scale_stride_n = k / group;
  d.scale_stride_g = 1;
  d.zero_const = (float)zconst;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_gemm_fp16_intx(&d, rb200_get_stream());
}

// (w_pre, scales, zeros|null, layout, weight_bits, group_size, zero_const, out fp16 [N, K])
// AutoGPTQ form (tests/python/dlight/test_gpu_gemv.py:639-661):
// (x, w_pre u32 [K/8, N], scales f16 [G, N], zeros f16 [G, N] (from unpack_zeros_autogptq), bias|null, out)
// out = bias + x @ ((q - zeros) * scales), groups in order along k (group size K / G).
int pf_gemm_autogptq(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "relax_b200.gemm_fp16_autogptq";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 6, "%s expects 6 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *s, *z, *bias, *out;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &s) || a.tensor(3, &z) || a.tensor(4, &bias, true) ||
      a.tensor(5, &out))
    return -1;
  if (check_tensor(fname, "x", x, kDLFloat, 16) || check_tensor(fname, "scales", s, kDLFloat, 16) ||
      check_tensor(fname, "zeros", z, kDLFloat, 16) || check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  PF_CHECK(w->ndim == 2 && w->dtype.bits == 32 && compact(w) && w->device.device_type == kDLCUDA,
           "%s: weight must be a compact uint32 [K/8, N] CUDA tensor", fname);
  const int64_t k = w->shape[0] * 8, n = w->shape[1];
  PF_CHECK(x->ndim >= 1 && x->shape[x->ndim - 1] == k, "%s: x inner extent != k=%lld", fname, (long long)k);
  const int64_t m = lead_rows(x);
  PF_CHECK(numel(out) == m * n, "%s: out has %lld elements, expected %lld", fname, (long long)numel(out),
           (long long)(m * n));
  PF_CHECK(s->ndim == 2 && s->shape[1] == n && s->shape[0] >= 1 && k % s->shape[0] == 0,
           "%s: scales must be [G, N] with G dividing k", fname);
  PF_CHECK(numel(z) == numel(s), "%s: zeros must have the shape of scales", fname);
  rb200_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  d.weight_bits = 4;
  d.x = data_of(x);
  d.w = data_of(w);
  d.scales = data_of(s);
  d.zeros = data_of(z);
  if (bias) {
    if (check_tensor(fname, "bias", bias, kDLFloat, 16)) return -1;
    PF_CHECK(numel(bias) == n || numel(bias) == m * n, "%s: bias must be [n] or [m, n]", fname);
    d.bias = data_of(bias);
    d.bias_stride = (numel(bias) == n) ? 0 : n;
  }
  d.out = data_of(out);
  d.m = m;
  d.n = n;
  d.k = k;
  d.ldx = k;
  d.ldo = n;
  d.group_size = k / s->shape[0];
  d.scale_stride_n = 1;
  d.scale_stride_g = n;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_gemm_fp16_intx(&d, rb200_get_stream());
}

// ------------------------------------------------------------------ grouped GEMM
// cutlass.group_gemm_fp16_sm90(x [M,K] f16, weight [E,N,K] f16, indptr [E] i64, workspace [..] u8, out [M,N] f16):
// the argument list of tvm_cutlass_group_gemm_sm90 (src/runtime/contrib/cutlass/fp16_group_gemm.cu:41-62).
int pf_group_gemm_fp16(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "cutlass.group_gemm_fp16_sm90";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 5, "%s expects 5 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *indptr, *ws, *out;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &indptr) || a.tensor(3, &ws, true) || a.tensor(4, &out))
    return -1;
  PF_CHECK(x->ndim == 2 && w->ndim == 3 && indptr->ndim == 1 && out->ndim == 2,
           "%s: expected x 2-D, weight 3-D, indptr 1-D, out 2-D", fname);
  if (check_tensor(fname, "x", x, kDLFloat, 16) || check_tensor(fname, "weight", w, kDLFloat, 16) ||
      check_tensor(fname, "indptr", indptr, kDLInt, 64) || check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  const int64_t E = w->shape[0], n = w->shape[1], k = w->shape[2];
  PF_CHECK(indptr->shape[0] == E, "%s: indptr has %lld entries for %lld groups", fname,
           (long long)indptr->shape[0], (long long)E);
  PF_CHECK(x->shape[1] == k && out->shape[0] == x->shape[0] && out->shape[1] == n,
           "%s: x / out shapes do not match weight [E, n, k]", fname);
  rb200_group_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  d.weight_bits = 16;
  d.x = data_of(x);
  d.w = data_of(w);
  d.indptr = static_cast<const int64_t*>(data_of(indptr));
  d.out = data_of(out);
  d.total_rows = x->shape[0];
  d.n = n;
  d.k = k;
  d.num_experts = E;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_group_gemm(&d, rb200_get_stream());
}

// Quantised experts.  layout 0 (cutlass.moe_gemm): FT form, w_pre int8 [E, K, N/2] (int4) or
// [E, K, N] (int8) as written by cutlass.ft_preprocess_weight, scales [E, K/g, N] or [E, N].
// layout 1 (relax_b200.moe_gemm_q4f16): w_pre [E, N, K/8] 32-bit words, scales [E, N, K/g].
int moe_gemm(const char* fname, int layout, const DLTensor* x, const DLTensor* w, const DLTensor* s,
             const DLTensor* z, const DLTensor* indptr, const DLTensor* out, int64_t group, double zero_const,
             int64_t indptr_has_prev = 0) {
  PF_CHECK(x->ndim == 2 && w->ndim == 3 && indptr->ndim == 1 && out->ndim == 2,
           "%s: expected x 2-D, weight 3-D, indptr 1-D, out 2-D", fname);
  if (check_tensor(fname, "x", x, kDLFloat, 16) || check_tensor(fname, "scales", s, kDLFloat, 16) ||
      check_tensor(fname, "indptr", indptr, kDLInt, 64) || check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  if (z && check_tensor(fname, "zeros", z, kDLFloat, 16)) return -1;
  PF_CHECK(compact(w) && w->device.device_type == kDLCUDA, "%s: weight must be a compact CUDA tensor", fname);
  const int64_t E = w->shape[0], k = x->shape[1], n = out->shape[1];
  rb200_group_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  if (layout == 0) {
    PF_CHECK(w->dtype.bits == 8 && w->shape[1] == k && (w->shape[2] == n || w->shape[2] * 2 == n),
             "%s: weight must be int8 [E, k, n/2] or [E, k, n]", fname);
    d.weight_bits = w->shape[2] == n ? 8 : 4;
    const int64_t per_e = numel(s) / E;
    PF_CHECK(numel(s) % E == 0 && per_e % n == 0 && per_e >= n, "%s: scales must be [E, k/g, n] or [E, n]", fname);
    const int64_t kg = per_e / n;
    d.group_size = kg == 1 ? -1 : k / kg;
    PF_CHECK(kg == 1 || (k % kg == 0), "%s: scale rows do not divide k", fname);
    d.scale_stride_n = 1;
    d.scale_stride_g = n;
    d.scale_stride_e = per_e;
    d.zero_const = d.weight_bits == 4 ? 8.0f : 128.0f;
  } else {
    PF_CHECK(w->dtype.bits == 32 && w->shape[1] == n && w->shape[2] * 8 == k,
             "%s: weight must be 32-bit words [E, n, k/8]", fname);
    PF_CHECK(group > 0 && k % group == 0, "%s: group_size must divide k", fname);
    d.weight_bits = 4;
    const int64_t kg = k / group;
    PF_CHECK(numel(s) == E * n * kg, "%s: scales must be [E, n, k/group_size]", fname);
    d.group_size = group;
    d.scale_stride_n = kg;
    d.scale_stride_g = 1;
    d.scale_stride_e = n * kg;
    d.zero_const = (float)zero_const;
  }
  PF_CHECK(!z || numel(z) == numel(s), "%s: zeros must have the shape of scales", fname);
  PF_CHECK(indptr->shape[0] == E && out->shape[0] == x->shape[0], "%s: indptr / out do not match x and weight", fname);
  d.x = data_of(x);
  d.w = data_of(w);
  d.scales = data_of(s);
  d.zeros = z ? data_of(z) : nullptr;
  d.indptr = static_cast<const int64_t*>(data_of(indptr));
  d.out = data_of(out);
  d.total_rows = x->shape[0];
  d.n = n;
  d.k = k;
  d.num_experts = E;
  d.indptr_has_prev = indptr_has_prev ? 1 : 0;
  return rb200_group_gemm(&d, rb200_get_stream());
}
// (x, w_pre, scales, zeros|null, indptr, workspace|null, out[, indptr_has_prev:int])
int pf_moe_gemm(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "cutlass.moe_gemm";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 7 || n_args == 8, "%s expects 7 or 8 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *s, *z, *indptr, *ws, *out;
  int64_t has_prev = 0;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &s) || a.tensor(3, &z, true) || a.tensor(4, &indptr) ||
      a.tensor(5, &ws, true) || a.tensor(6, &out))
    return -1;
  if (n_args == 8 && a.integer(7, &has_prev)) return -1;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return moe_gemm(fname, 0, x, w, s, z, indptr, out, 0, 0.0, has_prev);
}
// (x, w_pre, scales, zeros|null, indptr, group_size, zero_const, out)
int pf_moe_gemm_q4f16(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "relax_b200.moe_gemm_q4f16";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 8, "%s expects 8 arguments, got %d", fname, n_args);
  const DLTensor *x, *w, *s, *z, *indptr, *out;
  int64_t group;
  double zc;
  if (a.tensor(0, &x) || a.tensor(1, &w) || a.tensor(2, &s) || a.tensor(3, &z, true) || a.tensor(4, &indptr) ||
      a.integer(5, &group) || a.real(6, &zc) || a.tensor(7, &out))
    return -1;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return moe_gemm(fname, 1, x, w, s, z, indptr, out, group, zc);
}

int pf_dequantize(RB200Value* v, int* tc, int n_args, RB200Value*, int* ret_tc, void*) {
  const char* fname = "relax_b200.dequantize";
  Args a{v, tc, n_args, fname};
  PF_CHECK(n_args == 8, "%s expects 8 arguments, got %d", fname, n_args);
  const DLTensor *w, *s, *z, *out;
  int64_t layout, bits, group;
  double zconst;
  if (a.tensor(0, &w) || a.tensor(1, &s) || a.tensor(2, &z, true) || a.integer(3, &layout) ||
      a.integer(4, &bits) || a.integer(5, &group) || a.real(6, &zconst) || a.tensor(7, &out))
    return -1;
  if (check_tensor(fname, "scales", s, kDLFloat, 16) || check_tensor(fname, "out", out, kDLFloat, 16))
    return -1;
  PF_CHECK(out->ndim == 2, "%s: out must be [N, K]", fname);
  const int64_t n = out->shape[0], k = out->shape[1];
  PF_CHECK(numel(w) * (w->dtype.bits / 8) == n * k * bits / 8, "%s: weight bytes do not match [N, K]",
           fname);
  rb200_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.struct_size = sizeof(d);
  d.weight_bits = (int)bits;
  d.w = data_of(w);
  d.scales = data_of(s);
  d.zeros = z ? data_of(z) : nullptr;
  d.n = n;
  d.k = k;
  const bool per_col = group <= 0 || group >= k;
  d.group_size = per_col ? k : group;
  if (layout == RB200_LAYOUT_FT_KN) {
    d.scale_stride_n = 1;
    d.scale_stride_g = per_col ? 0 : n;
  } else {
    d.scale_stride_n = per_col ? 1 : k / group;
    d.scale_stride_g = per_col ? 0 : 1;
  }
  d.zero_const = (float)zconst;
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return rb200_dequantize(&d, data_of(out), rb200_get_stream());
}

int pf_get_stream(RB200Value*, int*, int, RB200Value* ret, int* ret_tc, void*) {
  if (ret) ret->v_handle = rb200_get_stream();
  if (ret_tc) *ret_tc = RB200_ARG_HANDLE;
  return 0;
}
int pf_set_stream(RB200Value* v, int* tc, int n, RB200Value*, int* ret_tc, void*) {
  PF_CHECK(n == 1 && (tc[0] == (int)RB200_ARG_HANDLE || tc[0] == (int)RB200_ARG_NULL ||
                      tc[0] == (int)RB200_ARG_INT),
           "runtime.set_cuda_stream expects one handle");
  rb200_set_stream(tc[0] == (int)RB200_ARG_NULL ? nullptr
                   : tc[0] == (int)RB200_ARG_INT ? reinterpret_cast<void*>(v[0].v_int64)
                                                 : v[0].v_handle);
  if (ret_tc) *ret_tc = RB200_ARG_NULL;
  return 0;
}

void register_builtin(const char* name, RB200PackedCFunc fn) {
  registry()[name] = new Entry{fn, nullptr, name};
}

void ensure_builtins() {
  static bool done = false;
  if (done) return;
  done = true;
  register_builtin("cutlass.ft_preprocess_weight", pf_ft_preprocess_weight);
  register_builtin("relax_b200.preprocess_weight_q4f16", pf_preprocess_q4f16);
  register_builtin("relax_b200.preprocess_weight_gate_up", pf_preprocess_gate_up);
  register_builtin("relax_b200.interleave_gate_up", pf_interleave_gate_up);
  register_builtin("relax_b200.preprocess_weight_autogptq", pf_preprocess_autogptq);
  register_builtin("relax_b200.unpack_zeros_autogptq", pf_unpack_zeros_autogptq);
  register_builtin("relax_b200.gptq_act_order", pf_gptq_act_order);
  register_builtin("relax_b200.gather_columns", pf_gather_columns);
  register_builtin("relax_b200.gemm_fp16_autogptq", pf_gemm_autogptq);
  register_builtin("cutlass.ft_gemm_fp16_int4", pf_ft_gemm_int4);
  register_builtin("cutlass.ft_gemm_fp16_int8", pf_ft_gemm_int8);
  register_builtin("relax_b200.gemm_fp16_q4f16", pf_gemm_q4f16);
  register_builtin("relax_b200.dequantize", pf_dequantize);
  register_builtin("cutlass.group_gemm_fp16_sm90", pf_group_gemm_fp16);
  register_builtin("cutlass.moe_gemm", pf_moe_gemm);
  register_builtin("relax_b200.moe_gemm_q4f16", pf_moe_gemm_q4f16);
  register_builtin("runtime.get_cuda_stream", pf_get_stream);
  register_builtin("runtime.set_cuda_stream", pf_set_stream);
}

}  // namespace

namespace rb200 {
// other translation units add their operators here (grouped GEMM, collectives)
void register_packed(const char* name, RB200PackedCFunc fn) {
  std::lock_guard<std::mutex> lock(reg_mutex());
  ensure_builtins();
  registry()[name] = new Entry{fn, nullptr, name};
}
}  // namespace rb200

extern "C" {

int RB200FuncGetGlobal(const char* name, RB200FunctionHandle* out) {
  std::lock_guard<std::mutex> lock(reg_mutex());
  ensure_builtins();
  PF_CHECK(name && out, "RB200FuncGetGlobal: NULL argument");
  auto it = registry().find(name);
  *out = it == registry().end() ? nullptr : it->second;  // NULL handle = not found, as TVMFuncGetGlobal
  return 0;
}

int RB200FuncCall(RB200FunctionHandle func, RB200Value* arg_values, int* type_codes, int num_args,
                  RB200Value* ret_val, int* ret_type_code) {
  PF_CHECK(func != nullptr, "RB200FuncCall: NULL function handle");
  Entry* e = static_cast<Entry*>(func);
  RB200Value dummy;
  int dummy_tc = RB200_ARG_NULL;
  return e->fn(arg_values, type_codes, num_args, ret_val ? ret_val : &dummy,
               ret_type_code ? ret_type_code : &dummy_tc, e->resource);
}

int RB200FuncRegisterGlobal(const char* name, RB200PackedCFunc f, void* resource_handle, int override) {
  std::lock_guard<std::mutex> lock(reg_mutex());
  ensure_builtins();
  PF_CHECK(name && f, "RB200FuncRegisterGlobal: NULL argument");
  auto it = registry().find(name);
  PF_CHECK(it == registry().end() || override, "global function '%s' is already registered", name);
  registry()[name] = new Entry{f, resource_handle, name};
  return 0;
}

int RB200FuncListGlobalNames(int* out_size, const char*** out_array) {
  std::lock_guard<std::mutex> lock(reg_mutex());
  ensure_builtins();
  static thread_local std::vector<const char*> names;
  names.clear();
  for (auto& kv : registry()) names.push_back(kv.second->name.c_str());
  *out_size = (int)names.size();
  *out_array = names.data();
  return 0;
}

}  // extern "C"
