/*
 * relax_b200 - PackedFunc-style calling convention over DLPack tensors.
 *
 * Mirrors the part of the reference runtime's C API that its generated operators and contrib
 * functions are reached through, so a host runtime that speaks that ABI can bind this library's
 * operators by global name:
 *   value union / type codes   include/tvm/runtime/c_runtime_api.h:174-215
 *   packed C function type     include/tvm/runtime/c_backend_api.h:49-51 (TVMBackendPackedCFunc)
 *   global registry            c_runtime_api.h:385-386 (TVMFuncCall), :467 (TVMFuncRegisterGlobal),
 *                              :478 (TVMFuncGetGlobal), :486 (TVMFuncListGlobalNames)
 *   errors                     c_runtime_api.h:245 (TVMAPISetLastError) - here rb200_last_error()
 * Tensors are DLTensor* (DLPack ABI).  Operators are destination-passing: the caller allocates
 * the output and passes it last (src/relax/transform/run_codegen.cc:106-113).
 */
#ifndef RELAX_B200_PACKED_H_
#define RELAX_B200_PACKED_H_

#include "relax_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- DLPack ABI (declared here only when no dlpack.h was included first) ---- */
#if !defined(DLPACK_DLPACK_H_) && !defined(DLPACK_VERSION) && !defined(DLPACK_MAJOR_VERSION)
#define RB200_OWN_DLPACK 1
typedef enum { kDLCPU = 1, kDLCUDA = 2, kDLCUDAHost = 3, kDLCUDAManaged = 13 } DLDeviceType;
typedef struct {
  DLDeviceType device_type;
  int32_t device_id;
} DLDevice;
typedef enum { kDLInt = 0U, kDLUInt = 1U, kDLFloat = 2U, kDLOpaqueHandle = 3U, kDLBfloat = 4U, kDLBool = 6U } DLDataTypeCode;
typedef struct {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
} DLDataType;
typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides; /* NULL = compact row-major */
  uint64_t byte_offset;
} DLTensor;
typedef struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(struct DLManagedTensor* self);
} DLManagedTensor;
#endif

/* ---- argument passing (c_runtime_api.h:174-215) ---- */
#define RB200_ARG_INT 0U          /* kTVMArgInt (also bool) */
#define RB200_ARG_FLOAT 2U        /* kTVMArgFloat */
#define RB200_ARG_HANDLE 3U       /* kTVMOpaqueHandle */
#define RB200_ARG_NULL 4U         /* kTVMNullptr */
#define RB200_ARG_DLTENSOR 7U     /* kTVMDLTensorHandle */
#define RB200_ARG_STR 11U         /* kTVMStr */
#define RB200_ARG_NDARRAY 13U     /* kTVMNDArrayHandle: accepted, read as DLTensor* (the handle's first member) */

typedef union {
  int64_t v_int64;
  double v_float64;
  void* v_handle;
  const char* v_str;
  DLDataType v_type;
  DLDevice v_device;
} RB200Value; /* layout-identical to TVMValue */

typedef int (*RB200PackedCFunc)(RB200Value* args, int* type_codes, int num_args,
                                RB200Value* out_ret_value, int* out_ret_tcode,
                                void* resource_handle);
typedef void* RB200FunctionHandle;

RB200_API int RB200FuncGetGlobal(const char* name, RB200FunctionHandle* out);
RB200_API int RB200FuncCall(RB200FunctionHandle func, RB200Value* arg_values, int* type_codes,
                            int num_args, RB200Value* ret_val, int* ret_type_code);
RB200_API int RB200FuncRegisterGlobal(const char* name, RB200PackedCFunc f, void* resource_handle,
                                      int override);
RB200_API int RB200FuncListGlobalNames(int* out_size, const char*** out_array);

/*
 * Global functions registered by the library (all launch on rb200_get_stream()):
 *
 *  "cutlass.ft_preprocess_weight"(packed_weight, sm:int, is_int4:bool[, out])
 *      src/runtime/contrib/cutlass/weight_preprocess.cc:38-58.  With the reference's own three
 *      arguments the result is allocated on the input's device (cudaMalloc / malloc) and
 *      returned as a DLManagedTensor* with type code RB200_ARG_HANDLE: the caller owns it and
 *      releases it by calling its deleter (the reference returns its runtime's NDArray object,
 *      which only that runtime can create; a bridge adopts the managed tensor with
 *      NDArray::FromDLPack, no copy).  With a fourth argument `out` (same shape / dtype /
 *      device) nothing is allocated and nothing is returned.  `sm` is accepted (70..120) and
 *      ignored: one layout.  2-D [K, N(/2)] or 3-D [E, K, N(/2)] int8; CUDA tensors, or CPU
 *      tensors (staged through the device - there is no host implementation).
 *  "relax_b200.preprocess_weight_q4f16"(packed_weight uint32 [N, K/8] or [E, N, K/8], out)
 *      the same step for the q4f16_1 layout of tests/python/dlight/test_gpu_gemv.py:189-206
 *      (no counterpart entry in the reference: it reaches that layout through generated TIR).
 *  "cutlass.ft_gemm_fp16_int4" / "cutlass.ft_gemm_fp16_int8"
 *      (x, w_pre, scales, bias|null, residual|null, activation:str, binary_op:str, unary_op:str,
 *       m:int, n:int, k:int, group_size:int, bias_stride:int, out)
 *      the argument list of fastertransformer::gemm_fp16_int_bias_act[_residual] as emitted by
 *      python/tvm/contrib/cutlass/gemm_operation.py:441-458, tensors first, `out` last.
 *  "relax_b200.gemm_fp16_q4f16"
 *      (x, w_pre, scales [N, K/g], zeros [N, K/g]|null, bias|null, residual|null, activation:str,
 *       binary_op:str, unary_op:str, group_size:int, zero_const:float, out)
 *      the decode + matmul of test_gpu_gemv.py:193-206 with fp32 accumulation.
 *  "relax_b200.dequantize"(w_pre, scales, zeros|null, layout:int, weight_bits:int, group_size:int,
 *       zero_const:float, out fp16 [N, K])        verification aid.
 *  "relax_b200.preprocess_weight_gate_up"(packed_weight, layout:int, is_int4:int, out)   repack with the
 *      gate/up row interleave; "relax_b200.interleave_gate_up"(f16 tensor, n_axis:int, out) permutes
 *      scales / zeros alike; activation "swiglu" of the matmul entries then writes silu(gate) * up.
 *  "relax_b200.preprocess_weight_autogptq"(qweight u32 [K/8, N], out[, perm i32 [K]])   AutoGPTQ source
 *      layout; with perm, source row perm[j] lands at position j of the reduction axis (act-order)
 *  "relax_b200.gptq_act_order"(g_idx i32 [K], groups:int, perm_out i32 [K])   the k rows group by group
 *      (tests/python/dlight/test_gpu_gemv.py:646-648 indexes scales and zeros through g_idx)
 *  "relax_b200.gather_columns"(x f16 [.., K], perm i32 [K], out f16 like x)   out[.., j] = x[.., perm[j]]
 *  "relax_b200.unpack_zeros_autogptq"(qzeros u32 [G, N/8], out f16 [G, N])   f16(zq) + 1
 *  "relax_b200.gemm_fp16_autogptq"(x, w_pre, scales f16 [G, N], zeros f16 [G, N], bias|null, out)
 *      the decode + matmul + add of tests/python/dlight/test_gpu_gemv.py:639-661, fp32 accumulation.
 *  "cutlass.group_gemm_fp16_sm90"(x f16 [M, K], weight f16 [E, N, K], indptr i64 [E] (device, end
 *       rows), workspace u8 [..]|null, out f16 [M, N])
 *      name and argument list of src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64.
 *  "cutlass.moe_gemm"(x, w_pre i8 [E, K, N/2] | [E, K, N], scales f16 [E, K/g, N] | [E, N],
 *       zeros|null, indptr i64 [E], workspace|null, out[, indptr_has_prev:int])
 *      the same grouping over FT-layout quantised experts (no counterpart in the reference).
 *      indptr_has_prev = 1: indptr is a view into a longer table whose element before the view is
 *      the first row of expert 0 - how a rank that holds experts [e0, e1) of a sharded layer calls.
 *  "relax_b200.moe_gemm_q4f16"(x, w_pre [E, N, K/8] words, scales f16 [E, N, K/g], zeros|null,
 *       indptr i64 [E], group_size:int, zero_const:float, out)
 *  "runtime.get_cuda_stream"() -> handle          src/runtime/cuda/cuda_device_api.cc:318-320
 *  "runtime.set_cuda_stream"(handle)
 */

#ifdef __cplusplus
}
#endif
#endif /* RELAX_B200_PACKED_H_ */
