/*
 * relax_b200 - C ABI of the B200 (sm_100a) weight-only dequantize-matmul library.
 *
 * Every entry point takes plain pointers and sizes, returns 0 on success and -1 on failure
 * (the message is then available from rb200_last_error(), thread local), never aborts the
 * process and never falls back to a CPU path.  Device pointers must belong to the CUDA
 * device that is current on the calling thread; `stream` is a cudaStream_t passed as void*.
 *
 * Each declaration names the interface of the reference project (mlc-ai/relax, paths inside
 * that project) that it stands in for.
 */
#ifndef RELAX_B200_H_
#define RELAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RB200_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ errors, streams */

/* Mirrors TVMGetLastError (include/tvm/runtime/c_runtime_api.h:245). */
RB200_API const char* rb200_last_error(void);

/*
 * The stream later PackedFunc-style calls on this thread launch on; stands in for the
 * "runtime.get_cuda_stream" lookup the generated host code performs
 * (python/tvm/contrib/cutlass/gemm_operation.py:432-434, src/runtime/cuda/cuda_device_api.cc:318-320)
 * and for TVMSetStream (c_runtime_api.h).  Plain C entry points take the stream explicitly.
 */
RB200_API int rb200_set_stream(void* stream);
RB200_API void* rb200_get_stream(void);

/*
 * Reads (and clears) the device-side status words that bounded waits inside the kernels set
 * when they give up: the one in the library's per-device scratch block and the one in the static
 * array of rb200_gemm_fp16_intx_noalloc.  Synchronises the given stream.  0 = no error recorded,
 * 1 = a wait ran out (the kernel skipped its remaining work and left outputs unwritten).
 * Allocates nothing: a status word that no call has created yet reads as 0.  After a non-zero
 * status the split-k flags and tickets of the scratch block are put back at rest.
 * Replaces nothing in the reference, whose kernels spin without a bound
 * (3rdparty/tensorrt_llm/custom_allreduce_kernels.cu:94-113) and whose collectives abort the
 * process on error (src/runtime/disco/nccl/nccl_context.h:50-56).
 */
RB200_API int rb200_check_async_error(void* stream, int* status_out);

/*
 * Upper bound, in milliseconds, of every wait on a flag that another CTA or another GPU writes
 * (split-k fix-up of the decode kernel, flag exchange of the all-reduce); 0 restores the default
 * of about two seconds.  Process-wide; read when a kernel is launched.  A host that detects a
 * missing peer by other means can set this short so that kernels already queued return quickly.
 */
RB200_API int rb200_set_wait_limit_ms(unsigned limit_ms);

/*
 * Launch overlap for serving loops (process-wide switch, default off; no counterpart in the
 * reference, whose generated host code launches every kernel fully stream-ordered).  When on,
 * the decode-path matmul kernels (m <= 32) are launched as programmatic dependents: a kernel may
 * become resident and start streaming its WEIGHT, SCALE and ZERO-POINT tensors while the previous
 * kernel on the stream is still finishing; it reads x / bias / residual and writes out / scratch
 * only after that kernel has completed, so activations stay ordered as before.
 * Contract when on: the weight, scale and zero-point tensors passed to a matmul call were not
 * written by the kernel immediately before it on the same stream (repack weights ahead of time,
 * or synchronise once after preprocessing).  Works inside CUDA-graph capture.
 */
RB200_API int rb200_set_launch_overlap(int enabled);
RB200_API int rb200_get_launch_overlap(void);

/* ------------------------------------------------------------------ weight preprocess */

/* Source layouts accepted by rb200_preprocess_weight. */
#define RB200_LAYOUT_FT_KN 0 /* int8 container [K, N/2] (int4, low nibble = even column) or [K, N] (int8), signed codes */
#define RB200_LAYOUT_Q4_NK 1 /* uint32 [N, K/8], nibble j of a word = element 8*word + j, unsigned codes */
#define RB200_LAYOUT_GATE_UP_INTERLEAVE 0x100 /* flag, OR-ed into a layout: fragment row block nb = gate rows 8nb..8nb+7
                                                 followed by up rows 8nb..8nb+7 (source rows [0, n/2) = gate, [n/2, n) = up) */
#define RB200_LAYOUT_AUTOGPTQ_KN 2 /* uint32 [K/8, N], nibble j of word (k/8, n) = element k = 8*(k/8) + j, unsigned
                                      codes (tests/python/dlight/test_gpu_gemv.py:639-649) */

/*
 * Repack a packed int4/int8 weight into the kernel-private fragment layout; the result has
 * exactly the byte size of the source.  Stands in for
 *   cutlass.ft_preprocess_weight(NDArray packed_weight, int sm, bool is_int4)
 *   (src/runtime/contrib/cutlass/weight_preprocess.cc:38-58), which calls
 *   fastertransformer::preprocess_weights(out, in, num_experts, rows, cols, is_int4, sm).
 * `k` and `n` are the logical (unpacked) reduction and output extents of ONE expert; both
 * buffers are device memory, `dst` must not alias `src`.  Signed FT codes are stored biased
 * to unsigned (int4: +8, int8: +128), as the reference's preprocess does.
 * Requirements: n % 16 == 0; k % 64 == 0 (int4) or k % 32 == 0 (int8).
 */
RB200_API int rb200_preprocess_weight(const void* src, void* dst, int64_t num_experts, int64_t k,
                                      int64_t n, int is_int4, int src_layout, void* stream);

/*
 * AutoGPTQ zero points (tests/python/dlight/test_gpu_gemv.py:639-649): zq uint32
 * [groups, n/8], nibble j of word (g, n/8) = column 8*(n/8) + j.  Writes fp16 [groups, n] holding
 * f16(zq) + f16(1) - the value that decode subtracts - ready to be passed as the `zeros` tensor
 * of rb200_gemm_fp16_intx with scale_stride_n = 1, scale_stride_g = n.  The matmul entries take
 * groups in order along k (g_idx[k] = k / group_size); for an arbitrary g_idx see
 * rb200_gptq_act_order below.
 */
RB200_API int rb200_unpack_zeros_autogptq(const void* zq, void* zeros_out, int64_t groups, int64_t n, void* stream);

/*
 * Act-order AutoGPTQ weights: the reference decode reads scale and zero of element k through
 * g_idx[k] (tests/python/dlight/test_gpu_gemv.py:646-648, `lv12[v_i]`).  The matmul kernels want
 * groups contiguous along k, so the reduction axis is permuted once at load time:
 *   rb200_gptq_act_order                  g_idx int32 [k] (device) -> perm int32 [k] (device): the k rows listed
 *                                         group by group, original order inside a group.  Every
 *                                         group must have exactly k / groups rows (error otherwise).
 *                                         Set-up routine: synchronises the stream, allocates 4 bytes.
 *   rb200_preprocess_weight_autogptq_perm repack of qweight uint32 [k/8, n] with row perm[j] of the
 *                                         source at position j of the reduction axis
 *   rb200_gather_columns                  out[m, j] = x[m, perm[j]] (fp16), run before each matmul
 * With these, gemm(gather(x), repacked weight, scales, zeros) sums the same products as the
 * reference's x @ decode(W, g_idx), in a different order.
 */
RB200_API int rb200_gptq_act_order(const int32_t* g_idx, int64_t k, int64_t groups, int32_t* perm_out, void* stream);
RB200_API int rb200_preprocess_weight_autogptq_perm(const void* qweight, void* dst, int64_t k, int64_t n,
                                                    const int32_t* perm, void* stream);
RB200_API int rb200_gather_columns(const void* x, const int32_t* perm, void* out, int64_t m, int64_t k,
                                   int64_t ldx, int64_t ldo, void* stream);

/* ------------------------------------------------------------------ dequantize-matmul */

#define RB200_ACT_IDENTITY 0
#define RB200_ACT_RELU 1
#define RB200_ACT_SILU 2
#define RB200_ACT_GELU 3
/* Fused gated MLP: the weight holds gate rows [0, n/2) and up rows [n/2, n) and was repacked with
 * RB200_LAYOUT_GATE_UP_INTERLEAVE (scales / zeros permuted with rb200_interleave_gate_up); the
 * output is fp16 [m, n/2] = silu(x @ gate^T) * (x @ up^T), both factors taken from the fp32
 * accumulators (the m > 32 kernel rounds them to fp16 first).  No bias / residual / unary op.
 * The reference leaves this to a separate split + silu + multiply after the matmul. */
#define RB200_ACT_SWIGLU 4
#define RB200_BIN_NONE 0
#define RB200_BIN_PLUS 1
#define RB200_BIN_MULTIPLY 2
#define RB200_UN_IDENTITY 0
#define RB200_UN_RELU 1

/*
 * Full description of one  out = unary(binary(act(x @ dequant(W)^T + bias), residual))  call.
 *   dequant:  wq[n,k] = f16_rn((f16(u[n,k]) - z) * s),  s = scales[n*scale_stride_n + (k/group)*scale_stride_g],
 *             z = zeros[same index] when zeros != NULL, else the constant `zero_const`.
 *   matmul :  fp32 accumulation, one rounding to fp16 after the epilogue.
 */
typedef struct rb200_gemm_desc {
  uint32_t struct_size;     /* sizeof(rb200_gemm_desc), for forward compatibility */
  int32_t weight_bits;      /* 4 or 8 */
  const void* x;            /* fp16 [m, k], row stride ldx elements */
  const void* w;            /* preprocessed weight from rb200_preprocess_weight */
  const void* scales;       /* fp16 */
  const void* zeros;        /* fp16 per-group zero points, or NULL */
  const void* bias;         /* fp16 or NULL */
  const void* residual;     /* fp16 [m, n] or NULL */
  void* out;                /* fp16 [m, n], row stride ldo elements */
  int64_t m, n, k;
  int64_t ldx, ldo;
  int64_t group_size;       /* <= 0 or >= k: one scale per output channel */
  int64_t scale_stride_n;   /* elements between consecutive n */
  int64_t scale_stride_g;   /* elements between consecutive k-groups */
  int64_t bias_stride;      /* 0: bias[n] broadcast over rows; n: bias[m, n] */
  float zero_const;         /* used when zeros == NULL (7 q4f16_1, 8 FT int4, 128 FT int8) */
  int32_t activation;       /* RB200_ACT_* */
  int32_t binary_op;        /* RB200_BIN_* (needs residual) */
  int32_t unary_op;         /* RB200_UN_* */
  int32_t reserved;
  void* workspace;          /* optional caller scratch (device); NULL -> library-owned per-device scratch */
  size_t workspace_bytes;
} rb200_gemm_desc;

/* General entry.  Chooses the decode kernel (m <= 32) or the tensor-core kernel (m > 32). */
RB200_API int rb200_gemm_fp16_intx(const rb200_gemm_desc* desc, void* stream);

/* Scratch bytes rb200_gemm_fp16_intx may use for this problem on the current device. */
RB200_API size_t rb200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k, int weight_bits);

/*
 * Stand-ins for the calls the reference's generated host code makes
 * (python/tvm/contrib/cutlass/gemm_operation.py:441-447 and :449-458):
 *   fastertransformer::gemm_fp16_int_bias_act<WeightT, QuantOp>(A, B, scales, bias, out, act,
 *        m, n, k, group_size, bias_stride, workspace, workspace_bytes, stream)
 *   fastertransformer::gemm_fp16_int_bias_act_residual<WeightT, QuantOp>(A, B, scales, bias,
 *        residual, out, act, binary_op, unary_op, m, n, k, group_size, workspace, bytes, stream)
 * WeightT becomes `weight_bits`; QuantOp follows from group_size (== k or <= 0: per column
 * scales [n]; otherwise fine-grained scales [k/group_size, n]).  B comes from
 * rb200_preprocess_weight(..., RB200_LAYOUT_FT_KN).  Activation / op names as the reference
 * passes them: "identity"|"relu"|"silu"|"gelu", "plus"|"multiply", "identity"|"relu".
 */
RB200_API int rb200_gemm_fp16_int_bias_act(const void* A, const void* B, const void* scales,
                                           const void* bias, void* out, const char* activation,
                                           int m, int n, int k, int group_size, int bias_stride,
                                           int weight_bits, void* workspace,
                                           size_t workspace_bytes, void* stream);
RB200_API int rb200_gemm_fp16_int_bias_act_residual(
    const void* A, const void* B, const void* scales, const void* bias, const void* residual,
    void* out, const char* activation, const char* binary_op, const char* unary_op, int m, int n,
    int k, int group_size, int weight_bits, void* workspace, size_t workspace_bytes, void* stream);

/*
 * No counterpart in the reference: the same decode-path computation as rb200_gemm_fp16_intx for
 * hosts that must not allocate device memory while running - runtimes whose own pool already
 * owns the whole device (a driver allocation from inside the library would fail), and serving
 * loops that forbid driver allocation calls on their hot thread because such calls stall the
 * device.  This entry point calls no cudaMalloc / cudaFree and no allocating library routine:
 * its split-k scratch is a fixed array inside the library image (about 5.06 MiB of device
 * memory on every GPU that loads the library, held until the process exits).
 *   Limits : m <= 16 and n <= 262144 (anything larger is rejected with an error, as is a
 *            problem whose partials would not fit); `workspace` in the descriptor is ignored;
 *            RB200_ACT_SWIGLU and unknown activation / op codes are rejected (the kernel behind
 *            this entry has no fused gate/up form).
 *   Set-up : the first call on each device resolves the array's device address and queries the
 *            device; make that first call with the device current and before any stream capture.
 *   Sharing: every call on a device uses the same array.  Each call clears the tickets it needs
 *            on `stream` before launching, so calls issued in stream order are independent; calls
 *            that overlap on the GPU (different streams, no dependency between them) race on the
 *            array and give undefined results.
 *   Status : a bounded wait that gives up sets the status word inside the array; it stays set
 *            until rb200_check_async_error reads it, which allocates nothing either.
 */
RB200_API int rb200_gemm_fp16_intx_noalloc(const rb200_gemm_desc* desc, void* stream);

/*
 * Grouped matmul (mixture of experts): rows [indptr[e-1], indptr[e]) of x (indptr[-1] = 0) are
 * multiplied by expert e's weight,  out[r] = x[r] @ decode(W[e])^T,  fp32 accumulation, fp16 out.
 * Replaces cutlass_group_gemm as called from tvm_cutlass_group_gemm_sm90
 * (src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64; argument building in
 * src/runtime/contrib/cutlass/group_gemm_runner.cuh:154-209): same x / indptr / out convention
 * (indptr is a DEVICE int64 array of end offsets, read by the kernel - no host synchronisation).
 * weight_bits 16: dense fp16 weights [num_experts, n, k] (the reference's form).
 * weight_bits 4 / 8: packed weights, one rb200_preprocess_weight result per expert
 * (num_experts * n * k * bits / 8 bytes), scales / zeros addressed
 *   e * scale_stride_e + n_idx * scale_stride_n + (k_idx / group_size) * scale_stride_g
 * - an extension: the reference has no quantised grouped GEMM.
 * Needs n % 128 == 0, k % 64 == 0, 16-byte aligned x / out rows, num_experts <= 64.
 * workspace is accepted for signature parity and not used (nothing is allocated per call).
 * Packed weights with at most 32 rows in all (decode-size batches) run as one launch of the
 * decode kernel per expert - each launch reads its row range from indptr on the device and
 * returns at once when the expert has no rows - and then need only n % 16 == 0.
 */
typedef struct rb200_group_gemm_desc {
  uint32_t struct_size;   /* sizeof(rb200_group_gemm_desc) */
  int32_t weight_bits;    /* 4, 8 or 16 */
  const void* x;          /* fp16 [total_rows, k], rows sorted by expert */
  const void* w;
  const void* scales;     /* fp16; NULL for 16-bit weights */
  const void* zeros;      /* fp16 or NULL */
  const int64_t* indptr;  /* device int64 [num_experts]: end row of each expert */
  void* out;              /* fp16 [total_rows, n] */
  int64_t total_rows, n, k, num_experts;
  int64_t group_size;     /* <= 0 or >= k: one scale per output channel */
  int64_t scale_stride_n, scale_stride_g, scale_stride_e;
  float zero_const;       /* used when zeros == NULL (FT int4: 8, FT int8: 128, q4f16_1: 7) */
  int32_t indptr_has_prev; /* non-zero: `indptr` points into a longer table and indptr[-1] is the first row of
                              expert 0 (a rank that holds experts [e0, e1) of a sharded layer passes
                              table + e0 and w / scales of its own experts; rows outside are left untouched) */
  void* workspace;
  size_t workspace_bytes;
} rb200_group_gemm_desc;
RB200_API int rb200_group_gemm(const rb200_group_gemm_desc* desc, void* stream);

/* ------------------------------------------------------------------ mixture-of-experts routing */

/*
 * The steps on either side of the grouped matmul.  The reference has no operator for them, only
 * the primitives its models compose (stable sort by key, scan: src/runtime/contrib/thrust/thrust.cu:215,325);
 * the row order and indptr convention are what cutlass.group_gemm_fp16_sm90 consumes
 * (src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64).
 *
 * rb200_moe_route: logits fp32 [tokens, num_experts] (device) -> softmax, top_k experts per token
 *   (equal probabilities: lower expert index first).  Assignments are numbered token-major,
 *   flat = token * top_k + j; rows are the assignments stably sorted by expert.  Writes (device):
 *     indptr       int64 [num_experts]      end row of every expert
 *     token_of_row int32 [tokens * top_k]
 *     gate_of_row  fp32  [tokens * top_k]   softmax probability of the assignment
 *     row_of_flat  int32 [tokens * top_k]   where assignment `flat` went
 *   workspace: rb200_moe_route_workspace_bytes(tokens, top_k) bytes of device memory.
 *   num_experts <= 64, top_k <= 8.
 * rb200_moe_gather:  out fp16 [rows, k] = x[token_of_row[row]].
 * rb200_moe_combine: out fp16 [tokens, n] = f16( sum_j gate_of_row[r_j] * y[r_j] ), r_j =
 *   row_of_flat[token * top_k + j], fp32 sum in j order (deterministic).
 */
RB200_API size_t rb200_moe_route_workspace_bytes(int64_t tokens, int64_t top_k);
RB200_API int rb200_moe_route(const void* logits, int64_t tokens, int64_t num_experts, int64_t top_k, int64_t* indptr,
                              int32_t* token_of_row, float* gate_of_row, int32_t* row_of_flat, void* workspace,
                              size_t workspace_bytes, void* stream);
RB200_API int rb200_moe_gather(const void* x, const int32_t* token_of_row, void* out, int64_t rows, int64_t k,
                               void* stream);
RB200_API int rb200_moe_combine(const void* y, const int32_t* row_of_flat, const float* gate_of_row, void* out,
                                int64_t tokens, int64_t top_k, int64_t n, void* stream);

/*
 * The row permutation of RB200_LAYOUT_GATE_UP_INTERLEAVE applied to an fp16 tensor viewed as
 * [outer][n][inner] (scales / zero points: [n, k/g] -> outer 1, inner k/g; [k/g, n] -> outer k/g,
 * inner 1; [n] -> outer 1, inner 1):  dst[o][16b + r][i] = src[o][r < 8 ? 8b + r : n/2 + 8b + r - 8][i].
 */
RB200_API int rb200_interleave_gate_up(const void* src, void* dst, int64_t outer, int64_t n, int64_t inner, void* stream);

/* ------------------------------------------------------------------ quantiser */

/*
 * The reference tests' encode step on the GPU (tests/python/relax/test_codegen_cutlass.py:1391-1457
 * int4, :1630-1676 int8, :2043-2109 int8 in groups of 64), which the reference runs as a CPU
 * transform_params stage: a fp16 [n, k] -> packed int8 [k, n/2] (int4, low nibble = even n) or
 * [k, n] (int8) and scales fp16 [n] (group_size <= 0 or >= k) or [k/group_size, n];
 * scale = max(absmax, 1e-4) / 8 (int4) or / 128 (int8) in fp32, codes rounded half away from zero
 * and clipped.  The result feeds rb200_preprocess_weight (layout RB200_LAYOUT_FT_KN).
 */
RB200_API int rb200_encode_ft(const void* a, void* packed, void* scales, int64_t n, int64_t k, int weight_bits,
                              int64_t group_size, void* stream);

/* ------------------------------------------------------------------ low-latency all-reduce */

/*
 * Sum all-reduce of small fp16 tensors across the GPUs of one node (the partial outputs of a
 * row-parallel matmul at decode batch sizes), one kernel per rank, peers' partial sums pulled
 * over NVLink.  Replaces the one-shot strategy of runtime.disco.cuda_ipc.custom_allreduce
 * (src/runtime/disco/cuda_ipc/custom_allreduce.cc:65-105; kernels in
 * 3rdparty/tensorrt_llm/custom_allreduce_kernels.cu:120-264).  Messages above the workspace's
 * max_count belong on NCCL, as in the reference (custom_allreduce.cc:69-76).
 *
 * Set-up (once per process group, mirrors src/runtime/disco/cuda_ipc/cuda_ipc_memory.cc):
 *   every rank:  rb200_peer_alloc(rb200_allreduce_workspace_bytes(max_count), &ws)   zero-filled
 *                rb200_peer_export(ws, handle)  -> exchange the 64-byte handles by any host channel
 *                rb200_peer_import(handle_of_rank_p, &ws_p) for every p != rank
 *   then a host barrier, so that no rank starts before all workspaces exist.
 * Call: workspaces[p] = this process's address of rank p's workspace (own pointer at [rank]).
 * All ranks must issue the same sequence of calls (same count each time).  in / out are ordinary
 * device tensors of `count` fp16 elements, 16-byte aligned; in == out is allowed.  The result is
 * bit-identical on every rank (fixed summation order, fp32 accumulation, one rounding).
 * A peer that never arrives makes the bounded wait give up after about two seconds: the status
 * word read by rb200_check_async_error becomes non-zero and `out` is left unwritten.
 * Works under CUDA-graph capture (the call number is kept on the device).
 */
#define RB200_PEER_HANDLE_BYTES 64
RB200_API size_t rb200_allreduce_workspace_bytes(int64_t max_count);
RB200_API int rb200_allreduce_oneshot(void* const* workspaces, int rank, int world, const void* in, void* out,
                                      int64_t count, int64_t max_count, void* stream);
/* Single-GPU self-test of the same kernel: all `world` ranks run inside one cooperative launch on
 * the current device (workspaces, ins and outs are `world` local buffers). */
RB200_API int rb200_allreduce_oneshot_selftest(void* const* workspaces, const void* const* ins, void* const* outs,
                                               int world, int64_t count, int64_t max_count, void* stream);
RB200_API int rb200_peer_alloc(size_t bytes, void** ptr);
RB200_API int rb200_peer_free(void* ptr);
RB200_API int rb200_peer_export(void* ptr, void* handle_out /* RB200_PEER_HANDLE_BYTES */);
RB200_API int rb200_peer_import(const void* handle, void** ptr);
RB200_API int rb200_peer_close(void* ptr);

/*
 * Row-parallel matmul finished by the sum over ranks, in ONE kernel per rank: the decode-path
 * (m <= 32) computation of rb200_gemm_fp16_intx on this rank's K-shard, whose epilogue exchanges
 * the fp32 partial tiles with the peers over NVLink (plain peer stores, flags, plain loads - no
 * multicast, no collective library), adds them in rank order and only then applies bias /
 * activation / residual and rounds to fp16.  Every rank ends with the same bits in `out`.
 * Replaces the pair the reference runs for a row-parallel layer: the matmul followed by
 * runtime.disco.allreduce (src/runtime/disco/nccl/nccl.cc:90-98) or its customized all-reduce
 * (src/runtime/disco/cuda_ipc/custom_allreduce.cc:65-105,
 * 3rdparty/tensorrt_llm/custom_allreduce_kernels.cu:120-169), which sums fp16 partials that were
 * rounded once already.
 *   Set-up : every rank allocates rb200_gemm_allreduce_workspace_bytes(max_n) bytes with
 *            rb200_peer_alloc (zero-filled), exports / imports the handles as for
 *            rb200_allreduce_oneshot, then a host barrier.  workspaces[p] = this process's address of
 *            rank p's workspace.
 *   Calls  : all ranks issue the same sequence of calls (same m, n).  Calls that share a workspace
 *            must be stream-ordered on each rank.  n <= max_n, m <= 32, k % 64 == 0, symmetric
 *            weights with per-channel scales or (int4) group-32 [N, K/32] scales; no fused gate/up
 *            activation, no caller workspace.  Larger batches: rb200_gemm_fp16_intx, then a
 *            collective library (messages of megabytes are bandwidth-bound, not latency-bound).
 *   Waits  : bounded (rb200_set_wait_limit_ms); a peer that never arrives leaves `out` unwritten
 *            for the blocks concerned and sets the status word.
 * Works under CUDA-graph capture (the call number is kept on the device).  world == 1 is the
 * plain matmul.
 */
RB200_API size_t rb200_gemm_allreduce_workspace_bytes(int64_t max_n);
RB200_API int rb200_gemm_fp16_intx_allreduce(const rb200_gemm_desc* desc, void* const* workspaces, int rank, int world,
                                             int64_t max_n, void* stream);

/*
 * Self-test of the fused form on ONE GPU: all `world` ranks run inside one cooperative launch
 * (every rank on its share of the SMs, all CTAs resident together, so ranks that wait on one
 * another cannot starve each other).  Every rank computes desc's matmul on the same x and
 * weights; rank r writes rows [r * m, (r + 1) * m) of desc->out, which therefore needs world * m
 * rows and must equal epilogue(world * (x @ W^T)) in every block of rows.  workspaces: `world`
 * zero-filled local buffers of rb200_gemm_allreduce_workspace_bytes(max_n) bytes.
 */
RB200_API int rb200_gemm_fp16_intx_allreduce_selftest(const rb200_gemm_desc* desc, void* const* workspaces, int world,
                                                      int64_t max_n, void* stream);

/*
 * Debug/verification entry: writes the dequantised weight wq fp16 [n, k] (row-major) that the
 * matmul kernels feed to the tensor cores, produced by the same device decode routine.  Uses
 * the w / scales / zeros / group / stride / zero_const fields of the descriptor.  The arithmetic
 * it exposes is the reference's decode TIR (tests/python/dlight/test_gpu_gemv.py:193-198,
 * tests/python/relax/test_codegen_cutlass.py:1371-1389, :1628, :2041).
 */
RB200_API int rb200_dequantize(const rb200_gemm_desc* desc, void* wq_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RELAX_B200_H_ */
