"""Typed convenience wrappers over the global PackedFuncs (what a Python user of the reference
would write with ``tvm.get_global_func`` + ``relax`` ops for this path)."""
from __future__ import annotations

from typing import Optional

import torch

from .packed_func import get_global_func

LAYOUT_FT_KN = 0
LAYOUT_Q4_NK = 1
LAYOUT_AUTOGPTQ_KN = 2


def preprocess_weight_ft(packed_weight: torch.Tensor, is_int4: bool, sm: int = 100) -> torch.Tensor:
    """``cutlass.ft_preprocess_weight(packed_weight, sm, is_int4)``
    (src/runtime/contrib/cutlass/weight_preprocess.cc:38-58)."""
    return get_global_func("cutlass.ft_preprocess_weight")(packed_weight, int(sm), bool(is_int4))


def preprocess_weight_q4f16(packed_weight: torch.Tensor) -> torch.Tensor:
    """Repack a q4f16_1 weight (uint32 [N, K/8], tests/python/dlight/test_gpu_gemv.py:189)."""
    return get_global_func("relax_b200.preprocess_weight_q4f16")(packed_weight)


def gemm_fp16_ft(x, w_pre, scales, weight_bits: int, bias=None, residual=None,
                 activation: str = "identity", binary_op: str = "", unary_op: str = "identity",
                 group_size: int = -1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(x @ decode(w) + bias)`` (optionally combined with a residual) for FT-layout weights:
    the call python/tvm/contrib/cutlass/gemm_operation.py:441-458 emits."""
    k = x.shape[-1]
    n = w_pre.shape[-1] * (2 if weight_bits == 4 else 1)
    m = x.numel() // k
    if out is None:
        out = torch.empty(*x.shape[:-1], n // 2 if activation == "swiglu" else n, dtype=torch.float16, device=x.device)
    bias_stride = 0
    if bias is not None and bias.numel() == m * n and m > 1:
        bias_stride = n
    name = "cutlass.ft_gemm_fp16_int4" if weight_bits == 4 else "cutlass.ft_gemm_fp16_int8"
    get_global_func(name)(x, w_pre, scales, bias, residual, activation, binary_op, unary_op, m, n, k,
                          int(group_size if group_size > 0 else k), bias_stride, out)
    return out


def gemm_fp16_q4f16(x, w_pre, scales, zeros=None, bias=None, residual=None,
                    activation: str = "identity", binary_op: str = "", unary_op: str = "identity",
                    group_size: int = 32, zero_const: float = 7.0,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode + matmul for q4f16_1-layout weights (tests/python/dlight/test_gpu_gemv.py:193-206),
    fp32 accumulation, fp16 output."""
    n = w_pre.shape[0] // (2 if activation == "swiglu" else 1)
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=torch.float16, device=x.device)
    get_global_func("relax_b200.gemm_fp16_q4f16")(x, w_pre, scales, zeros, bias, residual, activation,
                                                  binary_op, unary_op, int(group_size),
                                                  float(zero_const), out)
    return out


def dequantize(w_pre, scales, n: int, k: int, weight_bits: int, layout: int, zeros=None,
               group_size: int = -1, zero_const: float = 7.0) -> torch.Tensor:
    """The dequantised weight fp16 [N, K] exactly as the matmul kernels form it."""
    out = torch.empty(n, k, dtype=torch.float16, device=w_pre.device)
    get_global_func("relax_b200.dequantize")(w_pre, scales, zeros, int(layout), int(weight_bits),
                                             int(group_size), float(zero_const), out)
    return out


def group_gemm_fp16(x, weight, indptr, workspace=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[r0:r1] = x[r0:r1] @ weight[g].T`` for every group g with ``r1 = indptr[g]``: the call
    src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64 registers as
    ``cutlass.group_gemm_fp16_sm90`` (x fp16 [M, K], weight fp16 [E, N, K], indptr int64 [E] on
    the device)."""
    if out is None:
        out = torch.empty(x.shape[0], weight.shape[1], dtype=torch.float16, device=x.device)
    get_global_func("cutlass.group_gemm_fp16_sm90")(x, weight, indptr, workspace, out)
    return out


def moe_gemm_ft(x, w_pre, scales, indptr, zeros=None, out: Optional[torch.Tensor] = None,
                first_expert: int = 0) -> torch.Tensor:
    """Grouped decode-matmul over FT-layout experts: ``w_pre`` int8 [E, K, N/2] (int4) or
    [E, K, N] (int8) from :func:`preprocess_weight_ft`, ``scales`` fp16 [E, K/g, N] or [E, N].
    Expert-sharded layers: ``w_pre`` / ``scales`` hold experts ``first_expert ..`` only while
    ``indptr`` is the whole layer's table; rows of other experts are left untouched in ``out``."""
    n = scales.shape[-1]
    if out is None:
        out = torch.empty(x.shape[0], n, dtype=torch.float16, device=x.device)
    e_local = w_pre.shape[0]
    if first_expert or e_local != indptr.shape[0]:
        view = indptr[first_expert:first_expert + e_local]
        get_global_func("cutlass.moe_gemm")(x, w_pre, scales, zeros, view, None, out, 1 if first_expert else 0)
    else:
        get_global_func("cutlass.moe_gemm")(x, w_pre, scales, zeros, indptr, None, out)
    return out


def moe_gemm_q4f16(x, w_pre, scales, indptr, zeros=None, group_size: int = 32, zero_const: float = 7.0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped decode-matmul over q4f16_1-layout experts: ``w_pre`` [E, N, K/8] words from
    :func:`preprocess_weight_q4f16`, ``scales`` fp16 [E, N, K/g]."""
    if out is None:
        out = torch.empty(x.shape[0], w_pre.shape[1], dtype=torch.float16, device=x.device)
    get_global_func("relax_b200.moe_gemm_q4f16")(x, w_pre, scales, zeros, indptr, int(group_size),
                                                 float(zero_const), out)
    return out


def gptq_act_order(g_idx: torch.Tensor, groups: int) -> torch.Tensor:
    """Permutation of the reduction axis that makes the groups of an act-order AutoGPTQ weight
    contiguous: ``perm`` int32 [K] lists the k rows group by group (original order inside a group).
    Raises when a group does not have exactly ``K / groups`` rows."""
    g = g_idx.to(device=g_idx.device, dtype=torch.int32).contiguous()
    perm = torch.empty_like(g)
    get_global_func("relax_b200.gptq_act_order")(g, int(groups), perm)
    return perm


def gather_columns(x: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """``x[..., perm]`` for fp16 ``x`` (the activation side of an act-order weight)."""
    out = torch.empty_like(x)
    get_global_func("relax_b200.gather_columns")(x.contiguous(), perm, out)
    return out


def preprocess_weight_autogptq(qweight: torch.Tensor, perm: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Repack an AutoGPTQ weight (uint32 [K/8, N], 8 k-consecutive nibbles per word:
    tests/python/dlight/test_gpu_gemv.py:639-649).  ``perm`` (from :func:`gptq_act_order`) puts
    source row ``perm[j]`` at position ``j`` of the reduction axis."""
    if perm is None:
        return get_global_func("relax_b200.preprocess_weight_autogptq")(qweight)
    out = torch.empty_like(qweight)
    get_global_func("relax_b200.preprocess_weight_autogptq", raw=True)(qweight, out, perm)
    return out


def unpack_zeros_autogptq(qzeros: torch.Tensor) -> torch.Tensor:
    """AutoGPTQ zero points uint32 [G, N/8] -> fp16 [G, N] holding ``f16(zq) + 1``, the value the
    reference's decode subtracts (tests/python/dlight/test_gpu_gemv.py:648)."""
    out = torch.empty(qzeros.shape[0], qzeros.shape[1] * 8, dtype=torch.float16, device=qzeros.device)
    get_global_func("relax_b200.unpack_zeros_autogptq")(qzeros, out)
    return out


def gemm_fp16_autogptq(x, w_pre, scales, zeros, bias=None, g_idx=None, perm=None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``bias + x @ ((q - zeros[g_idx]) * scales[g_idx])`` for AutoGPTQ weights
    (tests/python/dlight/test_gpu_gemv.py:639-661): ``w_pre`` from
    :func:`preprocess_weight_autogptq`, ``scales`` fp16 [G, N], ``zeros`` fp16 [G, N] from
    :func:`unpack_zeros_autogptq`.  With groups in order along k (``g_idx = k // group_size``)
    nothing else is needed.  For an act-order weight pass the ``perm`` that ``w_pre`` was repacked
    with: ``x`` is gathered through it first.  A reordered ``g_idx`` without ``perm`` is rejected."""
    k, n = w_pre.shape[0] * 8, w_pre.shape[1]
    if perm is not None:
        x = gather_columns(x, perm)
    elif g_idx is not None:
        expect = torch.arange(k, device=g_idx.device) // (k // scales.shape[0])
        if not torch.equal(g_idx.to(torch.int64), expect):
            raise ValueError("g_idx reorders the groups: repack the weight with gptq_act_order's perm and pass perm")
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=torch.float16, device=x.device)
    get_global_func("relax_b200.gemm_fp16_autogptq")(x, w_pre, scales, zeros, bias, out)
    return out


def encode_ft(y: torch.Tensor, weight_bits: int, group_size: int = -1):
    """The reference tests' quantiser on the GPU (tests/python/relax/test_codegen_cutlass.py:1391-1457,
    :1630-1676, :2043-2109): ``y`` fp16 [N, K] -> ``(packed int8 [K, N/2] | [K, N], scales fp16 [N] |
    [K/group, N])``, ready for :func:`preprocess_weight_ft`."""
    import ctypes
    from . import _lib
    n, k = y.shape
    per_row = group_size <= 0 or group_size >= k
    packed = torch.empty(k, n // 2 if weight_bits == 4 else n, dtype=torch.int8, device=y.device)
    scales = torch.empty((n,) if per_row else (k // group_size, n), dtype=torch.float16, device=y.device)
    y = y.contiguous()
    _lib.check(_lib.load().rb200_encode_ft(ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(packed.data_ptr()),
                                           ctypes.c_void_p(scales.data_ptr()), n, k, int(weight_bits),
                                           int(group_size), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return packed, scales


def _ptr(t):
    import ctypes
    return ctypes.c_void_p(t.data_ptr())


def moe_route(logits: torch.Tensor, top_k: int, out=None, workspace: Optional[torch.Tensor] = None):
    """Softmax + top-k routing (``rb200_moe_route``): returns ``(indptr int64 [E], token_of_row int32
    [R], gate_of_row fp32 [R], row_of_flat int32 [R])`` with rows sorted by expert, the convention
    of the grouped matmul (src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64).  ``out`` (the same
    four tensors) and ``workspace`` (uint8, :func:`moe_route_workspace_bytes`) make the call
    allocation-free, e.g. for CUDA-graph capture; ``logits`` must then be contiguous fp32."""
    import ctypes
    from . import _lib
    lib = _lib.load()
    t, e = logits.shape
    r = t * top_k
    dev = logits.device
    if out is None:
        out = (torch.empty(e, dtype=torch.int64, device=dev), torch.empty(r, dtype=torch.int32, device=dev),
               torch.empty(r, dtype=torch.float32, device=dev), torch.empty(r, dtype=torch.int32, device=dev))
    indptr, token_of_row, gate_of_row, row_of_flat = out
    nbytes = lib.rb200_moe_route_workspace_bytes(t, top_k)
    if workspace is None:
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    elif workspace.numel() < nbytes:
        raise ValueError("routing workspace holds %d bytes, %d needed" % (workspace.numel(), nbytes))
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        logits = logits.contiguous().float()
    _lib.check(lib.rb200_moe_route(_ptr(logits), t, e, top_k, _ptr(indptr), _ptr(token_of_row), _ptr(gate_of_row),
                                   _ptr(row_of_flat), _ptr(workspace), workspace.numel(),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return indptr, token_of_row, gate_of_row, row_of_flat


def moe_route_workspace_bytes(tokens: int, top_k: int) -> int:
    from . import _lib
    return int(_lib.load().rb200_moe_route_workspace_bytes(tokens, top_k))


def moe_gather(x: torch.Tensor, token_of_row: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[r] = x[token_of_row[r]]``: the rows of x in the grouped matmul's order."""
    import ctypes
    from . import _lib
    if out is None:
        out = torch.empty(token_of_row.numel(), x.shape[1], dtype=torch.float16, device=x.device)
    x = x.contiguous()
    _lib.check(_lib.load().rb200_moe_gather(_ptr(x), _ptr(token_of_row), _ptr(out), token_of_row.numel(), x.shape[1],
                                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out


def moe_combine(y: torch.Tensor, row_of_flat: torch.Tensor, gate_of_row: torch.Tensor, top_k: int,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum over the token's top_k rows of gate * y[row]`` (fp32 sum, one rounding)."""
    import ctypes
    from . import _lib
    tokens = row_of_flat.numel() // top_k
    if out is None:
        out = torch.empty(tokens, y.shape[1], dtype=torch.float16, device=y.device)
    y = y.contiguous()
    _lib.check(_lib.load().rb200_moe_combine(_ptr(y), _ptr(row_of_flat), _ptr(gate_of_row), _ptr(out), tokens, top_k,
                                             y.shape[1], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return out


def preprocess_weight_gate_up(packed_weight: torch.Tensor, layout: int = LAYOUT_Q4_NK, is_int4: bool = True) -> torch.Tensor:
    """Repack a fused gate/up weight (gate rows [0, N/2), up rows [N/2, N)) with the row interleave
    the ``activation="swiglu"`` epilogue expects; scales and zero points need the same permutation
    (:func:`interleave_gate_up`)."""
    return get_global_func("relax_b200.preprocess_weight_gate_up")(packed_weight, int(layout), bool(is_int4))


def interleave_gate_up(t: torch.Tensor, n_axis: int = 0) -> torch.Tensor:
    """The gate/up row permutation applied to an fp16 scale / zero-point tensor along ``n_axis``."""
    out = torch.empty_like(t)
    get_global_func("relax_b200.interleave_gate_up")(t.contiguous(), int(n_axis), out)
    return out
