"""The reference's decode-matmul pattern names and what each one passes to the GEMM entry.

In the reference, which fused graph reaches ``gemm_fp16_int_bias_act[_residual]`` - and with which
epilogue - is decided by name: six base patterns (python/tvm/relax/backend/contrib/cutlass.py:271-314)
and, for the four of them that carry a bias, sixteen residual-block variants (``:344-372``).  The
annotator turns the name into call attributes (python/tvm/contrib/cutlass/build.py:701-777) and the
template into arguments (python/tvm/contrib/cutlass/gemm_operation.py:415-459).  This module is that
table, as data, plus the shape checks of ``_check_decode_matmul`` (``cutlass.py:213-268``) and a
dispatcher that calls the registered operator the way the generated host code would.  Host logic
only; nothing here computes.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import reduce
from typing import Dict, Optional, Sequence

BASE_PATTERNS = (
    "cutlass.decode_matmul",
    "cutlass.decode_matmul_bias",
    "cutlass.decode_matmul_cast",
    "cutlass.decode_matmul_cast_bias",
    "cutlass.decode_matmul_bias_gelu",
    "cutlass.decode_matmul_cast_bias_gelu",
)


@dataclass(frozen=True)
class PatternAttrs:
    """What a pattern name fixes about the call (build.py:718-775)."""
    name: str
    bias: bool          # the fused graph has `matmul + bias`
    cast: bool          # fp32 matmul followed by astype(fp16): same kernel call, fp16 output
    activation: str     # "identity" | "relu" | "silu" | "gelu"
    residual: bool      # residual-block form: gemm_fp16_int_bias_act_residual
    binary_op: str      # "" | "plus" | "multiply"
    unary_op: str       # "identity" | "relu"


def _residual_names():
    # the loop order of residual_block_patterns (cutlass.py:350-370)
    names = []
    for postfix in ("", "_relu"):
        for base in BASE_PATTERNS:
            if "bias" in base:
                for bin_op in ("add", "multiply"):
                    names.append(base + "_residual_" + bin_op + postfix)
    return tuple(names)


RESIDUAL_PATTERNS = _residual_names()
ALL_PATTERNS = BASE_PATTERNS + RESIDUAL_PATTERNS


def attrs_of(name: str) -> PatternAttrs:
    """The attributes ``handle_decode_matmul`` derives from the pattern name (build.py:742-775)."""
    if name not in ALL_PATTERNS:
        raise KeyError("not a decode-matmul pattern of the reference: %s" % name)
    residual_pos = name.find("residual_")
    head = name if residual_pos < 0 else name[:residual_pos]
    body = head[head.find("matmul") + len("matmul"):]
    activation = "identity"
    for act in ("relu", "silu", "gelu"):
        if act in body:
            activation = act
            break
    binary_op, unary_op = "", "identity"
    if residual_pos >= 0:
        postfix = name[residual_pos + len("residual_"):]
        binary_op = "multiply" if postfix.startswith("multiply") else "plus"
        unary_op = "relu" if "relu" in postfix else "identity"
    return PatternAttrs(name, "bias" in body, "cast" in body, activation, residual_pos >= 0, binary_op, unary_op)


PATTERN_TABLE: Dict[str, PatternAttrs] = {n: attrs_of(n) for n in ALL_PATTERNS}


def _is_bias_like(shape: Sequence[int], n: int) -> bool:
    return len(shape) >= 1 and shape[-1] == n and reduce(lambda a, b: a * b, shape, 1) == n


def check_decode_matmul(lhs_shape, lhs_dtype, w_shape, w_dtype, scales_shape, scales_dtype, out_shape, out_dtype,
                        bias_shape=None) -> bool:
    """``_check_decode_matmul`` (cutlass.py:213-268) on shapes and dtypes: fp16 activations, int8
    container, fp16 scales of shape (N,), (1, N) or (K // group_size, N), an fp16 result (fp32 only
    through the ``cast`` patterns), bias (N,)-like or of the output's shape."""
    n = out_shape[-1]
    if out_dtype != "float16" or lhs_dtype != "float16" or w_dtype != "int8" or scales_dtype != "float16":
        return False
    if len(scales_shape) > 2 or scales_shape[-1] != n:
        return False
    if bias_shape is not None:
        if not _is_bias_like(bias_shape, n) and tuple(bias_shape) != tuple(out_shape):
            return False
    return True


def call_arguments(name: str, lhs_shape, w_shape, scales_shape, out_shape, bias_shape=None) -> dict:
    """The integer arguments of the generated call (build.py:718-741, gemm_operation.py:415-421):
    m = product of the lhs batch dims, n / k from the packed weight, weight width from N against the
    container's columns, group size from the scale rows, bias_stride 0 for a row vector."""
    k = w_shape[0]
    n = out_shape[-1]
    if n == w_shape[1]:
        bits = 8
    elif n == w_shape[1] * 2:
        bits = 4
    else:
        raise ValueError("weight container [%d, %d] does not match N=%d" % (w_shape[0], w_shape[1], n))
    group = -1
    if len(scales_shape) == 2 and scales_shape[0] != 1:
        group = k // scales_shape[0]  # the reference hard-codes 64 here (build.py:723)
    m = reduce(lambda a, b: a * b, lhs_shape[:-1], 1)
    bias_stride = 0
    if bias_shape is not None and reduce(lambda a, b: a * b, bias_shape, 1) != bias_shape[-1]:
        bias_stride = bias_shape[-1]
    return {"m": m, "n": n, "k": k, "weight_bits": bits, "group_size": group, "bias_stride": bias_stride,
            "attrs": PATTERN_TABLE[name]}


def run_pattern(name: str, x, w_pre, scales, bias=None, residual=None, out=None):
    """Calls the registered operator for one pattern instance (tensors: torch, CUDA) the way the
    reference's generated host code does: ``cutlass.ft_gemm_fp16_int{4,8}`` with the pattern's
    activation / binary op / unary op names."""
    import torch

    from .packed_func import get_global_func
    a = PATTERN_TABLE[name]
    if a.bias != (bias is not None):
        raise ValueError("%s %s a bias" % (name, "takes" if a.bias else "does not take"))
    if a.residual != (residual is not None):
        raise ValueError("%s %s a residual" % (name, "takes" if a.residual else "does not take"))
    n = w_pre.shape[-1] * 2 if scales.shape[-1] == w_pre.shape[-1] * 2 else w_pre.shape[-1]
    out_shape = tuple(x.shape[:-1]) + (n,)
    ok = check_decode_matmul(tuple(x.shape), str(x.dtype).replace("torch.", ""), tuple(w_pre.shape),
                             str(w_pre.dtype).replace("torch.", ""), tuple(scales.shape),
                             str(scales.dtype).replace("torch.", ""), out_shape, "float16",
                             None if bias is None else tuple(bias.shape))
    if not ok:
        raise ValueError("%s: the reference's pattern check rejects these shapes / dtypes" % name)
    c = call_arguments(name, tuple(x.shape), tuple(w_pre.shape), tuple(scales.shape), out_shape,
                       None if bias is None else tuple(bias.shape))
    if out is None:
        out = torch.empty(out_shape, dtype=torch.float16, device=x.device)
    fn = get_global_func("cutlass.ft_gemm_fp16_int4" if c["weight_bits"] == 4 else "cutlass.ft_gemm_fp16_int8")
    fn(x, w_pre, scales, bias, residual, a.activation, a.binary_op, a.unary_op, c["m"], c["n"], c["k"],
       c["group_size"] if c["group_size"] > 0 else c["k"], c["bias_stride"], out)
    return out
