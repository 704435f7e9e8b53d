"""ctypes bindings of ``librelax_b200.so`` (the C ABI declared in ``include/relax_b200*.h``).

There is no fallback: if the shared library is missing or fails to load, importing this module
raises, and so does every operator of the package.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# RELAX_B200_LIBRARY overrides the in-tree location (e.g. an instrumented build of the same sources)
LIB_PATH = os.environ.get("RELAX_B200_LIBRARY") or os.path.join(_PKG, "librelax_b200.so")


class GemmDesc(ctypes.Structure):
    """``rb200_gemm_desc`` of include/relax_b200.h."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("weight_bits", ctypes.c_int32),
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("scales", ctypes.c_void_p),
        ("zeros", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("ldx", ctypes.c_int64), ("ldo", ctypes.c_int64),
        ("group_size", ctypes.c_int64), ("scale_stride_n", ctypes.c_int64),
        ("scale_stride_g", ctypes.c_int64), ("bias_stride", ctypes.c_int64),
        ("zero_const", ctypes.c_float),
        ("activation", ctypes.c_int32), ("binary_op", ctypes.c_int32), ("unary_op", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
    ]


class GroupGemmDesc(ctypes.Structure):
    """``rb200_group_gemm_desc`` of include/relax_b200.h."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("weight_bits", ctypes.c_int32),
        ("x", ctypes.c_void_p), ("w", ctypes.c_void_p), ("scales", ctypes.c_void_p),
        ("zeros", ctypes.c_void_p), ("indptr", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("total_rows", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("num_experts", ctypes.c_int64), ("group_size", ctypes.c_int64),
        ("scale_stride_n", ctypes.c_int64), ("scale_stride_g", ctypes.c_int64),
        ("scale_stride_e", ctypes.c_int64),
        ("zero_const", ctypes.c_float), ("indptr_has_prev", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
    ]


class DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p), ("device", DLDevice), ("ndim", ctypes.c_int32),
        ("dtype", DLDataType), ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)), ("byte_offset", ctypes.c_uint64),
    ]


class Value(ctypes.Union):
    """``RB200Value`` (layout of the reference's TVMValue)."""

    _fields_ = [("v_int64", ctypes.c_int64), ("v_float64", ctypes.c_double),
                ("v_handle", ctypes.c_void_p), ("v_str", ctypes.c_char_p)]


ARG_INT, ARG_FLOAT, ARG_HANDLE, ARG_NULL, ARG_DLTENSOR, ARG_STR = 0, 2, 3, 4, 7, 11

# every symbol the headers declare, with (restype, argtypes)
_V = ctypes.c_void_p
_I = ctypes.c_int
_I64 = ctypes.c_int64
_S = ctypes.c_char_p
SIGNATURES = {
    "rb200_last_error": (_S, []),
    "rb200_set_stream": (_I, [_V]),
    "rb200_get_stream": (_V, []),
    "rb200_check_async_error": (_I, [_V, ctypes.POINTER(_I)]),
    "rb200_set_wait_limit_ms": (_I, [ctypes.c_uint]),
    "rb200_set_launch_overlap": (_I, [_I]),
    "rb200_get_launch_overlap": (_I, []),
    "rb200_preprocess_weight": (_I, [_V, _V, _I64, _I64, _I64, _I, _I, _V]),
    "rb200_moe_route_workspace_bytes": (ctypes.c_size_t, [_I64, _I64]),
    "rb200_moe_route": (_I, [_V, _I64, _I64, _I64, _V, _V, _V, _V, _V, ctypes.c_size_t, _V]),
    "rb200_moe_gather": (_I, [_V, _V, _V, _I64, _I64, _V]),
    "rb200_moe_combine": (_I, [_V, _V, _V, _V, _I64, _I64, _I64, _V]),
    "rb200_interleave_gate_up": (_I, [_V, _V, _I64, _I64, _I64, _V]),
    "rb200_encode_ft": (_I, [_V, _V, _V, _I64, _I64, _I, _I64, _V]),
    "rb200_unpack_zeros_autogptq": (_I, [_V, _V, _I64, _I64, _V]),
    "rb200_gptq_act_order": (_I, [_V, _I64, _I64, _V, _V]),
    "rb200_preprocess_weight_autogptq_perm": (_I, [_V, _V, _I64, _I64, _V, _V]),
    "rb200_gather_columns": (_I, [_V, _V, _V, _I64, _I64, _I64, _I64, _V]),
    "rb200_gemm_fp16_intx": (_I, [ctypes.POINTER(GemmDesc), _V]),
    "rb200_gemm_fp16_intx_noalloc": (_I, [ctypes.POINTER(GemmDesc), _V]),
    "rb200_gemm_allreduce_workspace_bytes": (ctypes.c_size_t, [_I64]),
    "rb200_gemm_fp16_intx_allreduce": (_I, [ctypes.POINTER(GemmDesc), ctypes.POINTER(_V), _I, _I, _I64, _V]),
    "rb200_gemm_fp16_intx_allreduce_selftest": (_I, [ctypes.POINTER(GemmDesc), ctypes.POINTER(_V), _I, _I64, _V]),
    "rb200_gemm_workspace_bytes": (ctypes.c_size_t, [_I64, _I64, _I64, _I]),
    "rb200_gemm_fp16_int_bias_act": (_I, [_V, _V, _V, _V, _V, _S, _I, _I, _I, _I, _I, _I, _V,
                                          ctypes.c_size_t, _V]),
    "rb200_gemm_fp16_int_bias_act_residual": (_I, [_V, _V, _V, _V, _V, _V, _S, _S, _S, _I, _I, _I,
                                                   _I, _I, _V, ctypes.c_size_t, _V]),
    "rb200_dequantize": (_I, [ctypes.POINTER(GemmDesc), _V, _V]),
    "rb200_group_gemm": (_I, [ctypes.POINTER(GroupGemmDesc), _V]),
    "rb200_allreduce_workspace_bytes": (ctypes.c_size_t, [_I64]),
    "rb200_allreduce_oneshot": (_I, [ctypes.POINTER(_V), _I, _I, _V, _V, _I64, _I64, _V]),
    "rb200_allreduce_oneshot_selftest": (_I, [ctypes.POINTER(_V), ctypes.POINTER(_V), ctypes.POINTER(_V), _I,
                                              _I64, _I64, _V]),
    "rb200_peer_alloc": (_I, [ctypes.c_size_t, ctypes.POINTER(_V)]),
    "rb200_peer_free": (_I, [_V]),
    "rb200_peer_export": (_I, [_V, _V]),
    "rb200_peer_import": (_I, [_V, ctypes.POINTER(_V)]),
    "rb200_peer_close": (_I, [_V]),
    "RB200FuncGetGlobal": (_I, [_S, ctypes.POINTER(_V)]),
    "RB200FuncCall": (_I, [_V, ctypes.POINTER(Value), ctypes.POINTER(_I), _I,
                           ctypes.POINTER(Value), ctypes.POINTER(_I)]),
    "RB200FuncRegisterGlobal": (_I, [_S, _V, _V, _I]),
    "RB200FuncListGlobalNames": (_I, [ctypes.POINTER(_I), ctypes.POINTER(ctypes.POINTER(_S))]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "relax_b200: %s is missing - build it with `python relax_b200/build.py`; there is no "
            "fallback path" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class RB200Error(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        msg = load().rb200_last_error()
        raise RB200Error(msg.decode() if msg else "relax_b200 call failed")
