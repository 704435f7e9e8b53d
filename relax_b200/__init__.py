"""relax_b200 - B200 (sm_100a) weight-only dequantize-matmul behind the reference's operator surface.

The package is a thin host mirror over ``librelax_b200.so``; importing it loads the library and
raises if it is absent (no CPU or eager fallback exists).
"""
from . import _lib
from ._lib import RB200Error
from .packed_func import get_global_func, list_global_func_names
from . import ops
from .ops import (dequantize, gemm_fp16_ft, gemm_fp16_q4f16, preprocess_weight_ft,
                  preprocess_weight_q4f16)

_lib.load()

__all__ = [
    "RB200Error", "get_global_func", "list_global_func_names", "ops", "dequantize",
    "gemm_fp16_ft", "gemm_fp16_q4f16", "preprocess_weight_ft", "preprocess_weight_q4f16",
]
