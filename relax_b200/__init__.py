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


def set_launch_overlap(enabled: bool) -> None:
    """``rb200_set_launch_overlap``: let decode-path kernels start streaming their weights while
    the previous kernel on the stream is still finishing (see include/relax_b200.h for the
    contract on weight tensors)."""
    _lib.check(_lib.load().rb200_set_launch_overlap(1 if enabled else 0))


def get_launch_overlap() -> bool:
    return bool(_lib.load().rb200_get_launch_overlap())


__all__ = [
    "RB200Error", "get_global_func", "list_global_func_names", "ops", "dequantize",
    "gemm_fp16_ft", "gemm_fp16_q4f16", "preprocess_weight_ft", "preprocess_weight_q4f16",
    "set_launch_overlap", "get_launch_overlap",
]
