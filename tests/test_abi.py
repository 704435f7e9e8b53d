"""CPU checks of the drop-in boundary: the shared library loads without a GPU, exports every
symbol the public headers declare, registers the reference's global function names, and turns
bad arguments into error codes (never aborts, never computes on the host)."""
import ctypes
import os
import re

import pytest
import torch

import relax_b200
from relax_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for h in ("relax_b200.h", "relax_b200_packed.h", "relax_b200_collective.h"):
        p = os.path.join(ROOT, "include", h)
        if not os.path.exists(p):
            continue
        text = re.sub(r"/\*.*?\*/", "", open(p).read(), flags=re.S)
        names += re.findall(r"RB200_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), "library does not export %s" % name
    # and the Python binding table covers the same set
    assert set(declared) <= set(_lib.SIGNATURES), set(declared) - set(_lib.SIGNATURES)


def test_global_function_names_of_the_reference_surface():
    names = relax_b200.list_global_func_names()
    for n in ["cutlass.ft_preprocess_weight", "cutlass.ft_gemm_fp16_int4", "cutlass.ft_gemm_fp16_int8",
              "relax_b200.gemm_fp16_q4f16", "relax_b200.preprocess_weight_q4f16",
              "runtime.get_cuda_stream"]:
        assert n in names
    with pytest.raises(ValueError):
        relax_b200.get_global_func("cutlass.no_such_function")
    assert relax_b200.get_global_func("cutlass.no_such_function", allow_missing=True) is None


def test_bad_arguments_become_errors_not_crashes():
    f = relax_b200.packed_func.get_global_func("cutlass.ft_gemm_fp16_int4")
    x = torch.zeros(2, 64, dtype=torch.float16)
    with pytest.raises(relax_b200.RB200Error):
        f(x, x)  # wrong arity
    w = torch.zeros(64, 8, dtype=torch.int8)
    s = torch.zeros(16, dtype=torch.float16)
    out = torch.zeros(2, 16, dtype=torch.float16)
    with pytest.raises(relax_b200.RB200Error, match="CUDA"):
        f(x, w, s, None, None, "identity", "", "identity", 2, 16, 64, 64, 0, out)  # CPU tensors
    lib = _lib.load()
    d = _lib.GemmDesc()
    d.struct_size = 3
    assert lib.rb200_gemm_fp16_intx(ctypes.byref(d), None) == -1
    assert b"struct_size" in lib.rb200_last_error()
    assert lib.rb200_preprocess_weight(None, None, 1, 64, 16, 1, 0, None) == -1
    assert lib.rb200_preprocess_weight(ctypes.c_void_p(16), ctypes.c_void_p(32), 1, 60, 16, 1, 0, None) == -1
    assert b"k %" in lib.rb200_last_error()


def test_user_registered_function_round_trip():
    lib = _lib.load()
    CB = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_lib.Value), ctypes.POINTER(ctypes.c_int),
                          ctypes.c_int, ctypes.POINTER(_lib.Value), ctypes.POINTER(ctypes.c_int),
                          ctypes.c_void_p)

    def add_one(args, codes, n, ret, ret_code, _res):
        ret[0].v_int64 = args[0].v_int64 + 1
        ret_code[0] = _lib.ARG_INT
        return 0

    cb = CB(add_one)
    assert lib.RB200FuncRegisterGlobal(b"test.add_one", ctypes.cast(cb, ctypes.c_void_p), None, 1) == 0
    assert relax_b200.packed_func.get_global_func("test.add_one")(41) == 42
    assert lib.RB200FuncRegisterGlobal(b"test.add_one", ctypes.cast(cb, ctypes.c_void_p), None, 0) == -1


def test_desc_struct_layout_matches_header():
    """ctypes mirror and C struct agree on size (the library rejects a mismatching struct_size)."""
    lib = _lib.load()
    d = _lib.GemmDesc()
    d.struct_size = ctypes.sizeof(_lib.GemmDesc)
    d.weight_bits = 5
    assert lib.rb200_gemm_fp16_intx(ctypes.byref(d), None) == -1
    assert b"weight_bits" in lib.rb200_last_error()
