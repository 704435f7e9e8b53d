"""Host-side mirror of the reference's PackedFunc surface for the dequantize-matmul path.

``get_global_func(name)`` plays the role of ``tvm.get_global_func`` (used by the reference's
tests, e.g. tests/python/contrib/test_cutlass.py:1113,1146): it returns a callable bound to the
library's global registry.  Arguments are torch tensors (passed as DLTensor views, no copy),
ints, floats, strings or None; the call launches on torch's current CUDA stream.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Any, Callable, List

import torch

from . import _lib
from ._lib import (ARG_DLTENSOR, ARG_FLOAT, ARG_HANDLE, ARG_INT, ARG_NULL, ARG_STR, DLDataType,
                   DLDevice, DLTensor, Value)

_DTYPES = {
    torch.float16: (2, 16), torch.float32: (2, 32), torch.int8: (0, 8), torch.uint8: (1, 8),
    torch.int32: (0, 32), torch.int64: (0, 64), torch.bfloat16: (4, 16),
}
if hasattr(torch, "uint32"):
    _DTYPES[torch.uint32] = (1, 32)


def as_dltensor(t: torch.Tensor, keep: list) -> DLTensor:
    """A DLTensor struct viewing ``t`` (DLPack ABI); ``keep`` receives the objects that must
    outlive the call."""
    code, bits = _DTYPES[t.dtype]
    shape = (ctypes.c_int64 * max(t.dim(), 1))(*t.shape)
    keep.append(shape)
    strides = None
    if not t.is_contiguous():
        strides = (ctypes.c_int64 * max(t.dim(), 1))(*t.stride())
        keep.append(strides)
    dl = DLTensor()
    dl.data = t.data_ptr()
    dl.device = DLDevice(2 if t.is_cuda else 1, t.device.index or 0 if t.is_cuda else 0)
    dl.ndim = t.dim()
    dl.dtype = DLDataType(code, bits, 1)
    dl.shape = ctypes.cast(shape, ctypes.POINTER(ctypes.c_int64))
    dl.strides = ctypes.cast(strides, ctypes.POINTER(ctypes.c_int64)) if strides is not None else None
    dl.byte_offset = 0
    keep.append(dl)
    return dl


# DLTensor structs of recently seen tensors: a serving loop passes the same buffers on every step,
# and building the ctypes structs costs more host time than a decode kernel runs.  Keyed by
# everything the struct encodes; bounded.
_DL_CACHE: dict = {}
_DL_CACHE_MAX = 8192


def _cached_dltensor(t: torch.Tensor):
    key = (t.data_ptr(), tuple(t.shape), t.dtype, t.device.type, t.device.index,
           None if t.is_contiguous() else tuple(t.stride()))
    hit = _DL_CACHE.get(key)
    if hit is not None:
        return hit[0]
    if len(_DL_CACHE) >= _DL_CACHE_MAX:
        _DL_CACHE.clear()
    keep: List[Any] = []
    dl = as_dltensor(t, keep)
    _DL_CACHE[key] = (dl, keep)
    return dl


class _StreamMemo(threading.local):
    """The stream this thread most recently handed to rb200_set_stream (thread local there too)."""
    value = None


_LAST_STREAM = _StreamMemo()


class BoundCall:
    """A PackedFunc call with its argument arrays built once (``PackedFunc.bind``): a serving loop
    that passes the same buffers on every step pays for the ctypes marshalling only the first
    time.  Calling it launches on torch's current stream of the current device."""

    __slots__ = ("_fn", "_handle", "_values", "_codes", "_n", "_keep", "_ret", "_ret_code", "_set_stream", "_check")

    def __init__(self, handle, values, codes, n, keep):
        lib = _lib.load()
        self._fn = lib.RB200FuncCall
        self._set_stream = lib.rb200_set_stream
        self._handle, self._values, self._codes, self._n, self._keep = handle, values, codes, n, keep
        self._ret = Value()
        self._ret_code = ctypes.c_int(ARG_NULL)
        self._check = _lib.check

    def __call__(self):
        stream = torch.cuda.current_stream().cuda_stream
        if _LAST_STREAM.value != stream:
            self._set_stream(ctypes.c_void_p(stream))
            _LAST_STREAM.value = stream
        rc = self._fn(self._handle, self._values, self._codes, self._n, ctypes.byref(self._ret),
                      ctypes.byref(self._ret_code))
        if rc != 0:
            self._check(rc)


class PackedFunc:
    """One global function of the registry (what ``TVMFuncGetGlobal`` hands back)."""

    def __init__(self, name: str, handle: int):
        self.name = name
        self.handle = handle

    def _marshal(self, args):
        n = len(args)
        values = (Value * max(n, 1))()
        codes = (ctypes.c_int * max(n, 1))()
        keep: List[Any] = []
        for i, a in enumerate(args):
            if a is None:
                values[i].v_handle = None
                codes[i] = ARG_NULL
            elif isinstance(a, torch.Tensor):
                dl = as_dltensor(a, keep)
                keep.append(a)
                values[i].v_handle = ctypes.addressof(dl)
                codes[i] = ARG_DLTENSOR
            elif isinstance(a, bool) or isinstance(a, int):
                values[i].v_int64 = int(a)
                codes[i] = ARG_INT
            elif isinstance(a, float):
                values[i].v_float64 = a
                codes[i] = ARG_FLOAT
            elif isinstance(a, str):
                b = a.encode()
                keep.append(b)
                values[i].v_str = b
                codes[i] = ARG_STR
            else:
                raise TypeError("unsupported PackedFunc argument %r" % type(a))
        return values, codes, n, keep

    def bind(self, *args: Any) -> BoundCall:
        """Marshals ``args`` once; the returned object repeats the call (same tensors, same
        scalars) with no per-call argument work.  The tensors are kept alive by the binding."""
        values, codes, n, keep = self._marshal(args)
        return BoundCall(self.handle, values, codes, n, keep)

    def __call__(self, *args: Any):
        lib = _lib.load()
        n = len(args)
        values = (Value * max(n, 1))()
        codes = (ctypes.c_int * max(n, 1))()
        keep: List[Any] = []
        cuda_dev = None
        for i, a in enumerate(args):
            if a is None:
                values[i].v_handle = None
                codes[i] = ARG_NULL
            elif isinstance(a, torch.Tensor):
                dl = _cached_dltensor(a)
                values[i].v_handle = ctypes.addressof(dl)
                codes[i] = ARG_DLTENSOR
                if a.is_cuda and cuda_dev is None:
                    cuda_dev = a.device
            elif isinstance(a, bool) or isinstance(a, int):
                values[i].v_int64 = int(a)
                codes[i] = ARG_INT
            elif isinstance(a, float):
                values[i].v_float64 = a
                codes[i] = ARG_FLOAT
            elif isinstance(a, str):
                b = a.encode()
                keep.append(b)
                values[i].v_str = b
                codes[i] = ARG_STR
            else:
                raise TypeError("unsupported PackedFunc argument %r" % type(a))
        ret = Value()
        ret_code = ctypes.c_int(ARG_NULL)
        if cuda_dev is not None or torch.cuda.is_available():
            cur = torch.cuda.current_device()
            dev_index = cur if cuda_dev is None or cuda_dev.index is None else cuda_dev.index
            if dev_index == cur:
                stream = torch.cuda.current_stream().cuda_stream
                lib.rb200_set_stream(ctypes.c_void_p(stream))
                _LAST_STREAM.value = stream
                rc = lib.RB200FuncCall(self.handle, values, codes, n, ctypes.byref(ret),
                                       ctypes.byref(ret_code))
            else:
                with torch.cuda.device(dev_index):
                    _LAST_STREAM.value = None
                    lib.rb200_set_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                    rc = lib.RB200FuncCall(self.handle, values, codes, n, ctypes.byref(ret),
                                           ctypes.byref(ret_code))
        else:
            rc = lib.RB200FuncCall(self.handle, values, codes, n, ctypes.byref(ret),
                                   ctypes.byref(ret_code))
        _lib.check(rc)
        if ret_code.value == ARG_HANDLE:
            return ret.v_handle
        if ret_code.value == ARG_INT:
            return ret.v_int64
        return None


def list_global_func_names() -> List[str]:
    lib = _lib.load()
    n = ctypes.c_int()
    arr = ctypes.POINTER(ctypes.c_char_p)()
    _lib.check(lib.RB200FuncListGlobalNames(ctypes.byref(n), ctypes.byref(arr)))
    return [arr[i].decode() for i in range(n.value)]


def _wrap_preprocess(pf: PackedFunc) -> Callable:
    """The reference's ft_preprocess_weight returns a freshly allocated array of the input's
    shape, dtype and device (weight_preprocess.cc:55-57); allocate it here and pass it as the
    destination."""

    def call(packed_weight: torch.Tensor, *rest):
        out = torch.empty_like(packed_weight)
        pf(packed_weight, *rest, out)
        return out

    call.__name__ = pf.name
    return call


_ALLOCATING = {"cutlass.ft_preprocess_weight", "relax_b200.preprocess_weight_q4f16",
               "relax_b200.preprocess_weight_autogptq", "relax_b200.preprocess_weight_gate_up"}
_CACHE = {}


def adopt_managed_tensor(handle: int) -> torch.Tensor:
    """Turns a ``DLManagedTensor*`` returned by a PackedFunc (the allocating form of
    ``cutlass.ft_preprocess_weight``) into a torch tensor without a copy; torch calls the
    tensor's deleter when the last reference goes away."""
    new_capsule = ctypes.pythonapi.PyCapsule_New
    new_capsule.restype = ctypes.py_object
    new_capsule.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    return torch.utils.dlpack.from_dlpack(new_capsule(handle, b"dltensor", None))


def get_global_func(name: str, allow_missing: bool = False, raw: bool = False):
    """``tvm.get_global_func`` counterpart.  Destination-passing operators are returned as is;
    the preprocess functions are wrapped so that they allocate and return their result, like the
    reference's.  ``raw=True`` returns the registered function itself (what a C host gets from
    ``RB200FuncGetGlobal``), without that wrapper."""
    if raw:
        lib = _lib.load()
        h = ctypes.c_void_p()
        _lib.check(lib.RB200FuncGetGlobal(name.encode(), ctypes.byref(h)))
        if not h.value:
            raise ValueError("Cannot find global function %s" % name)
        return PackedFunc(name, h.value)
    hit = _CACHE.get(name)
    if hit is not None:
        return hit
    lib = _lib.load()
    h = ctypes.c_void_p()
    _lib.check(lib.RB200FuncGetGlobal(name.encode(), ctypes.byref(h)))
    if not h.value:
        if allow_missing:
            return None
        raise ValueError("Cannot find global function %s" % name)
    pf = PackedFunc(name, h.value)
    fn = _wrap_preprocess(pf) if name in _ALLOCATING else pf
    _CACHE[name] = fn
    return fn
