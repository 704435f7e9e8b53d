"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two independent restatements of the reference arithmetic live here:

* ``C`` - ctypes bindings of ``liboracle.so`` (``oracle.c``), fast enough for layer-sized cases
  and used as the timed CPU baseline;
* ``np_*`` - a numpy restatement written separately from the C one, used to pin the C oracle
  and to generate the committed fixtures under ``tests/golden``.

Only the tests, the smoke check and the bench's CPU legs may import this module; the product
package never does.  Reference formulas followed (paths inside the reference project):
decode ``tests/python/dlight/test_gpu_gemv.py:193-198``,
``tests/python/relax/test_codegen_cutlass.py:1358-1389,1615-1628,2029-2041``; encode
``test_codegen_cutlass.py:1391-1457,1630-1676,2043-2109``; matmul
``python/tvm/relax/transform/legalize_ops/linear_algebra.py:46-85``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_fp16.so")


def build(force: bool = False) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.check_call(["make", "-C", _HERE, "all"], stdout=subprocess.DEVNULL)


def _p(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None else None


class _C:
    """ctypes bindings of oracle.c; every array argument is a C-contiguous numpy array."""

    def __init__(self):
        build()
        self.lib = ctypes.CDLL(_LIB_PATH)
        L = self.lib
        L.orc_f32_to_f16.restype = ctypes.c_uint16
        L.orc_f32_to_f16.argtypes = [ctypes.c_float]
        L.orc_f16_to_f32.restype = ctypes.c_float
        L.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.orc_f64_to_f16.restype = ctypes.c_uint16
        L.orc_f64_to_f16.argtypes = [ctypes.c_double]
        L.orc_num_threads.restype = ctypes.c_int

    @property
    def num_threads(self) -> int:
        return int(self.lib.orc_num_threads())

    def decode_q4_nk(self, W, S, Z=None, zconst=7.0, group=32):
        W = np.ascontiguousarray(W, dtype=np.uint32)
        S = np.ascontiguousarray(S, dtype=np.float16)
        N, K = W.shape[0], W.shape[1] * 8
        Zc = None if Z is None else np.ascontiguousarray(Z, dtype=np.float16)
        out = np.empty((N, K), dtype=np.float16)
        self.lib.orc_decode_q4_nk(
            _p(W, ctypes.c_uint32), _p(S.view(np.uint16), ctypes.c_uint16),
            _p(None if Zc is None else Zc.view(np.uint16), ctypes.c_uint16),
            ctypes.c_float(zconst), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(group),
            _p(out.view(np.uint16), ctypes.c_uint16))
        return out

    def decode_ft_kn(self, A, B, bits, group=-1):
        A = np.ascontiguousarray(A, dtype=np.int8)
        B = np.ascontiguousarray(B, dtype=np.float16)
        K = A.shape[0]
        N = A.shape[1] * (2 if bits == 4 else 1)
        out = np.empty((K, N), dtype=np.float16)
        fn = self.lib.orc_decode_ft_int4_kn if bits == 4 else self.lib.orc_decode_ft_int8_kn
        fn(_p(A, ctypes.c_int8), _p(B.view(np.uint16), ctypes.c_uint16), ctypes.c_int64(K),
           ctypes.c_int64(N), ctypes.c_int64(group), _p(out.view(np.uint16), ctypes.c_uint16))
        return out

    def decode_codes(self, codes, S, Z, zconst, group, s_n, s_g):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        S = np.ascontiguousarray(S, dtype=np.float16)
        Zc = None if Z is None else np.ascontiguousarray(Z, dtype=np.float16)
        N, K = codes.shape
        out = np.empty((N, K), dtype=np.float16)
        self.lib.orc_decode_codes(
            _p(codes, ctypes.c_uint8), _p(S.view(np.uint16), ctypes.c_uint16),
            _p(None if Zc is None else Zc.view(np.uint16), ctypes.c_uint16),
            ctypes.c_float(zconst), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(group),
            ctypes.c_int64(s_n), ctypes.c_int64(s_g), _p(out.view(np.uint16), ctypes.c_uint16))
        return out

    def decode_autogptq(self, Wq, Zq, S, g_idx):
        Wq = np.ascontiguousarray(Wq, dtype=np.uint32)
        Zq = np.ascontiguousarray(Zq, dtype=np.uint32)
        S = np.ascontiguousarray(S, dtype=np.float16)
        g_idx = np.ascontiguousarray(g_idx, dtype=np.uint32)
        K, N = Wq.shape[0] * 8, Wq.shape[1]
        out = np.empty((K, N), dtype=np.float16)
        self.lib.orc_decode_autogptq(
            _p(Wq, ctypes.c_uint32), _p(Zq, ctypes.c_uint32), _p(S.view(np.uint16), ctypes.c_uint16),
            _p(g_idx, ctypes.c_uint32), ctypes.c_int64(K), ctypes.c_int64(N),
            _p(out.view(np.uint16), ctypes.c_uint16))
        return out

    def matmul_f32(self, x, w, w_nk=True):
        x = np.ascontiguousarray(x, dtype=np.float16)
        w = np.ascontiguousarray(w, dtype=np.float16)
        M, K = x.shape
        N = w.shape[0] if w_nk else w.shape[1]
        acc = np.empty((M, N), dtype=np.float32)
        self.lib.orc_matmul_f32(
            _p(x.view(np.uint16), ctypes.c_uint16), _p(w.view(np.uint16), ctypes.c_uint16),
            ctypes.c_int(1 if w_nk else 0), ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K),
            _p(acc, ctypes.c_float))
        return acc

    ACT = {"identity": 0, "": 0, "relu": 1, "silu": 2, "gelu": 3}
    BIN = {"": 0, "none": 0, "plus": 1, "multiply": 2}
    UN = {"": 0, "identity": 0, "relu": 1}

    def epilogue(self, acc, bias=None, residual=None, activation="identity", binary_op="",
                 unary_op="identity"):
        acc = np.ascontiguousarray(acc, dtype=np.float32)
        M, N = acc.shape
        b = None
        stride = 0
        if bias is not None:
            b = np.ascontiguousarray(bias, dtype=np.float16)
            stride = N if b.size == M * N and M > 1 else 0
        r = None if residual is None else np.ascontiguousarray(residual, dtype=np.float16)
        out = np.empty((M, N), dtype=np.float16)
        self.lib.orc_epilogue(
            _p(acc, ctypes.c_float), _p(None if b is None else b.view(np.uint16), ctypes.c_uint16),
            ctypes.c_int64(stride), _p(None if r is None else r.view(np.uint16), ctypes.c_uint16),
            ctypes.c_int(self.ACT[activation]), ctypes.c_int(self.BIN[binary_op]),
            ctypes.c_int(self.UN[unary_op]), ctypes.c_int64(M), ctypes.c_int64(N),
            _p(out.view(np.uint16), ctypes.c_uint16))
        return out

    def group_gemm_f32(self, x, wq, indptr):
        x = np.ascontiguousarray(x, dtype=np.float16)
        wq = np.ascontiguousarray(wq, dtype=np.float16)
        indptr = np.ascontiguousarray(indptr, dtype=np.int64)
        E, N, K = wq.shape
        acc = np.zeros((x.shape[0], N), dtype=np.float32)
        self.lib.orc_group_gemm_f32(
            _p(x.view(np.uint16), ctypes.c_uint16), _p(wq.view(np.uint16), ctypes.c_uint16),
            _p(indptr, ctypes.c_int64), ctypes.c_int64(E), ctypes.c_int64(N), ctypes.c_int64(K),
            _p(acc, ctypes.c_float))
        return acc

    def baseline_q4_nk(self, x, W, S, group, n0, n1):
        """Reference-style CPU lowering (materialise decode, then matmul) on rows [n0, n1)."""
        x = np.ascontiguousarray(x, dtype=np.float16)
        W = np.ascontiguousarray(W, dtype=np.uint32)
        S = np.ascontiguousarray(S, dtype=np.float16)
        M, K = x.shape
        N = W.shape[0]
        scratch = np.empty(((n1 - n0), K), dtype=np.float16)
        out = np.zeros((M, N), dtype=np.float16)
        self.lib.orc_baseline_q4_nk(
            _p(x.view(np.uint16), ctypes.c_uint16), _p(W, ctypes.c_uint32),
            _p(S.view(np.uint16), ctypes.c_uint16), ctypes.c_int64(M), ctypes.c_int64(N),
            ctypes.c_int64(K), ctypes.c_int64(group), ctypes.c_int64(n0), ctypes.c_int64(n1),
            _p(scratch.view(np.uint16), ctypes.c_uint16), _p(out.view(np.uint16), ctypes.c_uint16))
        return out


_c_singleton = None


def C() -> _C:
    global _c_singleton
    if _c_singleton is None:
        _c_singleton = _C()
    return _c_singleton


def ref_fp16():
    """The reference's own converters (oracle/_ref), or None when they were never built."""
    if not os.path.exists(_REF_PATH):
        return None
    lib = ctypes.CDLL(_REF_PATH)
    lib.ref_f32_to_f16.restype = ctypes.c_uint16
    lib.ref_f32_to_f16.argtypes = [ctypes.c_float]
    lib.ref_f16_to_f32.restype = ctypes.c_float
    lib.ref_f16_to_f32.argtypes = [ctypes.c_uint16]
    lib.ref_f64_to_f16.restype = ctypes.c_uint16
    lib.ref_f64_to_f16.argtypes = [ctypes.c_double]
    return lib


# --------------------------------------------------------------------------- numpy restatement

def np_unpack_q4_nk(W):
    """uint32 [N, K/8] -> codes uint8 [N, K]; nibble j of a word is element 8*word + j."""
    W = np.asarray(W, dtype=np.uint32)
    sh = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    return ((W[:, :, None] >> sh) & 15).astype(np.uint8).reshape(W.shape[0], -1)


def np_decode_q4_nk(W, S, Z=None, zconst=7.0, group=32):
    """(f16(u) - z) * s evaluated in float16 ops (numpy rounds each op to nearest even)."""
    u = np_unpack_q4_nk(W).astype(np.float16)
    S = np.asarray(S, dtype=np.float16)
    z = np.float16(zconst) if Z is None else np.repeat(np.asarray(Z, np.float16), group, axis=1)
    return ((u - z).astype(np.float16) * np.repeat(S, group, axis=1)).astype(np.float16)


def np_unpack_ft_int4_kn(A):
    """int8 [K, N/2] -> signed values int8 [K, N]; low nibble = even column."""
    A = np.asarray(A, dtype=np.int8).astype(np.int32)
    lo = ((A & 15) << 28) >> 28
    hi = (((A >> 4) & 15) << 28) >> 28
    out = np.empty((A.shape[0], A.shape[1] * 2), dtype=np.int8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


def np_decode_ft_kn(A, B, bits, group=-1):
    v = np_unpack_ft_int4_kn(A) if bits == 4 else np.asarray(A, dtype=np.int8)
    K, N = v.shape
    B = np.asarray(B, dtype=np.float16)
    if group <= 0 or group >= K:
        s = B.reshape(1, N)
    else:
        s = np.repeat(B.reshape(K // group, N), group, axis=0)
    return (v.astype(np.float16) * s).astype(np.float16)


def np_matmul_f32(x, w_nk):
    """fp32 products, fp32 sums (numpy's pairwise order; equal to the sequential order only
    up to fp32 rounding - use for tolerance checks, not bit checks)."""
    return np.asarray(x, np.float32) @ np.asarray(w_nk, np.float32).T


def _round_half_away(v):
    """T.round lowers to round-half-away-from-zero (llvm.round), unlike numpy's half-to-even."""
    # in float64 so that |v| + 0.5 is exact for float32 inputs (0.49999997 must round to 0)
    v64 = np.asarray(v, dtype=np.float64)
    return (np.sign(v64) * np.floor(np.abs(v64) + 0.5)).astype(np.float32)


def np_encode_ft(y, bits, group=-1):
    """The reference tests' quantiser (test_codegen_cutlass.py:1391-1457 int4, :1630-1676 int8,
    :2043-2109 int8 group 64).  y fp16 [N, K] -> (packed int8 [K, N/2] or [K, N], scales fp16)."""
    y = np.asarray(y, dtype=np.float16)
    N, K = y.shape
    qmax = 8.0 if bits == 4 else 128.0
    mul = np.float32(0.125) if bits == 4 else np.float32(0.0078125)
    if group <= 0 or group >= K:
        absmax = np.max(np.abs(y), axis=1).astype(np.float32)  # [N]
        scale = np.maximum(absmax, np.float32(1e-4)) * mul  # fp32 [N]
        q = _round_half_away(y.astype(np.float32) / scale[:, None])
        scales16 = scale.astype(np.float16)
    else:
        yg = y.reshape(N, K // group, group)
        absmax = np.max(np.abs(yg), axis=2).astype(np.float32)  # [N, K/g]
        scale = np.maximum(absmax, np.float32(1e-4)) * mul
        q = _round_half_away(yg.astype(np.float32) / scale[:, :, None]).reshape(N, K)
        scales16 = np.ascontiguousarray(scale.T).astype(np.float16)  # [K/g, N]
    q = np.clip(q, -qmax, qmax - 1).astype(np.int8)  # [N, K]
    qt = np.ascontiguousarray(q.T)  # [K, N]
    if bits == 8:
        return qt, scales16
    packed = ((qt[:, 0::2].astype(np.int32) & 15) | ((qt[:, 1::2].astype(np.int32) & 15) << 4))
    return packed.astype(np.uint8).view(np.int8), scales16


def np_moe_route(logits, top_k):
    """Routing restatement: softmax, top-k (ties to the lower expert index), assignments numbered
    token-major and stably sorted by expert.  Returns (indptr, token_of_row, gate_of_row,
    row_of_flat) - the inputs of the grouped matmul's convention
    (src/runtime/contrib/cutlass/fp16_group_gemm.cu:39-64, group_gemm_runner.cuh:161-171)."""
    logits = np.asarray(logits, dtype=np.float32)
    t, e = logits.shape
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p = p / p.sum(axis=1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :top_k]
    flat_expert = order.reshape(-1)
    flat_gate = np.take_along_axis(p, order, axis=1).reshape(-1).astype(np.float32)
    perm = np.argsort(flat_expert, kind="stable")
    indptr = np.cumsum(np.bincount(flat_expert, minlength=e)).astype(np.int64)
    row_of_flat = np.empty(t * top_k, dtype=np.int32)
    row_of_flat[perm] = np.arange(t * top_k, dtype=np.int32)
    return indptr, (perm // top_k).astype(np.int32), flat_gate[perm], row_of_flat
