"""Generates the committed fixtures in this directory.

The reference stores no golden vectors for the dequantize-matmul path and cannot be imported
where this was written (its build needs LLVM and un-vendored submodules), so the fixtures are
produced by the numpy restatement of the reference TIR in ``oracle/oracle.py`` (``np_*``), which
is written independently of the C oracle the GPU tests use as checker.  Each fixture stores the
inputs and the expected outputs so the C oracle, and through it the CUDA path, can be checked
against them.  Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as orc  # noqa: E402
from relax_b200 import synth  # noqa: E402


def q4_fixture(name, seed, m, k, n, group, asym):
    g = np.random.Generator(np.random.PCG64(seed))
    case = synth.q4_case(g, m, k, n, group, asymmetric=asym)
    if asym:  # make a few zero points non-integer so the general subtraction path is pinned
        case.zeros[0, 0] = np.float16(3.25)
        case.zeros[-1, -1] = np.float16(0.1)
    wq = orc.np_decode_q4_nk(case.w, case.scales, case.zeros, case.zero_const, group)
    acc = orc.np_matmul_f32(case.x, wq)
    np.savez_compressed(os.path.join(HERE, name), x=case.x, w=case.w, scales=case.scales,
                        zeros=case.zeros if asym else np.zeros(0, np.float16), group=group,
                        wq=wq, out=acc.astype(np.float16))


def ft_fixture(name, seed, m, k, n, bits, group):
    """Reproduces the flow of the reference's end-to-end tests: encode a random fp16 weight
    (tests/python/relax/test_codegen_cutlass.py:1391-1457 / :1630-1676 / :2043-2109), decode it,
    multiply."""
    rs = np.random.RandomState(seed)
    x = rs.randn(m, k).astype(np.float16)
    y = rs.normal(0, 0.002, size=(n, k)).astype(np.float16)
    bias = rs.randn(1, n).astype(np.float16)
    packed, scales = orc.np_encode_ft(y, bits, group)
    wq_kn = orc.np_decode_ft_kn(packed, scales, bits, group)
    acc = orc.np_matmul_f32(x, wq_kn.T)
    np.savez_compressed(os.path.join(HERE, name), x=x, y=y, bias=bias, packed=packed, scales=scales,
                        bits=bits, group=group, wq_kn=wq_kn, out=(acc + bias.astype(np.float32)).astype(np.float16))


def all_codes_fixture(name):
    """Every int4 code against a sweep of scales (incl. products that land in the fp16
    subnormal range) and zero points: pins the rounding of the decode itself."""
    scales = np.array([1.0, 0.001, 0.01, 6.1e-5, 1e-6, 3.3e-7, 0.3333, 65504.0 / 8, 2.5e-5,
                       1.5e-5, 7.7e-4, 0.0999], dtype=np.float16)
    n, k, group = 16 * len(scales), 64, 64
    codes = np.tile(np.arange(16, dtype=np.uint8), (n, k // 16))
    codes = (codes + np.arange(n, dtype=np.uint8)[:, None]) % 16
    w = synth.pack_q4_nk(codes.astype(np.uint8))
    s = np.repeat(scales, 16)[:, None].astype(np.float16)
    wq7 = orc.np_decode_q4_nk(w, s, None, 7.0, group)
    z = (np.arange(n) % 16).astype(np.float16)[:, None]
    z[5, 0] = np.float16(2.5)
    z[9, 0] = np.float16(0.0999)
    wqz = orc.np_decode_q4_nk(w, s, z, 0.0, group)
    np.savez_compressed(os.path.join(HERE, name), w=w, scales=s, zeros=z, group=group, wq7=wq7, wqz=wqz)


if __name__ == "__main__":
    q4_fixture("q4_g32_m3.npz", 11, 3, 256, 48, 32, False)
    q4_fixture("q4_g128_asym_m5.npz", 12, 5, 256, 32, 128, True)
    ft_fixture("ft_int4_percol.npz", 0, 64, 64, 128, 4, -1)       # shapes of test_fp16A_int4B_gemm
    ft_fixture("ft_int8_percol.npz", 0, 64, 64, 64, 8, -1)        # test_fp16A_int8B_gemm
    ft_fixture("ft_int8_g64.npz", 0, 16, 128, 128, 8, 64)         # ..._batched_finegrained
    all_codes_fixture("q4_all_codes.npz")
    print("fixtures written to", HERE)
