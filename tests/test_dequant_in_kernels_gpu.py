"""Bit-exact dequantised weights as the MATMUL kernels form them, with no debug hook: with rows of
the identity as activations the product has a single non-zero term, so

    out[i, n] == wq[n, k0 + i]        (x[i] = e_{k0 + i})

bit for bit (1.0 * wq is exact in fp32, every other term is an exact zero, the final rounding to
fp16 returns wq).  This pins the decode routines inside the warp-MMA decode kernels and - with
m = k > 32 - the separate routines of the tensor-core kernels (ungrouped, split-k and grouped
forms), which the dequantize entry point does not share."""
import numpy as np
import pytest
import torch

from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status
from tests.util import bits16, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


def _same_bits(got, exp):
    got, exp = bits16(got).copy(), bits16(exp).copy()
    got[got == 0x8000] = 0  # a sum of zeros is +0 where the decoded weight may be -0
    exp[exp == 0x8000] = 0
    return np.array_equal(got, exp)


def _eye_rows(k0, m, k):
    x = torch.zeros(m, k, dtype=torch.float16, device="cuda")
    x[torch.arange(m), torch.arange(k0, k0 + m)] = 1.0
    return x


def _q4_forms(k, n):
    g = np.random.Generator(np.random.PCG64(k * 3 + n))
    yield "g32", synth.q4_case(g, 1, k, n, 32)
    asym = synth.q4_case(g, 1, k, n, 128 if k % 128 == 0 else 64, asymmetric=True)
    asym.zeros[1, 0] = np.float16(2.625)  # a zero point that is not an integer: rounded subtraction
    yield "g128z", asym


@pytest.mark.parametrize("k,n", [(256, 128), (512, 4224)])
def test_decode_kernels_q4(oracle, k, n):
    """m = 32 identity rows at a time through the cluster kernel (n <= 4096) and the stream-k kernel."""
    for tag, case in _q4_forms(k, n):
        pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
        s = to_dev(case.scales)
        z = None if case.zeros is None else to_dev(case.zeros)
        exp = oracle.C().decode_q4_nk(case.w, case.scales, case.zeros, 7.0, case.group)  # [n, k]
        for k0 in range(0, k, 32):
            out = ops.gemm_fp16_q4f16(_eye_rows(k0, 32, k), pre, s, z, group_size=case.group)
            assert _same_bits(out.cpu().numpy(), exp[:, k0:k0 + 32].T), (tag, k0)
        _check_status()


@pytest.mark.parametrize("bits,group", [(4, -1), (4, 64), (8, -1), (8, 64)])
def test_decode_kernels_ft(oracle, bits, group):
    rs = np.random.RandomState(bits + max(group, 0))
    k, n = 256, 4224
    y = rs.normal(0, 0.002, size=(n, k)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, group)
    exp = oracle.C().decode_ft_kn(packed, scales, bits, group)  # [k, n]
    pre = ops.preprocess_weight_ft(to_dev(packed), bits == 4)
    for k0 in range(0, k, 32):
        out = ops.gemm_fp16_ft(_eye_rows(k0, 32, k), pre, to_dev(scales), bits, group_size=group)
        assert _same_bits(out.cpu().numpy(), exp[k0:k0 + 32]), k0
    _check_status()


@pytest.mark.parametrize("k", [64, 256, 512, 1024])
def test_tensor_core_kernel_q4(oracle, k):
    """m = k identity through the tcgen05 kernel; n = 128 with k = 1024 takes the split-k form,
    n = 2560 the unsplit persistent form."""
    for n in (128, 2560):
        for tag, case in _q4_forms(k, n):
            pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
            z = None if case.zeros is None else to_dev(case.zeros)
            out = ops.gemm_fp16_q4f16(_eye_rows(0, k, k), pre, to_dev(case.scales), z, group_size=case.group)
            torch.cuda.synchronize()
            _check_status()
            exp = oracle.C().decode_q4_nk(case.w, case.scales, case.zeros, 7.0, case.group)
            assert _same_bits(out.cpu().numpy(), exp.T), (tag, n)


@pytest.mark.parametrize("bits,group", [(4, -1), (4, 64), (4, 128), (8, -1), (8, 64)])
@pytest.mark.parametrize("k", [256, 1024])
def test_tensor_core_kernel_ft(oracle, bits, group, k):
    rs = np.random.RandomState(bits * 7 + max(group, 0) + k)
    n = 256
    y = rs.normal(0, 0.002, size=(n, k)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, group)
    exp = oracle.C().decode_ft_kn(packed, scales, bits, group)  # [k, n]
    pre = ops.preprocess_weight_ft(to_dev(packed), bits == 4)
    out = ops.gemm_fp16_ft(_eye_rows(0, k, k), pre, to_dev(scales), bits, group_size=group)
    torch.cuda.synchronize()
    _check_status()
    assert _same_bits(out.cpu().numpy(), exp)


@pytest.mark.parametrize("bits,group", [(4, 128), (4, -1), (8, -1), (8, 64)])
def test_grouped_kernel_ft(oracle, bits, group):
    """One block of identity rows per expert: rows [e*k, (e+1)*k) of x are the identity, so the
    grouped kernel's output block of expert e is that expert's dequantised weight."""
    g = np.random.Generator(np.random.PCG64(bits * 100 + max(group, 0)))
    E, k, n = 3, 256, 256
    w = g.integers(-128, 128, size=(E, k, n // 2 if bits == 4 else n), dtype=np.int8)
    scales = g.uniform(0.001, 0.01, size=(E, k // group, n) if group > 0 else (E, n)).astype(np.float16)
    pre = ops.preprocess_weight_ft(to_dev(w), bits == 4)
    x = torch.cat([_eye_rows(0, k, k) for _ in range(E)], dim=0)
    indptr = torch.tensor([k, 2 * k, 3 * k], dtype=torch.int64, device="cuda")
    out = ops.moe_gemm_ft(x, pre, to_dev(scales), indptr)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    for e in range(E):
        exp = C.decode_ft_kn(w[e], scales[e], bits, group)  # [k, n]
        assert _same_bits(out[e * k:(e + 1) * k].cpu().numpy(), exp), e


def test_grouped_kernel_q4(oracle):
    g = np.random.Generator(np.random.PCG64(9))
    E, k, n = 2, 512, 128
    cases = [synth.q4_case(g, 1, k, n, 32), synth.q4_case(g, 1, k, n, 32)]
    pre = ops.preprocess_weight_q4f16(u32_to_dev(np.stack([c.w for c in cases])))
    s = to_dev(np.stack([c.scales for c in cases]))
    x = torch.cat([_eye_rows(0, k, k) for _ in range(E)], dim=0)
    indptr = torch.tensor([k, 2 * k], dtype=torch.int64, device="cuda")
    out = ops.moe_gemm_q4f16(x, pre, s, indptr, group_size=32)
    torch.cuda.synchronize()
    _check_status()
    for e in range(E):
        exp = oracle.C().decode_q4_nk(cases[e].w, cases[e].scales, None, 7.0, 32)
        assert _same_bits(out[e * k:(e + 1) * k].cpu().numpy(), exp.T), e
