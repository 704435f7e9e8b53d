"""GPU parity for the AutoGPTQ-style group-128 asymmetric int4 form, the only in-tree decode with
packed zero points (tests/python/dlight/test_gpu_gemv.py:639-661): qweight uint32 [K/8, N],
qzeros uint32 [K/128, N/8], scales fp16 [K/128, N], w = (q - (zq + 1)) * s."""
import numpy as np
import pytest
import torch

from relax_b200 import ops
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, bits16, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


def _case(seed, m, k, n, group=128):
    g = np.random.Generator(np.random.PCG64(seed))
    qweight = g.integers(0, 2**32, size=(k // 8, n), dtype=np.uint64).astype(np.uint32)
    qzeros = g.integers(0, 2**32, size=(k // group, n // 8), dtype=np.uint64).astype(np.uint32)
    scales = g.uniform(0.001, 0.01, size=(k // group, n)).astype(np.float16)
    g_idx = (np.arange(k) // group).astype(np.uint32)
    x = g.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    bias = g.standard_normal((n,), dtype=np.float32).astype(np.float16)
    return qweight, qzeros, scales, g_idx, x, bias


@pytest.mark.parametrize("k,n", [(256, 64), (4096, 4096)])
def test_autogptq_dequant_bit_exact(oracle, k, n):
    qweight, qzeros, scales, g_idx, _, _ = _case(k + n, 1, k, n)
    pre = ops.preprocess_weight_autogptq(u32_to_dev(qweight))
    zeros = ops.unpack_zeros_autogptq(u32_to_dev(qzeros))
    wq = ops.dequantize(pre, to_dev(scales), n, k, 4, ops.LAYOUT_FT_KN, zeros=zeros, group_size=128, zero_const=0.0)
    torch.cuda.synchronize()
    exp_kn = oracle.C().decode_autogptq(qweight, qzeros, scales, g_idx)
    assert np.array_equal(bits16(wq.cpu().numpy()), bits16(np.ascontiguousarray(exp_kn.T)))
    # the unpacked zero tensor is f16(zq) + 1
    zq = (qzeros[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))[None, None, :]) & 15
    assert np.array_equal(zeros.cpu().numpy(), (zq.reshape(qzeros.shape[0], -1) + 1).astype(np.float16))


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (8, 512, 256), (64, 1024, 384), (300, 512, 256)])
def test_autogptq_matmul(oracle, m, k, n):
    """m = 1, k = n = 4096 is the reference test's own size; larger m runs the prefill kernel."""
    qweight, qzeros, scales, g_idx, x, bias = _case(m * 3 + k, m, k, n)
    pre = ops.preprocess_weight_autogptq(u32_to_dev(qweight))
    zeros = ops.unpack_zeros_autogptq(u32_to_dev(qzeros))
    out = ops.gemm_fp16_autogptq(to_dev(x), pre, to_dev(scales), zeros, bias=to_dev(bias),
                                 g_idx=torch.from_numpy(g_idx.astype(np.int64)))
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq_kn = C.decode_autogptq(qweight, qzeros, scales, g_idx)
    exp = C.epilogue(C.matmul_f32(x, wq_kn, False), bias)
    assert_close(out.cpu().numpy(), exp)


def test_autogptq_reordered_groups_are_rejected():
    qweight, qzeros, scales, g_idx, x, _ = _case(1, 1, 256, 64)
    pre = ops.preprocess_weight_autogptq(u32_to_dev(qweight))
    zeros = ops.unpack_zeros_autogptq(u32_to_dev(qzeros))
    bad = torch.from_numpy(g_idx[::-1].astype(np.int64).copy())
    with pytest.raises(ValueError):
        ops.gemm_fp16_autogptq(to_dev(x), pre, to_dev(scales), zeros, g_idx=bad)


def _act_order_g_idx(seed, k, group):
    """An activation-ordered g_idx: row k belongs to group rank(k) // group for a random ranking,
    the form AutoGPTQ writes with desc_act; every group has exactly `group` rows."""
    g = np.random.Generator(np.random.PCG64(seed))
    rank = g.permutation(k)
    return (rank // group).astype(np.uint32)


@pytest.mark.parametrize("k,n,group", [(256, 64, 128), (4096, 512, 128), (1024, 256, 64)])
def test_act_order_dequant_bit_exact(oracle, k, n, group):
    """wq[perm[j], n] of the reference decode (scales and zeros through g_idx,
    tests/python/dlight/test_gpu_gemv.py:646-648) = row j of the repacked weight, bit for bit."""
    qweight, qzeros, scales, _, _, _ = _case(7 * k + n, 1, k, n, group)
    g_idx = _act_order_g_idx(k + 1, k, group)
    perm = ops.gptq_act_order(torch.from_numpy(g_idx.astype(np.int32)).cuda(), k // group)
    perm_h = perm.cpu().numpy()
    # stable: group by group, original order inside a group
    assert np.array_equal(perm_h, np.argsort(g_idx, kind="stable").astype(np.int32))
    pre = ops.preprocess_weight_autogptq(u32_to_dev(qweight), perm=perm)
    zeros = ops.unpack_zeros_autogptq(u32_to_dev(qzeros))
    wq = ops.dequantize(pre, to_dev(scales), n, k, 4, ops.LAYOUT_FT_KN, zeros=zeros, group_size=group, zero_const=0.0)
    torch.cuda.synchronize()
    exp_kn = oracle.C().decode_autogptq(qweight, qzeros, scales, g_idx)
    assert np.array_equal(bits16(wq.cpu().numpy()), bits16(np.ascontiguousarray(exp_kn[perm_h].T)))


@pytest.mark.parametrize("m,k,n", [(1, 4096, 4096), (8, 512, 256), (300, 512, 256)])
def test_act_order_matmul(oracle, m, k, n):
    qweight, qzeros, scales, _, x, bias = _case(m * 5 + k, m, k, n)
    g_idx = _act_order_g_idx(m + k, k, 128)
    perm = ops.gptq_act_order(torch.from_numpy(g_idx.astype(np.int32)).cuda(), k // 128)
    pre = ops.preprocess_weight_autogptq(u32_to_dev(qweight), perm=perm)
    zeros = ops.unpack_zeros_autogptq(u32_to_dev(qzeros))
    out = ops.gemm_fp16_autogptq(to_dev(x), pre, to_dev(scales), zeros, bias=to_dev(bias), perm=perm)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq_kn = C.decode_autogptq(qweight, qzeros, scales, g_idx)
    exp = C.epilogue(C.matmul_f32(x, wq_kn, False), bias)
    assert_close(out.cpu().numpy(), exp)


def test_act_order_uneven_groups_are_rejected():
    g_idx = np.zeros(256, dtype=np.int32)  # every row in group 0 of 2
    with pytest.raises(RuntimeError):
        ops.gptq_act_order(torch.from_numpy(g_idx).cuda(), 2)
