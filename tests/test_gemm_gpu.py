"""GPU parity of the prefill path (m > 32, tcgen05 kernel) through the C ABI: outputs within
tolerance of the oracle (fp32 sequential accumulate, fp16 out) at sizes the oracle finishes in
seconds (the full prefill configuration is checked against the oracle in
tests/test_full_configs_gpu.py)."""
import os

import numpy as np
import pytest
import torch

from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status, _run_q4
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [33, 64, 100, 256, 300, 513])
@pytest.mark.parametrize("k,n,group,asym", [(512, 256, 32, False), (1024, 384, 128, True), (320, 128, 64, False),
                                            (256, 128, 256, True)])
def test_prefill_q4(oracle, m, k, n, group, asym):
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m * 7 + k + n)), m, k, n, group, asymmetric=asym)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


def test_prefill_q4_many_tiles_per_cta(oracle):
    """More (weight tile, batch tile) pairs than SMs: every persistent CTA walks several tiles and
    the accumulator / ring phases wrap."""
    case = synth.q4_case(np.random.Generator(np.random.PCG64(5)), 2100, 512, 2560, 32)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


@pytest.mark.parametrize("m,k,n,group,asym", [(64, 4096, 128, 32, False), (100, 2048, 256, 128, True),
                                               (300, 1024, 128, 64, False), (100, 1088, 128, 32, False),
                                               (64, 2752, 256, 32, True)])
def test_prefill_split_k(oracle, m, k, n, group, asym):
    """Fewer tiles than SMs: every tile is cut along k over several CTAs (8, 4, 2 and - with a
    ragged last weight stage - 2 and 5 unequal ranges here); the partial tiles meet in scratch and
    are added in split order.  Two calls in a row: the tickets are back at rest after the first."""
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m + k)), m, k, n, group, asymmetric=asym)
    rs = np.random.RandomState(m)
    bias = rs.randn(n).astype(np.float16)
    got, exp = _run_q4(oracle, case, bias=bias, activation="silu")
    assert_close(got, exp, tight=False)
    got2, _ = _run_q4(oracle, case, bias=bias, activation="silu")
    assert np.array_equal(got, got2)


def test_prefill_epilogues(oracle):
    rs = np.random.RandomState(11)
    m, k, n = 130, 512, 256
    case = synth.q4_case(np.random.Generator(np.random.PCG64(78)), m, k, n, 32)
    bias = rs.randn(n).astype(np.float16)
    res = rs.randn(m, n).astype(np.float16)
    for epi in [dict(bias=bias), dict(bias=bias, activation="gelu"),
                dict(bias=bias, residual=res, binary_op="plus"),
                dict(bias=bias, residual=res, activation="silu", binary_op="multiply", unary_op="relu"),
                dict(bias=rs.randn(m, n).astype(np.float16))]:
        got, exp = _run_q4(oracle, case, **epi)
        assert_close(got, exp, tight=False)


@pytest.mark.parametrize("bits,group,m,k", [(4, -1, 77, 256), (4, 64, 256, 512), (4, 128, 90, 384), (8, -1, 77, 256),
                                            (8, -1, 300, 192), (8, 64, 64, 256)])
def test_prefill_ft_layout(oracle, bits, group, m, k):
    """The reference tests' flow (tests/python/relax/test_codegen_cutlass.py:1355-1609) at m > 32:
    encode, ft_preprocess_weight, fused decode-matmul with bias."""
    rs = np.random.RandomState(bits + m)
    n = 256
    x = rs.randn(m, k).astype(np.float16)
    y = rs.normal(0, 0.002, size=(n, k)).astype(np.float16)
    bias = rs.randn(1, n).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, group)
    pre = ops.preprocess_weight_ft(to_dev(packed), bits == 4, 80)
    out = ops.gemm_fp16_ft(to_dev(x), pre, to_dev(scales), bits, bias=to_dev(bias), group_size=group)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    exp = C.epilogue(C.matmul_f32(x, C.decode_ft_kn(packed, scales, bits, group), False), bias)
    assert_close(out.cpu().numpy(), exp, tight=False)
    if bits == 8:
        # against the unquantised product at the reference's own tolerance (int4 over k >= 256
        # carries more quantisation noise than that tolerance allows; the reference tests it at
        # k = 64, which tests/test_gemv_gpu.py repeats)
        ref = np.dot(x.astype(np.float32), y.astype(np.float32).T) + bias.astype(np.float32)
        np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), ref, rtol=1e-2, atol=1e-2)


def test_prefill_shapes_outside_the_kernel_fall_back_to_slices(oracle):
    """n not a multiple of 128: batch slices on the decode kernel, same answer."""
    case = synth.q4_case(np.random.Generator(np.random.PCG64(9)), 70, 256, 272, 32)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


def test_prefill_int8_llama70b_shard(oracle):
    """Configuration 3 at 1/8 shard, m = 256: column-parallel gate_up and row-parallel down."""
    for name in ("gate_up", "down"):
        case = synth.config3(name, 256, shard=(5, 8))
        pre = ops.preprocess_weight_ft(to_dev(case.w), False)
        out = ops.gemm_fp16_ft(to_dev(case.x), pre, to_dev(case.scales), 8)
        torch.cuda.synchronize()
        _check_status()
        C = oracle.C()
        exp = C.epilogue(C.matmul_f32(case.x, C.decode_ft_kn(case.w, case.scales, 8, -1), False))
        assert_close(out.cpu().numpy(), exp)
