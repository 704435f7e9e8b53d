"""The GPU quantiser against the numpy restatement of the reference's encode TIR
(tests/python/relax/test_codegen_cutlass.py:1391-1457, :1630-1676, :2043-2109): codes and scales
bit for bit, then the reference tests' whole flow - encode, preprocess, fused decode-matmul -
against the unquantised product at the reference's tolerance."""
import numpy as np
import pytest
import torch

from relax_b200 import ops
from tests.util import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,group,n,k", [(4, -1, 128, 64), (8, -1, 128, 64), (8, 64, 128, 128), (4, 64, 96, 256),
                                            (4, -1, 1000, 2048), (8, 128, 250, 1024)])
def test_encode_matches_reference_quantiser(oracle, bits, group, n, k):
    rs = np.random.RandomState(bits + n)
    y = rs.normal(0, 0.002, size=(n, k)).astype(np.float16)
    y[3, :] = 0  # an all-zero row exercises the 1e-4 floor of the scale
    packed, scales = ops.encode_ft(to_dev(y), bits, group)
    torch.cuda.synchronize()
    exp_packed, exp_scales = oracle.np_encode_ft(y, bits, group)
    assert np.array_equal(scales.cpu().numpy().view(np.uint16), exp_scales.view(np.uint16))
    assert np.array_equal(packed.cpu().numpy(), exp_packed)


def test_reference_flow_entirely_on_gpu():
    """x 64x64, y 128x64 as in test_fp16A_int4B_gemm: encode -> ft_preprocess_weight -> matmul + bias."""
    rs = np.random.RandomState(0)
    x = rs.randn(64, 64).astype(np.float16)
    y = rs.normal(0, 0.002, size=(128, 64)).astype(np.float16)
    bias = rs.randn(1, 128).astype(np.float16)
    packed, scales = ops.encode_ft(to_dev(y), 4)
    pre = ops.preprocess_weight_ft(packed, True, 80)
    out = ops.gemm_fp16_ft(to_dev(x), pre, scales, 4, bias=to_dev(bias))
    ref = np.dot(x.astype(np.float32), y.astype(np.float32).T) + bias.astype(np.float32)
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), ref, rtol=1e-2, atol=1e-2)
