"""Every one of the reference's 22 decode-matmul pattern names, run through the operator it
selects (python/tvm/relax/backend/contrib/cutlass.py:271-314,344-372) on both the decode kernel
(m = 8) and the tensor-core kernel (m = 80), against the oracle's epilogue order
out = unary(binary(act(acc + bias), residual))."""
import numpy as np
import pytest
import torch

from relax_b200 import ops, patterns
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m", [8, 80])
@pytest.mark.parametrize("bits", [4, 8])
def test_every_pattern_name(oracle, bits, m):
    rs = np.random.RandomState(bits * 10 + m)
    k, n = 256, 256
    x = rs.randn(m, k).astype(np.float16)
    y = rs.normal(0, 0.004, size=(n, k)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, -1)
    pre = ops.preprocess_weight_ft(to_dev(packed), bits == 4)
    bias = rs.randn(1, n).astype(np.float16)
    residual = rs.randn(m, n).astype(np.float16)
    C = oracle.C()
    acc = C.matmul_f32(x, C.decode_ft_kn(packed, scales, bits, -1), False)
    xd, sd, bd, rd = to_dev(x), to_dev(scales), to_dev(bias), to_dev(residual)
    for name in patterns.ALL_PATTERNS:
        a = patterns.PATTERN_TABLE[name]
        out = patterns.run_pattern(name, xd, pre, sd, bd if a.bias else None, rd if a.residual else None)
        torch.cuda.synchronize()
        exp = C.epilogue(acc, bias if a.bias else None, residual if a.residual else None, a.activation,
                         a.binary_op, a.unary_op)
        assert_close(out.cpu().numpy(), exp, tight=False)
    _check_status()


def test_pattern_with_fine_grained_scales_and_full_bias(oracle):
    """(K // group_size, N) scales and a bias of the output's shape (bias_stride = n)."""
    rs = np.random.RandomState(3)
    m, k, n = 5, 256, 128
    x = rs.randn(m, k).astype(np.float16)
    y = rs.normal(0, 0.004, size=(n, k)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, 8, 64)
    bias = rs.randn(m, n).astype(np.float16)
    out = patterns.run_pattern("cutlass.decode_matmul_bias_gelu", to_dev(x), ops.preprocess_weight_ft(to_dev(packed), False),
                               to_dev(scales), to_dev(bias))
    torch.cuda.synchronize()
    C = oracle.C()
    exp = C.epilogue(C.matmul_f32(x, C.decode_ft_kn(packed, scales, 8, 64), False), bias, None, "gelu")
    assert_close(out.cpu().numpy(), exp, tight=False)
    with pytest.raises(ValueError):
        patterns.run_pattern("cutlass.decode_matmul", to_dev(x), ops.preprocess_weight_ft(to_dev(packed), False),
                             to_dev(scales), to_dev(bias))
