"""Fused gated-MLP epilogue (activation "swiglu"): one matmul over the fused gate/up weight that
writes silu(gate) * up of half the width.  Checked against the oracle's unfused result
(sequential-fp32 matmul of the full width, then silu(gate) * up in fp32, one rounding)."""
import numpy as np
import pytest
import torch

from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


def _expected(oracle, case):
    C = oracle.C()
    wq = C.decode_q4_nk(case.w, case.scales, case.zeros, case.zero_const, case.group)
    acc = C.matmul_f32(case.x, wq)                       # [m, 2f]: gate | up
    f = acc.shape[1] // 2
    gate, up = acc[:, :f].astype(np.float64), acc[:, f:].astype(np.float64)
    return (gate / (1.0 + np.exp(-gate)) * up).astype(np.float16)


# n <= 4096 takes the cluster kernel, larger n the stream-k kernel, m > 32 the tcgen05 kernel
@pytest.mark.parametrize("m,k,n,group,asym", [(1, 512, 256, 32, False), (8, 1024, 4096, 32, False),
                                               (5, 512, 8192, 32, False), (32, 512, 4608, 128, True),
                                               (17, 1024, 512, 64, False), (100, 512, 256, 32, False),
                                               (300, 1024, 384 * 2, 128, True), (64, 4096, 256, 32, False)])
def test_swiglu_matches_unfused_oracle(oracle, m, k, n, group, asym):
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m + k + n)), m, k, n, group, asymmetric=asym)
    pre = ops.preprocess_weight_gate_up(u32_to_dev(case.w), ops.LAYOUT_Q4_NK, True)
    s = ops.interleave_gate_up(to_dev(case.scales), 0)
    z = None if case.zeros is None else ops.interleave_gate_up(to_dev(case.zeros), 0)
    out = ops.gemm_fp16_q4f16(to_dev(case.x), pre, s, z, activation="swiglu", group_size=group,
                              zero_const=case.zero_const)
    torch.cuda.synchronize()
    _check_status()
    assert out.shape == (m, n // 2)
    # the m > 32 kernel rounds gate and up to fp16 before the activation: reference tolerance only
    assert_close(out.cpu().numpy(), _expected(oracle, case), tight=False)


def test_interleave_is_the_documented_permutation():
    n = 64
    t = torch.arange(n, dtype=torch.float16, device="cuda").reshape(n, 1).repeat(1, 3).contiguous()
    got = ops.interleave_gate_up(t, 0).cpu().numpy()[:, 0]
    exp = np.array([(8 * (j // 16) + j % 16) if j % 16 < 8 else (n // 2 + 8 * (j // 16) + j % 16 - 8) for j in range(n)])
    assert np.array_equal(got, exp.astype(np.float16))
    t2 = torch.arange(n, dtype=torch.float16, device="cuda").reshape(1, n).repeat(2, 1).contiguous()
    assert np.array_equal(ops.interleave_gate_up(t2, 1).cpu().numpy()[1], exp.astype(np.float16))


def test_swiglu_rejects_bias():
    case = synth.q4_case(np.random.Generator(np.random.PCG64(1)), 2, 256, 64, 32)
    pre = ops.preprocess_weight_gate_up(u32_to_dev(case.w), ops.LAYOUT_Q4_NK, True)
    import relax_b200
    with pytest.raises(relax_b200.RB200Error):
        ops.gemm_fp16_q4f16(to_dev(case.x), pre, to_dev(case.scales), bias=torch.zeros(64, dtype=torch.float16, device="cuda"),
                            activation="swiglu")
