"""Calling forms at the drop-in boundary that the operator tests do not reach."""
import ctypes

import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import _lib, ops, synth
from relax_b200.packed_func import adopt_managed_tensor, get_global_func
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,experts", [(4, 1), (8, 1), (4, 3)])
def test_ft_preprocess_weight_with_the_reference_argument_list(bits, experts):
    """cutlass.ft_preprocess_weight(packed_weight, sm, is_int4) -> new tensor
    (src/runtime/contrib/cutlass/weight_preprocess.cc:38-58): three arguments, the result allocated
    by the callee on the input's device and handed back; same bytes as the destination-passing form."""
    rs = np.random.RandomState(bits + experts)
    shape = (experts, 128, 64 // (2 if bits == 4 else 1))
    a = rs.randint(-128, 128, size=shape).astype(np.int8)
    src = to_dev(a if experts > 1 else a[0])
    raw = get_global_func("cutlass.ft_preprocess_weight", raw=True)
    handle = raw(src, 80, bits == 4)
    assert handle, "the three-argument form must return the new tensor"
    got = adopt_managed_tensor(handle)
    torch.cuda.synchronize()
    assert got.is_cuda and got.dtype == torch.int8 and tuple(got.shape) == tuple(src.shape)
    dps = torch.empty_like(src)
    assert raw(src, 80, bits == 4, dps) is None
    torch.cuda.synchronize()
    assert torch.equal(got, dps)
    del got  # runs the tensor's deleter (cudaFree)
    # host tensors: allocated with malloc, staged through the device
    host = adopt_managed_tensor(raw(src.cpu(), 80, bits == 4))
    assert not host.is_cuda and torch.equal(host, dps.cpu())
    with pytest.raises(relax_b200.RB200Error):
        raw(src, 80)


def test_gate_up_form_with_default_output_pitch_on_the_tensor_core_kernel(oracle):
    """A plain C caller leaves ldo at 0: with the fused gate/up activation the default row pitch is
    n / 2 on every kernel, the m > 32 kernel included."""
    lib = _lib.load()
    m, k, n = 64, 512, 256
    case = synth.q4_case(np.random.Generator(np.random.PCG64(31)), m, k, n, 32)
    w = u32_to_dev(case.w)
    pre = ops.preprocess_weight_gate_up(w)
    s = ops.interleave_gate_up(to_dev(case.scales), 0)
    x = to_dev(case.x)
    out = torch.full((m + 1, n // 2), float("nan"), dtype=torch.float16, device="cuda")  # one guard row
    d = _lib.GemmDesc()
    d.struct_size = ctypes.sizeof(_lib.GemmDesc)
    d.weight_bits = 4
    d.x, d.w, d.scales, d.out = x.data_ptr(), pre.data_ptr(), s.data_ptr(), out.data_ptr()
    d.m, d.n, d.k = m, n, k
    d.ldx, d.ldo = 0, 0
    d.group_size = 32
    d.scale_stride_n, d.scale_stride_g = k // 32, 1
    d.zero_const = 7.0
    d.activation = 4  # RB200_ACT_SWIGLU
    _lib.check(lib.rb200_gemm_fp16_intx(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    _check_status()
    assert torch.isnan(out[m]).all(), "rows were written at the wrong pitch"
    C = oracle.C()
    acc = C.matmul_f32(case.x, C.decode_q4_nk(case.w, case.scales, None, 7.0, 32))
    gate, up = acc[:, :n // 2], acc[:, n // 2:]
    exp = (gate / (1.0 + np.exp(-gate)) * up).astype(np.float16)
    assert_close(out[:m].cpu().numpy(), exp, tight=False)


def test_unknown_op_codes_are_rejected(oracle):
    lib = _lib.load()
    case = synth.q4_case(np.random.Generator(np.random.PCG64(2)), 4, 256, 64, 32)
    x, s = to_dev(case.x), to_dev(case.scales)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    out = torch.empty(4, 64, dtype=torch.float16, device="cuda")
    for field in ("activation", "binary_op", "unary_op"):
        d = _lib.GemmDesc()
        d.struct_size = ctypes.sizeof(_lib.GemmDesc)
        d.weight_bits = 4
        d.x, d.w, d.scales, d.out = x.data_ptr(), pre.data_ptr(), s.data_ptr(), out.data_ptr()
        d.m, d.n, d.k, d.group_size = 4, 64, 256, 32
        d.scale_stride_n, d.scale_stride_g, d.zero_const = 8, 1, 7.0
        setattr(d, field, 11)
        assert lib.rb200_gemm_fp16_intx(ctypes.byref(d), None) == -1
        assert b"unknown" in lib.rb200_last_error()
