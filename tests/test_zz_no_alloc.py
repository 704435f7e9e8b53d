"""The allocation-free decode entry point, checked against the ordinary one.

`rb200_gemm_fp16_intx_noalloc` exists for hosts that cannot let the library allocate device
memory (their own pool owns the device, or driver allocation calls are banned on the serving
thread).  It keeps its split-k scratch in a fixed array inside the library, shared by all calls,
so the things worth checking are: same result as `rb200_gemm_fp16_intx` on the same inputs, still
the same on a second call right after the first (the array then holds the first call's leftovers),
and a clear refusal beyond its size limits.  Collected last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import _lib, ops, synth
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _desc(x, pre, scales, out, group, zeros=None, zero_const=7.0):
    m, k = x.shape
    n = out.shape[1]
    d = _lib.GemmDesc()
    d.struct_size = ctypes.sizeof(_lib.GemmDesc)
    d.weight_bits = 4
    d.x, d.w, d.scales, d.out = x.data_ptr(), pre.data_ptr(), scales.data_ptr(), out.data_ptr()
    d.zeros = zeros.data_ptr() if zeros is not None else None
    d.m, d.n, d.k, d.ldx, d.ldo = m, n, k, k, n
    d.group_size = group
    d.scale_stride_n, d.scale_stride_g = k // group, 1
    d.zero_const = zero_const
    return d


def _call(fn, d):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = fn(ctypes.byref(d), stream)
    if rc != 0:
        raise relax_b200.RB200Error(_lib.load().rb200_last_error().decode())


@pytest.mark.parametrize("m,k,n,group,asym", [(1, 4096, 4096, 32, False), (8, 4096, 4096, 32, False),
                                              (16, 11008, 4096, 32, False), (5, 1024, 272, 128, True)])
def test_noalloc_matches_regular_entry_twice_in_a_row(oracle, m, k, n, group, asym):
    lib = _lib.load()
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m + k + n)), m, k, n, group, asymmetric=asym)
    x = torch.from_numpy(case.x).cuda()
    s = torch.from_numpy(case.scales).cuda()
    z = torch.from_numpy(case.zeros).cuda() if asym else None
    pre = ops.preprocess_weight_q4f16(torch.from_numpy(case.w.view(np.int32)).cuda())
    ref = torch.empty(m, n, dtype=torch.float16, device="cuda")
    _call(lib.rb200_gemm_fp16_intx, _desc(x, pre, s, ref, group, z))
    torch.cuda.synchronize()
    outs = []
    for attempt in range(2):  # the second call sees the first call's leftovers in the shared array
        out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _call(lib.rb200_gemm_fp16_intx_noalloc, _desc(x, pre, s, out, group, z))
        torch.cuda.synchronize()
        # the two entry points may split k differently, so they agree to accumulation order
        assert_close(out.cpu().numpy(), ref.cpu().numpy())
        outs.append(out)
    # the entry point itself is deterministic: leftovers of the first call change nothing
    assert torch.equal(outs[0], outs[1])
    # and each of them agrees with the CPU oracle directly
    C = oracle.C()
    wq = C.decode_q4_nk(case.w, case.scales, case.zeros, 7.0, group)
    exp = C.epilogue(C.matmul_f32(case.x, wq))
    assert_close(outs[0].cpu().numpy(), exp)
    assert_close(ref.cpu().numpy(), exp)
    # no bounded wait gave up; asking allocates nothing either
    st = ctypes.c_int(-1)
    assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0 and st.value == 0


def test_noalloc_epilogue_matches_oracle(oracle):
    """bias + silu + residual (multiply) + relu through the allocation-free entry."""
    lib = _lib.load()
    m, k, n = 6, 1024, 512
    case = synth.q4_case(np.random.Generator(np.random.PCG64(99)), m, k, n, 32)
    rs = np.random.RandomState(5)
    bias = rs.randn(n).astype(np.float16)
    res = rs.randn(m, n).astype(np.float16)
    x = torch.from_numpy(case.x).cuda()
    s = torch.from_numpy(case.scales).cuda()
    pre = ops.preprocess_weight_q4f16(torch.from_numpy(case.w.view(np.int32)).cuda())
    bd, rd = torch.from_numpy(bias).cuda(), torch.from_numpy(res).cuda()
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    d = _desc(x, pre, s, out, 32)
    d.bias, d.residual = bd.data_ptr(), rd.data_ptr()
    d.activation, d.binary_op, d.unary_op = 2, 2, 1  # silu, multiply, relu
    for _ in range(2):
        _call(lib.rb200_gemm_fp16_intx_noalloc, d)
    torch.cuda.synchronize()
    C = oracle.C()
    exp = C.epilogue(C.matmul_f32(case.x, C.decode_q4_nk(case.w, case.scales, None, 7.0, 32)), bias, res, "silu",
                     "multiply", "relu")
    assert_close(out.cpu().numpy(), exp, tight=False)


def test_noalloc_refuses_the_fused_gate_up_form_and_unknown_codes(oracle):
    lib = _lib.load()
    case = synth.q4_case(np.random.Generator(np.random.PCG64(2)), 4, 256, 64, 32)
    x = torch.from_numpy(case.x).cuda()
    s = torch.from_numpy(case.scales).cuda()
    pre = ops.preprocess_weight_q4f16(torch.from_numpy(case.w.view(np.int32)).cuda())
    out = torch.empty(4, 64, dtype=torch.float16, device="cuda")
    d = _desc(x, pre, s, out, 32)
    d.activation = 4  # RB200_ACT_SWIGLU
    with pytest.raises(relax_b200.RB200Error, match="gate/up"):
        _call(lib.rb200_gemm_fp16_intx_noalloc, d)
    for field in ("activation", "binary_op", "unary_op"):
        d = _desc(x, pre, s, out, 32)
        setattr(d, field, 9)
        with pytest.raises(relax_b200.RB200Error, match="unknown"):
            _call(lib.rb200_gemm_fp16_intx_noalloc, d)


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch(oracle):
    lib = _lib.load()
    case = synth.q4_case(np.random.Generator(np.random.PCG64(1)), 17, 256, 64, 32)
    x = torch.from_numpy(case.x).cuda()
    s = torch.from_numpy(case.scales).cuda()
    pre = ops.preprocess_weight_q4f16(torch.from_numpy(case.w.view(np.int32)).cuda())
    out = torch.empty(17, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(relax_b200.RB200Error, match="m <= 16"):
        _call(lib.rb200_gemm_fp16_intx_noalloc, _desc(x, pre, s, out, 32))
    d = _desc(x[:4], pre, s, out[:4], 32)
    d.n = 16 * 16385  # more row blocks than the array has tickets for
    with pytest.raises(relax_b200.RB200Error, match="fixed scratch"):
        _call(lib.rb200_gemm_fp16_intx_noalloc, d)
