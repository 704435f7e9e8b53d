"""GPU parity of the decode path (m <= 32) through the C ABI / PackedFunc surface:
repacked bytes against the layout statement, dequantised weights bit-exact against the oracle,
outputs within tolerance of the oracle (fp32 sequential accumulate, fp16 out)."""
import glob
import os

import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import ops, synth
from tests.layout_ref import fragment_layout
from tests.util import assert_close, bits16, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _check_status():
    import ctypes
    lib = relax_b200._lib.load()
    st = ctypes.c_int(0)
    assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0
    assert st.value == 0, "a bounded wait inside a kernel gave up (status %d)" % st.value


# ------------------------------------------------------------------ preprocess + decode
@pytest.mark.parametrize("n,k", [(16, 64), (48, 256), (128, 4096)])
def test_preprocess_q4_bytes(oracle, n, k):
    g = np.random.Generator(np.random.PCG64(n * 7 + k))
    codes = g.integers(0, 16, size=(n, k), dtype=np.uint8)
    w = synth.pack_q4_nk(codes)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(w))
    assert pre.shape == (n, k // 8) and pre.dtype == torch.int32
    got = pre.cpu().numpy().view(np.uint8).reshape(-1)
    assert np.array_equal(got, fragment_layout(codes, 4))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("experts", [1, 3])
def test_preprocess_ft_bytes(oracle, bits, experts):
    rs = np.random.RandomState(bits + experts)
    k, n = 128, 64
    shape = (experts, k, n // 2 if bits == 4 else n)
    a = rs.randint(-128, 128, size=shape).astype(np.int8)
    src = a if experts > 1 else a[0]
    pre = ops.preprocess_weight_ft(to_dev(src), bits == 4)
    assert pre.shape == src.shape and pre.dtype == torch.int8
    got = pre.cpu().numpy().view(np.uint8).reshape(experts, -1)
    for e in range(experts):
        v = oracle.np_unpack_ft_int4_kn(a[e]) if bits == 4 else a[e]
        u = (v.astype(np.int32) + (8 if bits == 4 else 128)).astype(np.uint8).T  # [N, K] biased codes
        assert np.array_equal(got[e], fragment_layout(np.ascontiguousarray(u), bits))


def test_preprocess_accepts_host_tensor_and_matches_device(oracle):
    rs = np.random.RandomState(5)
    a = rs.randint(-128, 128, size=(64, 32)).astype(np.int8)
    on_host = ops.preprocess_weight_ft(torch.from_numpy(a), True, 80)
    assert not on_host.is_cuda
    on_dev = ops.preprocess_weight_ft(to_dev(a), True, 80)
    assert torch.equal(on_host, on_dev.cpu())


def test_dequant_bit_exact_all_codes(oracle):
    f = np.load(os.path.join(GOLDEN, "q4_all_codes.npz"))
    g = int(f["group"])
    n, k = f["w"].shape[0], f["w"].shape[1] * 8
    pre = ops.preprocess_weight_q4f16(u32_to_dev(f["w"]))
    s = to_dev(f["scales"])
    wq = ops.dequantize(pre, s, n, k, 4, ops.LAYOUT_Q4_NK, None, g, 7.0)
    assert np.array_equal(bits16(wq), bits16(f["wq7"]))
    wq = ops.dequantize(pre, s, n, k, 4, ops.LAYOUT_Q4_NK, to_dev(f["zeros"]), g, 0.0)
    assert np.array_equal(bits16(wq), bits16(f["wqz"]))


@pytest.mark.parametrize("group,asym", [(32, False), (64, False), (128, True), (256, False), (16, True)])
def test_dequant_q4_bit_exact(oracle, group, asym):
    g = np.random.Generator(np.random.PCG64(group))
    case = synth.q4_case(g, 1, 512, 64, group, asymmetric=asym)
    if asym:
        case.zeros[1, 0] = np.float16(2.625)
    exp = oracle.C().decode_q4_nk(case.w, case.scales, case.zeros, 7.0, group)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    z = None if case.zeros is None else to_dev(case.zeros)
    wq = ops.dequantize(pre, to_dev(case.scales), 64, 512, 4, ops.LAYOUT_Q4_NK, z, group, 7.0)
    assert np.array_equal(bits16(wq), bits16(exp))


@pytest.mark.parametrize("bits,group", [(4, -1), (8, -1), (8, 64), (4, 64)])
def test_dequant_ft_bit_exact(oracle, bits, group):
    rs = np.random.RandomState(bits * 3 + max(group, 0))
    y = rs.normal(0, 0.002, size=(128, 128)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, group)
    exp_kn = oracle.C().decode_ft_kn(packed, scales, bits, group)
    pre = ops.preprocess_weight_ft(to_dev(packed), bits == 4)
    wq = ops.dequantize(pre, to_dev(scales), 128, 128, bits, ops.LAYOUT_FT_KN, None, group,
                        8.0 if bits == 4 else 128.0)
    assert np.array_equal(bits16(wq), bits16(np.ascontiguousarray(exp_kn.T)))


# ------------------------------------------------------------------ GEMV parity
def _run_q4(oracle, case, **epi):
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    z = None if case.zeros is None else to_dev(case.zeros)
    out = ops.gemm_fp16_q4f16(to_dev(case.x), pre, to_dev(case.scales), z, group_size=case.group,
                              zero_const=case.zero_const,
                              **{k: (to_dev(v) if isinstance(v, np.ndarray) else v) for k, v in epi.items()})
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq = C.decode_q4_nk(case.w, case.scales, case.zeros, case.zero_const, case.group)
    exp = C.epilogue(C.matmul_f32(case.x, wq), epi.get("bias"), epi.get("residual"),
                     epi.get("activation", "identity"), epi.get("binary_op", ""),
                     epi.get("unary_op", "identity"))
    return out.cpu().numpy(), exp


@pytest.mark.parametrize("m", [1, 2, 7, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("k,n", [(256, 128), (4096, 4096), (1024, 272), (320, 16)])
def test_gemv_q4_g32(oracle, m, k, n):
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m * 131 + k + n)), m, k, n, 32)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


def test_gemv_config0_full(oracle):
    """Configuration 0 exactly: x [1,4096], W uint32 [4096,512], scales [4096,128]."""
    case = synth.config0()
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


@pytest.mark.parametrize("group,asym", [(64, False), (128, False), (128, True), (512, False), (16, True), (96, False)])
def test_gemv_q4_groups_and_zero_points(oracle, group, asym):
    k = 1536
    case = synth.q4_case(np.random.Generator(np.random.PCG64(group)), 4, k, 144, group, asymmetric=asym)
    if asym:
        case.zeros[2, 1] = np.float16(5.5)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


def test_gemv_epilogues(oracle):
    rs = np.random.RandomState(3)
    case = synth.q4_case(np.random.Generator(np.random.PCG64(77)), 6, 512, 256, 32)
    bias = rs.randn(256).astype(np.float16)
    res = rs.randn(6, 256).astype(np.float16)
    for epi in [dict(bias=bias), dict(bias=bias, activation="relu"), dict(activation="silu"),
                dict(bias=bias, activation="gelu"),
                dict(bias=bias, residual=res, binary_op="plus"),
                dict(bias=bias, residual=res, activation="silu", binary_op="multiply", unary_op="relu"),
                dict(bias=rs.randn(6, 256).astype(np.float16))]:
        got, exp = _run_q4(oracle, case, **epi)
        assert_close(got, exp, tight=False)


@pytest.mark.parametrize("bits,group,m", [(4, -1, 3), (8, -1, 16), (8, 64, 5), (4, 64, 32), (8, 32, 1)])
def test_gemv_ft_layout(oracle, bits, group, m):
    """The reference tests' flow (test_codegen_cutlass.py:1355-1609): encode, ft_preprocess_weight,
    fused decode-matmul with bias; checked against the oracle and against the unquantised numpy
    product at the reference's own rtol = atol = 1e-2."""
    rs = np.random.RandomState(bits + m)
    k, n = 256, 128
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
    ref = np.dot(x.astype(np.float32), y.astype(np.float32).T) + bias.astype(np.float32)
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), ref, rtol=1e-2, atol=1e-2)


def test_gemv_int8_per_channel_llama70b_shard(oracle):
    """Configuration 3 shapes at 1/8 shard: gate_up columns, down rows (m = 16)."""
    for name in ("gate_up", "down"):
        case = synth.config3(name, 16, shard=(3, 8))
        pre = ops.preprocess_weight_ft(to_dev(case.w), False)
        out = ops.gemm_fp16_ft(to_dev(case.x), pre, to_dev(case.scales), 8)
        torch.cuda.synchronize()
        _check_status()
        C = oracle.C()
        exp = C.epilogue(C.matmul_f32(case.x, C.decode_ft_kn(case.w, case.scales, 8, -1), False))
        assert_close(out.cpu().numpy(), exp)


@pytest.mark.parametrize("name", sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "*.npz"))))
def test_gemv_against_golden(oracle, name):
    f = np.load(os.path.join(GOLDEN, name))
    if name.startswith("q4_all_codes"):
        pytest.skip("decode-only fixture")
    if name.startswith("q4_"):
        g = int(f["group"])
        z = to_dev(f["zeros"]) if f["zeros"].size else None
        pre = ops.preprocess_weight_q4f16(u32_to_dev(f["w"]))
        n, k = f["w"].shape[0], f["w"].shape[1] * 8
        assert np.array_equal(bits16(ops.dequantize(pre, to_dev(f["scales"]), n, k, 4, ops.LAYOUT_Q4_NK, z, g, 7.0)),
                              bits16(f["wq"]))
        out = ops.gemm_fp16_q4f16(to_dev(f["x"]), pre, to_dev(f["scales"]), z, group_size=g)
    else:
        bits, g = int(f["bits"]), int(f["group"])
        if f["x"].shape[0] > 32:
            pytest.skip("m > 32: covered by the tensor-core tests")
        pre = ops.preprocess_weight_ft(to_dev(f["packed"]), bits == 4)
        out = ops.gemm_fp16_ft(to_dev(f["x"]), pre, to_dev(f["scales"]), bits, bias=to_dev(f["bias"]), group_size=g)
    assert_close(out.cpu().numpy(), f["out"], tight=False)


def test_gemv_repeatable_and_scratch_self_resets(oracle):
    """Split-k tickets reset themselves: back-to-back launches give identical bits."""
    case = synth.q4_case(np.random.Generator(np.random.PCG64(3)), 8, 4096, 4096, 32)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    x, s = to_dev(case.x), to_dev(case.scales)
    outs = [ops.gemm_fp16_q4f16(x, pre, s).clone() for _ in range(4)]
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    _check_status()


def test_m_zero_and_bad_shapes_rejected(oracle):
    case = synth.q4_case(np.random.Generator(np.random.PCG64(4)), 1, 256, 64, 32)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    out = ops.gemm_fp16_q4f16(torch.zeros(0, 256, dtype=torch.float16, device="cuda"), pre, to_dev(case.scales))
    assert out.shape == (0, 64)
    with pytest.raises(relax_b200.RB200Error):
        ops.gemm_fp16_q4f16(torch.zeros(1, 128, dtype=torch.float16, device="cuda"), pre, to_dev(case.scales))
    with pytest.raises(relax_b200.RB200Error):
        ops.preprocess_weight_q4f16(torch.zeros(24, 8, dtype=torch.int32, device="cuda"))  # n % 16 != 0


@pytest.mark.parametrize("m,k,n,group,asym", [(33, 512, 256, 32, False), (100, 1024, 384, 128, True), (256, 512, 128, 32, False)])
def test_large_batch_q4(oracle, m, k, n, group, asym):
    """m > 32 (sliced over the batch): same parity bar as the decode path."""
    case = synth.q4_case(np.random.Generator(np.random.PCG64(m + k)), m, k, n, group, asymmetric=asym)
    rs = np.random.RandomState(m)
    bias = rs.randn(m, n).astype(np.float16)
    res = rs.randn(m, n).astype(np.float16)
    got, exp = _run_q4(oracle, case, bias=bias, residual=res, binary_op="plus", activation="relu")
    assert_close(got, exp, tight=False)


def test_reference_int4_test_flow_m64(oracle):
    """tests/python/relax/test_codegen_cutlass.py:1355-1609 with its own shapes (x 64x64, y 128x64):
    main_bias, main_cast_bias and main_residual against numpy at rtol = atol = 1e-2."""
    f = np.load(os.path.join(GOLDEN, "ft_int4_percol.npz"))
    x, y, bias = f["x"], f["y"], f["bias"]
    rs = np.random.RandomState(1)
    residual = rs.randn(64, 128).astype(np.float16)
    pre = ops.preprocess_weight_ft(to_dev(f["packed"]), True, 80)
    ref = np.dot(x.astype(np.float32), y.astype(np.float32).T) + bias.astype(np.float32)
    out = ops.gemm_fp16_ft(to_dev(x), pre, to_dev(f["scales"]), 4, bias=to_dev(bias))
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), ref, rtol=1e-2, atol=1e-2)
    assert_close(out.cpu().numpy(), f["out"], tight=False)
    out = ops.gemm_fp16_ft(to_dev(x), pre, to_dev(f["scales"]), 4, bias=to_dev(bias), residual=to_dev(residual),
                           binary_op="plus")
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), ref + residual.astype(np.float32),
                               rtol=1e-2, atol=1e-2)
