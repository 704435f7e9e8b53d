"""CPU checks that pin the oracle: half-precision conversion against the reference's own
converters (oracle/_ref, when built), the C restatement against the numpy restatement and the
committed fixtures, and the reference tests' pass criterion (rtol = atol = 1e-2 against numpy,
tests/python/relax/test_codegen_cutlass.py:1609,1755,2023,2180)."""
import glob
import os

import numpy as np
import pytest

from relax_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float16).view(np.uint16)


def test_f16_conversion_matches_numpy_everywhere(oracle):
    C = oracle.C()
    allh = np.arange(65536, dtype=np.uint16)
    f = allh.view(np.float16).astype(np.float32)
    got = np.array([C.lib.orc_f16_to_f32(int(h)) for h in allh[::7]], dtype=np.float32)
    exp = f[::7]
    assert np.array_equal(got.view(np.uint32)[~np.isnan(exp)], exp.view(np.uint32)[~np.isnan(exp)])
    rs = np.random.RandomState(1)
    vals = np.concatenate([
        rs.randn(4000).astype(np.float32), (rs.randn(2000) * 1e-5).astype(np.float32),
        (rs.randn(2000) * 6e-8).astype(np.float32), (rs.randn(500) * 7e4).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.98e-8, 2.9802322e-8, np.inf, -np.inf],
                 dtype=np.float32),
        # exact ties between adjacent halves
        ((np.arange(1024, 1124).astype(np.float32) + 0.5) / 1024.0).astype(np.float32)])
    got = np.array([C.lib.orc_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    with np.errstate(over="ignore"):
        exp = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, exp)
    dv = vals.astype(np.float64) * 1.0000001
    got = np.array([C.lib.orc_f64_to_f16(float(v)) for v in dv], dtype=np.uint16)
    with np.errstate(over="ignore"):
        exp = dv.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, exp)


def test_f16_conversion_matches_reference_converters(oracle):
    ref = oracle.ref_fp16()
    if ref is None:
        pytest.skip("oracle/_ref was not built (reference tree absent at build time)")
    C = oracle.C()
    rs = np.random.RandomState(2)
    vals = np.concatenate([rs.randn(5000), rs.randn(3000) * 1e-5, rs.randn(3000) * 6e-8,
                           rs.randn(500) * 7e4, [0.0, 65504.0, 65520.0, 2.9802322e-8]]).astype(np.float32)
    for v in vals:
        assert C.lib.orc_f32_to_f16(float(v)) == ref.ref_f32_to_f16(float(v)), v
        assert C.lib.orc_f64_to_f16(float(v) * 1.0000001) == ref.ref_f64_to_f16(float(v) * 1.0000001), v
    for h in range(0, 65536, 5):
        a, b = C.lib.orc_f16_to_f32(h), ref.ref_f16_to_f32(h)
        assert (a != a and b != b) or a == b


@pytest.mark.parametrize("group,asym", [(32, False), (128, True), (64, True)])
def test_c_decode_q4_matches_numpy(oracle, group, asym):
    g = np.random.Generator(np.random.PCG64(5))
    case = synth.q4_case(g, 2, 512, 48, group, asymmetric=asym)
    if asym:
        case.zeros[3, 1] = np.float16(1.75)
    got = oracle.C().decode_q4_nk(case.w, case.scales, case.zeros, 7.0, group)
    exp = oracle.np_decode_q4_nk(case.w, case.scales, case.zeros, 7.0, group)
    assert np.array_equal(_bits(got), _bits(exp))


@pytest.mark.parametrize("bits,group", [(4, -1), (8, -1), (8, 64), (4, 64)])
def test_c_decode_ft_matches_numpy(oracle, bits, group):
    rs = np.random.RandomState(3)
    y = rs.normal(0, 0.002, size=(128, 128)).astype(np.float16)
    packed, scales = oracle.np_encode_ft(y, bits, group)
    got = oracle.C().decode_ft_kn(packed, scales, bits, group)
    exp = oracle.np_decode_ft_kn(packed, scales, bits, group)
    assert np.array_equal(_bits(got), _bits(exp))


def test_decode_codes_is_the_common_form(oracle):
    """(u - z) * s over unpacked codes equals each layout-specific decode."""
    g = np.random.Generator(np.random.PCG64(6))
    case = synth.q4_case(g, 1, 256, 32, 32)
    codes = oracle.np_unpack_q4_nk(case.w)
    a = oracle.C().decode_codes(codes, case.scales, None, 7.0, 32, 256 // 32, 1)
    b = oracle.C().decode_q4_nk(case.w, case.scales, None, 7.0, 32)
    assert np.array_equal(_bits(a), _bits(b))
    rs = np.random.RandomState(4)
    A = rs.randint(-128, 128, size=(64, 32)).astype(np.int8)   # [K, N/2] int4 pairs
    B = rs.uniform(0.001, 0.01, size=(64,)).astype(np.float16)
    v = oracle.np_unpack_ft_int4_kn(A)                          # [K, N] signed
    u = (v.astype(np.int32) + 8).astype(np.uint8).T             # [N, K] biased codes
    a = oracle.C().decode_codes(np.ascontiguousarray(u), B, None, 8.0, 64, 1, 0)
    b = oracle.C().decode_ft_kn(A, B, 4, -1)
    assert np.array_equal(_bits(a), _bits(b.T))


def test_autogptq_decode_equals_common_form(oracle):
    """tests/python/dlight/test_gpu_gemv.py:639-649: z = zq + 1 per (group, n)."""
    rs = np.random.RandomState(8)
    K, N, G = 256, 64, 2
    q = rs.randint(0, 16, size=(K, N)).astype(np.uint8)
    zq = rs.randint(0, 15, size=(G, N)).astype(np.uint8)
    S = rs.uniform(0.001, 0.01, size=(G, N)).astype(np.float16)
    Wq = np.bitwise_or.reduce(q.reshape(K // 8, 8, N).astype(np.uint32) <<
                              (np.arange(8, dtype=np.uint32) * 4)[None, :, None], axis=1)
    Zq = np.bitwise_or.reduce(zq.reshape(G, N // 8, 8).astype(np.uint32) <<
                              (np.arange(8, dtype=np.uint32) * 4)[None, None, :], axis=2)
    g_idx = (np.arange(K) // (K // G)).astype(np.uint32)
    got = oracle.C().decode_autogptq(Wq, Zq, S, g_idx)                        # [K, N]
    z = (zq.astype(np.float16) + np.float16(1)).T                            # [N, G]
    exp = oracle.C().decode_codes(np.ascontiguousarray(q.T), np.ascontiguousarray(S.T),
                                  np.ascontiguousarray(z), 0.0, K // G, G, 1)
    assert np.array_equal(_bits(got.T), _bits(exp))


def test_matmul_and_epilogue(oracle):
    rs = np.random.RandomState(9)
    x = rs.randn(5, 96).astype(np.float16)
    w = (rs.randn(24, 96) * 0.05).astype(np.float16)
    acc = oracle.C().matmul_f32(x, w, True)
    acc2 = oracle.C().matmul_f32(x, np.ascontiguousarray(w.T), False)
    assert np.array_equal(acc, acc2)
    # sequential fp32 order, restated with a python loop on one element
    s = np.float32(0)
    for k in range(96):
        s = np.float32(s + np.float32(x[2, k]) * np.float32(w[7, k]))
    assert acc[2, 7] == s
    np.testing.assert_allclose(acc, x.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-5, atol=1e-5)
    bias = rs.randn(24).astype(np.float16)
    res = rs.randn(5, 24).astype(np.float16)
    out = oracle.C().epilogue(acc, bias, res, "relu", "multiply", "relu")
    exp = np.maximum(np.maximum(acc + bias.astype(np.float32), 0) * res.astype(np.float32), 0)
    assert np.array_equal(_bits(out), _bits(exp.astype(np.float16)))
    out = oracle.C().epilogue(acc, bias, None, "silu")
    v = acc + bias.astype(np.float32)
    np.testing.assert_allclose(out.astype(np.float32), v / (1 + np.exp(-v)), rtol=2e-3, atol=1e-3)
    from scipy.special import erf
    out = oracle.C().epilogue(acc, None, None, "gelu")
    np.testing.assert_allclose(out.astype(np.float32), 0.5 * acc * (1 + erf(acc / np.sqrt(2))),
                               rtol=2e-3, atol=1e-3)


def test_group_gemm(oracle):
    rs = np.random.RandomState(10)
    E, N, K = 4, 32, 64
    rows = [0, 5, 1, 9]           # an empty group and ragged sizes
    indptr = np.cumsum(rows).astype(np.int64)
    x = rs.randn(sum(rows), K).astype(np.float16)
    w = (rs.randn(E, N, K) * 0.05).astype(np.float16)
    acc = oracle.C().group_gemm_f32(x, w, indptr)
    r0 = 0
    for e in range(E):
        r1 = int(indptr[e])
        if r1 > r0:
            np.testing.assert_allclose(acc[r0:r1], x[r0:r1].astype(np.float32) @ w[e].astype(np.float32).T,
                                       rtol=1e-5, atol=1e-5)
        r0 = r1


@pytest.mark.parametrize("name", sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "*.npz"))))
def test_c_oracle_reproduces_golden(oracle, name):
    f = np.load(os.path.join(GOLDEN, name))
    C = oracle.C()
    if name.startswith("q4_all_codes"):
        g = int(f["group"])
        assert np.array_equal(_bits(C.decode_q4_nk(f["w"], f["scales"], None, 7.0, g)), _bits(f["wq7"]))
        assert np.array_equal(_bits(C.decode_q4_nk(f["w"], f["scales"], f["zeros"], 0.0, g)), _bits(f["wqz"]))
    elif name.startswith("q4_"):
        g = int(f["group"])
        z = f["zeros"] if f["zeros"].size else None
        wq = C.decode_q4_nk(f["w"], f["scales"], z, 7.0, g)
        assert np.array_equal(_bits(wq), _bits(f["wq"]))
        out = C.epilogue(C.matmul_f32(f["x"], wq))
        np.testing.assert_allclose(out.astype(np.float32), f["out"].astype(np.float32), rtol=2e-3, atol=2e-3)
    else:
        bits, g = int(f["bits"]), int(f["group"])
        wq = C.decode_ft_kn(f["packed"], f["scales"], bits, g)
        assert np.array_equal(_bits(wq), _bits(f["wq_kn"]))
        out = C.epilogue(C.matmul_f32(f["x"], wq, False), f["bias"])
        np.testing.assert_allclose(out.astype(np.float32), f["out"].astype(np.float32), rtol=2e-3, atol=2e-3)
        # the reference tests' own criterion: the quantised result against the unquantised numpy product
        ref = np.dot(f["x"].astype(np.float32), f["y"].astype(np.float32).T) + f["bias"].astype(np.float32)
        np.testing.assert_allclose(out.astype(np.float32), ref, rtol=1e-2, atol=1e-2)


def test_layout_reference_roundtrip():
    """The fragment layout is a permutation: every code appears exactly once."""
    from tests.layout_ref import fragment_layout
    rs = np.random.RandomState(12)
    codes = rs.randint(0, 16, size=(32, 128)).astype(np.uint8)
    lay = fragment_layout(codes, 4)
    assert lay.size == 32 * 128 // 2
    assert np.bincount(np.concatenate([lay & 15, lay >> 4]), minlength=16).tolist() == \
        np.bincount(codes.reshape(-1), minlength=16).tolist()
    codes8 = rs.randint(0, 256, size=(16, 64)).astype(np.uint8)
    lay8 = fragment_layout(codes8, 8)
    assert sorted(lay8.tolist()) == sorted(codes8.reshape(-1).tolist())


def test_moe_route_restatement_invariants(oracle):
    """np_moe_route: rows sorted by expert with ties broken by assignment order, indptr = end rows,
    row_of_flat the inverse permutation, gates = the chosen softmax probabilities."""
    g = np.random.Generator(np.random.PCG64(12))
    t, e, k = 50, 8, 2
    logits = g.standard_normal((t, e), dtype=np.float32)
    logits[7] = 0.0  # all experts tie: the two lowest indices win
    indptr, token_of_row, gate_of_row, row_of_flat = oracle.np_moe_route(logits, k)
    assert indptr[-1] == t * k and np.all(np.diff(np.concatenate([[0], indptr])) >= 0)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    r0 = 0
    for ex in range(e):
        rows = np.arange(r0, indptr[ex])
        # every row of the block belongs to a token that has `ex` among its top-k
        for r in rows:
            tok = token_of_row[r]
            assert ex in np.argsort(-p[tok], kind="stable")[:k]
            assert abs(gate_of_row[r] - p[tok, ex]) < 1e-7
        assert np.all(np.diff(token_of_row[rows]) >= 0)  # stable: token order kept inside an expert
        r0 = indptr[ex]
    assert sorted(row_of_flat.tolist()) == list(range(t * k))
    assert set(token_of_row[row_of_flat[7 * k:7 * k + k]].tolist()) == {7}
    experts_of_7 = [int(np.searchsorted(indptr, r, side="right")) for r in row_of_flat[7 * k:7 * k + k]]
    assert experts_of_7 == [0, 1]
