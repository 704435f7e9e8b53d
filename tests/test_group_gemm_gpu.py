"""GPU parity of the grouped (mixture-of-experts) matmul through the PackedFunc surface:
`cutlass.group_gemm_fp16_sm90` with the reference test's own sizes and tolerance
(tests/python/contrib/test_cutlass.py:1110-1162), and the quantised expert forms against the
oracle (decode per expert, sequential-fp32 grouped matmul)."""
import numpy as np
import pytest
import torch

from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


def _oracle_grouped(oracle, x, wq_enk, indptr):
    """fp16 result of the grouped matmul over decoded weights wq [E, N, K]."""
    C = oracle.C()
    return C.epilogue(C.group_gemm_f32(x, wq_enk, indptr))


def test_group_gemm_fp16_reference_test_sizes(oracle):
    """verify_group_gemm("cutlass.group_gemm_fp16_sm90", M=8, N=128, K=128, num_groups=4, ...,
    rtol=1e-3, atol=1e-3): equal groups of M / num_groups rows, numpy product as the expectation."""
    rs = np.random.RandomState(0)
    M, N, K, G = 8, 128, 128, 4
    a = rs.uniform(-1, 1, (M, K)).astype(np.float16)
    b = rs.uniform(-1, 1, (G, N, K)).astype(np.float16)
    per = M // G
    indptr = (np.arange(1, G + 1) * per).astype(np.int64)
    c = np.concatenate([a[i * per:(i + 1) * per].astype(np.float32) @ b[i].astype(np.float32).T for i in range(G)], axis=0)
    workspace = torch.empty(4096 * 1024, dtype=torch.uint8, device="cuda")
    out = ops.group_gemm_fp16(to_dev(a), to_dev(b), torch.from_numpy(indptr).cuda(), workspace)
    torch.cuda.synchronize()
    _check_status()
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), c, rtol=1e-3, atol=1e-3)
    assert_close(out.cpu().numpy(), _oracle_grouped(oracle, a, b, indptr))


@pytest.mark.parametrize("rows", [[0, 5, 1, 9], [300, 0, 0, 17], [64, 64, 64, 64], [1, 0, 0, 0], [0, 0, 0, 33]])
def test_group_gemm_fp16_ragged_and_empty_groups(oracle, rows):
    rs = np.random.RandomState(sum(rows))
    E, N, K = len(rows), 256, 192
    indptr = np.cumsum(rows).astype(np.int64)
    x = rs.randn(sum(rows), K).astype(np.float16)
    w = (rs.randn(E, N, K) * 0.05).astype(np.float16)
    out = ops.group_gemm_fp16(to_dev(x), to_dev(w), torch.from_numpy(indptr).cuda())
    torch.cuda.synchronize()
    _check_status()
    assert_close(out.cpu().numpy(), _oracle_grouped(oracle, x, w, indptr))


@pytest.mark.parametrize("bits,group", [(4, 128), (4, 64), (4, -1), (8, -1), (8, 64)])
def test_moe_gemm_ft_layout(oracle, bits, group):
    """Experts in the FT layout (int8 [E, K, N/2] or [E, K, N]), ragged rows incl. an empty expert."""
    g = np.random.Generator(np.random.PCG64(bits * 100 + max(group, 0)))
    E, K, N = 4, 256, 256
    rows = [37, 0, 130, 3]
    indptr = np.cumsum(rows).astype(np.int64)
    x = g.standard_normal((sum(rows), K), dtype=np.float32).astype(np.float16)
    w = g.integers(-128, 128, size=(E, K, N // 2 if bits == 4 else N), dtype=np.int8)
    kg = 1 if group <= 0 else K // group
    scales = g.uniform(0.001, 0.01, size=(E, kg, N) if group > 0 else (E, N)).astype(np.float16)
    pre = ops.preprocess_weight_ft(to_dev(w), bits == 4)
    out = ops.moe_gemm_ft(to_dev(x), pre, to_dev(scales), torch.from_numpy(indptr).cuda())
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq = np.stack([np.ascontiguousarray(C.decode_ft_kn(w[e], scales[e], bits, group).T) for e in range(E)])
    assert_close(out.cpu().numpy(), _oracle_grouped(oracle, x, wq, indptr))


@pytest.mark.parametrize("group,asym", [(32, False), (128, True)])
def test_moe_gemm_q4f16_layout(oracle, group, asym):
    g = np.random.Generator(np.random.PCG64(group))
    E, K, N = 3, 512, 128
    rows = [70, 5, 260]
    indptr = np.cumsum(rows).astype(np.int64)
    cases = [synth.q4_case(g, 1, K, N, group, asymmetric=asym) for _ in range(E)]
    x = g.standard_normal((sum(rows), K), dtype=np.float32).astype(np.float16)
    w = np.stack([c.w for c in cases])
    s = np.stack([c.scales for c in cases])
    z = np.stack([c.zeros for c in cases]) if asym else None
    pre = ops.preprocess_weight_q4f16(u32_to_dev(w))
    out = ops.moe_gemm_q4f16(to_dev(x), pre, to_dev(s), torch.from_numpy(indptr).cuda(),
                             zeros=None if z is None else to_dev(z), group_size=group)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq = np.stack([C.decode_q4_nk(cases[e].w, cases[e].scales, cases[e].zeros, 7.0, group) for e in range(E)])
    assert_close(out.cpu().numpy(), _oracle_grouped(oracle, x, wq, indptr))


@pytest.mark.parametrize("bits,group,rows", [
    (4, 128, [1, 0, 1, 0, 0, 2, 0, 0]),     # two tokens, top-2 of eight experts
    (4, -1, [0, 0, 0, 0, 0, 0, 0, 1]),
    (8, 64, [3, 9, 0, 5]),
    (4, 64, [8, 8, 8, 8]),                  # exactly 32 rows: still the decode-size path
    (8, -1, [0, 31, 0, 1]),
])
def test_moe_gemm_decode_size_batches(oracle, bits, group, rows):
    """At most 32 rows in all: every expert with rows is one launch of the decode kernel over
    its own weights (rows taken from indptr on the device); experts without rows launch and
    return.  Same oracle as the large-batch form."""
    g = np.random.Generator(np.random.PCG64(bits * 1000 + max(group, 0) + sum(rows)))
    E, K, N = len(rows), 512, 384
    indptr = np.cumsum(rows).astype(np.int64)
    x = g.standard_normal((sum(rows), K), dtype=np.float32).astype(np.float16)
    w = g.integers(-128, 128, size=(E, K, N // 2 if bits == 4 else N), dtype=np.int8)
    kg = 1 if group <= 0 else K // group
    scales = g.uniform(0.001, 0.01, size=(E, kg, N) if group > 0 else (E, N)).astype(np.float16)
    pre = ops.preprocess_weight_ft(to_dev(w), bits == 4)
    out = torch.full((sum(rows), N), float("nan"), dtype=torch.float16, device="cuda")
    ops.moe_gemm_ft(to_dev(x), pre, to_dev(scales), torch.from_numpy(indptr).cuda(), out=out)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq = np.stack([np.ascontiguousarray(C.decode_ft_kn(w[e], scales[e], bits, group).T) for e in range(E)])
    assert_close(out.cpu().numpy(), _oracle_grouped(oracle, x, wq, indptr))


def test_moe_gemm_decode_size_expert_sub_range(oracle):
    """A rank that owns experts [2, 4) of a longer routing table passes indptr + 2 with
    indptr_has_prev: its first expert starts at indptr[1], not at row 0."""
    g = np.random.Generator(np.random.PCG64(77))
    E, K, N = 4, 256, 256
    rows = [2, 1, 3, 2]
    indptr = np.cumsum(rows).astype(np.int64)
    x = g.standard_normal((sum(rows), K), dtype=np.float32).astype(np.float16)
    w = g.integers(-128, 128, size=(E, K, N // 2), dtype=np.int8)
    scales = g.uniform(0.001, 0.01, size=(E, N)).astype(np.float16)
    pre = ops.preprocess_weight_ft(to_dev(w), True)
    out = torch.zeros((sum(rows), N), dtype=torch.float16, device="cuda")
    ops.moe_gemm_ft(to_dev(x), pre[2:], to_dev(scales[2:]), torch.from_numpy(indptr).cuda(), out=out, first_expert=2)
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    wq = np.stack([np.ascontiguousarray(C.decode_ft_kn(w[e], scales[e], 4, -1).T) for e in range(E)])
    exp = _oracle_grouped(oracle, x, wq, indptr)
    got = out.cpu().numpy()
    assert_close(got[3:], exp[3:])
    assert not got[:3].any()  # rows of the experts this rank does not own are left alone
