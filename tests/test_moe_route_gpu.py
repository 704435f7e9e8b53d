"""Routing front-end and combine around the grouped matmul, against the numpy restatement, and a
whole expert layer (route -> gather -> grouped decode-matmul -> combine) against the oracle."""
import numpy as np
import pytest
import torch

from relax_b200 import ops
from tests.test_gemv_gpu import _check_status
from tests.util import assert_close, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 8, 2), (37, 8, 2), (512, 8, 2), (300, 64, 8), (1000, 4, 1), (5, 40, 3)])
def test_route_matches_restatement(oracle, tokens, experts, top_k):
    g = np.random.Generator(np.random.PCG64(tokens + experts))
    logits = g.standard_normal((tokens, experts), dtype=np.float32)
    indptr, token_of_row, gate_of_row, row_of_flat = ops.moe_route(to_dev(logits), top_k)
    torch.cuda.synchronize()
    e_indptr, e_tok, e_gate, e_rof = oracle.np_moe_route(logits, top_k)
    assert np.array_equal(indptr.cpu().numpy(), e_indptr)
    assert np.array_equal(token_of_row.cpu().numpy(), e_tok)
    assert np.array_equal(row_of_flat.cpu().numpy(), e_rof)
    np.testing.assert_allclose(gate_of_row.cpu().numpy(), e_gate, rtol=2e-6, atol=1e-8)


def test_ties_go_to_the_lower_expert():
    logits = np.zeros((3, 8), dtype=np.float32)
    logits[1, 5] = 1.0
    indptr, token_of_row, gate_of_row, row_of_flat = ops.moe_route(to_dev(logits), 2)
    torch.cuda.synchronize()
    # token 0 and 2: experts 0, 1; token 1: experts 5, 0
    assert indptr.cpu().tolist() == [3, 5, 5, 5, 5, 6, 6, 6]
    assert token_of_row.cpu().tolist() == [0, 1, 2, 0, 2, 1]


def test_gather_and_combine(oracle):
    g = np.random.Generator(np.random.PCG64(3))
    tokens, experts, top_k, k, n = 129, 8, 2, 256, 384
    logits = g.standard_normal((tokens, experts), dtype=np.float32)
    x = g.standard_normal((tokens, k), dtype=np.float32).astype(np.float16)
    indptr, token_of_row, gate_of_row, row_of_flat = ops.moe_route(to_dev(logits), top_k)
    xg = ops.moe_gather(to_dev(x), token_of_row)
    assert np.array_equal(xg.cpu().numpy(), x[token_of_row.cpu().numpy()])
    y = g.standard_normal((tokens * top_k, n), dtype=np.float32).astype(np.float16)
    out = ops.moe_combine(to_dev(y), row_of_flat, gate_of_row, top_k)
    torch.cuda.synchronize()
    rof = row_of_flat.cpu().numpy().reshape(tokens, top_k)
    gate = gate_of_row.cpu().numpy()
    acc = np.zeros((tokens, n), dtype=np.float32)
    for j in range(top_k):
        acc = acc + gate[rof[:, j]][:, None] * y[rof[:, j]].astype(np.float32)
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), acc, rtol=2e-3, atol=1e-3)


def test_expert_layer_end_to_end(oracle):
    """route -> gather -> grouped int4 decode-matmul -> combine on a small Mixtral-shaped layer."""
    g = np.random.Generator(np.random.PCG64(11))
    tokens, experts, top_k, k, n, group = 96, 8, 2, 256, 256, 128
    logits = g.standard_normal((tokens, experts), dtype=np.float32)
    x = g.standard_normal((tokens, k), dtype=np.float32).astype(np.float16)
    w = g.integers(-128, 128, size=(experts, k, n // 2), dtype=np.int8)
    scales = g.uniform(0.001, 0.01, size=(experts, k // group, n)).astype(np.float16)
    indptr, token_of_row, gate_of_row, row_of_flat = ops.moe_route(to_dev(logits), top_k)
    xg = ops.moe_gather(to_dev(x), token_of_row)
    y = ops.moe_gemm_ft(xg, ops.preprocess_weight_ft(to_dev(w), True), to_dev(scales), indptr)
    out = ops.moe_combine(y, row_of_flat, gate_of_row, top_k)
    torch.cuda.synchronize()
    C = oracle.C()
    e_indptr, e_tok, e_gate, e_rof = oracle.np_moe_route(logits, top_k)
    wq = np.stack([np.ascontiguousarray(C.decode_ft_kn(w[e], scales[e], 4, group).T) for e in range(experts)])
    y_ref = C.epilogue(C.group_gemm_f32(x[e_tok], wq, e_indptr)).astype(np.float32)
    rof = e_rof.reshape(tokens, top_k)
    acc = np.zeros((tokens, n), dtype=np.float32)
    for j in range(top_k):
        acc = acc + e_gate[rof[:, j]][:, None] * y_ref[rof[:, j]]
    assert_close(out.cpu().numpy(), acc.astype(np.float16), tight=False)


def test_expert_layer_with_caller_buffers_replays_from_a_graph():
    """The same layer with every output and the routing workspace supplied by the caller: nothing
    allocates inside it, so it can be captured once and replayed; the replay on new logits and
    activations must equal the eager, allocating form bit for bit."""
    g = np.random.Generator(np.random.PCG64(12))
    tokens, experts, top_k, k, n, group = 64, 8, 2, 256, 256, 128
    w = g.integers(-128, 128, size=(experts, k, n // 2), dtype=np.int8)
    scales = g.uniform(0.001, 0.01, size=(experts, k // group, n)).astype(np.float16)
    pre, sd = ops.preprocess_weight_ft(to_dev(w), True), to_dev(scales)
    logits = torch.zeros((tokens, experts), dtype=torch.float32, device="cuda")
    x = torch.zeros((tokens, k), dtype=torch.float16, device="cuda")
    rows = tokens * top_k
    route = (torch.empty(experts, dtype=torch.int64, device="cuda"), torch.empty(rows, dtype=torch.int32, device="cuda"),
             torch.empty(rows, dtype=torch.float32, device="cuda"), torch.empty(rows, dtype=torch.int32, device="cuda"))
    ws = torch.empty(ops.moe_route_workspace_bytes(tokens, top_k), dtype=torch.uint8, device="cuda")
    xg = torch.empty((rows, k), dtype=torch.float16, device="cuda")
    y = torch.empty((rows, n), dtype=torch.float16, device="cuda")
    out = torch.empty((tokens, n), dtype=torch.float16, device="cuda")

    def layer():
        indptr, tok, gate, rof = ops.moe_route(logits, top_k, out=route, workspace=ws)
        ops.moe_gather(x, tok, out=xg)
        ops.moe_gemm_ft(xg, pre, sd, indptr, out=y)
        ops.moe_combine(y, rof, gate, top_k, out=out)

    layer()  # first call outside the capture (library scratch)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer()
    for seed in (1, 2):
        gg = np.random.Generator(np.random.PCG64(100 + seed))
        logits.copy_(to_dev(gg.standard_normal((tokens, experts), dtype=np.float32)))
        x.copy_(to_dev(gg.standard_normal((tokens, k), dtype=np.float32).astype(np.float16)))
        graph.replay()
        torch.cuda.synchronize()
        indptr, tok, gate, rof = ops.moe_route(logits, top_k)
        exp = ops.moe_combine(ops.moe_gemm_ft(ops.moe_gather(x, tok), pre, sd, indptr), rof, gate, top_k)
        torch.cuda.synchronize()
        assert torch.equal(out, exp)
    _check_status()
