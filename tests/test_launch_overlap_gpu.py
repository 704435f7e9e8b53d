"""Launch overlap (programmatic dependent launch) keeps results identical: a chain of dependent
decode matmuls - each consumes the previous one's output - gives bit-identical results with the
switch on and off, eagerly and from a CUDA graph."""
import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status
from tests.util import to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


def _chain(layers, x):
    for pre, sc in layers:
        x = ops.gemm_fp16_q4f16(x, pre, sc)
    return x


@pytest.mark.parametrize("m", [1, 8, 32])
def test_dependent_chain_is_bit_identical(m):
    g = np.random.Generator(np.random.PCG64(m))
    dims = [(1024, 4096), (4096, 8192), (8192, 1024), (1024, 4096), (4096, 1024)]  # (k, n): both decode kernels
    layers = []
    for k, n in dims:
        c = synth.q4_case(g, 1, k, n, 32)
        layers.append((ops.preprocess_weight_q4f16(u32_to_dev(c.w)), to_dev(c.scales)))
    x = to_dev(g.standard_normal((m, dims[0][0]), dtype=np.float32).astype(np.float16))
    torch.cuda.synchronize()
    assert not relax_b200.get_launch_overlap()
    ref = _chain(layers, x).clone()
    torch.cuda.synchronize()
    relax_b200.set_launch_overlap(True)
    try:
        for _ in range(5):
            got = _chain(layers, x)
        torch.cuda.synchronize()
        _check_status()
        assert torch.equal(got, ref)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = _chain(layers, x)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        _check_status()
        assert torch.equal(out, ref)
    finally:
        relax_b200.set_launch_overlap(False)
