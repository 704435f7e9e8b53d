"""CUDA-graph replay of a single split-k decode launch.  The kernel's split-k flags must come
back to rest inside every launch: a replay whose flags still showed the previous replay's state
would add stale partial sums.  One launch of a shape that takes the stream-k kernel (n > 4096) is
captured alone and replayed with the activations rewritten between replays; every replay must
equal the eager result for the same activations bit for bit."""
import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status
from tests.util import to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 12288), (16, 4096, 12288), (32, 2048, 8192), (4, 11008, 4096)])
def test_single_launch_graph_replays_with_new_activations(m, k, n, overlap):
    g = np.random.Generator(np.random.PCG64(m + n))
    case = synth.q4_case(g, m, k, n, 32)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    s = to_dev(case.scales)
    xs = [to_dev(g.standard_normal((m, k), dtype=np.float32).astype(np.float16)) for _ in range(4)]
    eager = [ops.gemm_fp16_q4f16(x, pre, s).clone() for x in xs]
    torch.cuda.synchronize()
    relax_b200.set_launch_overlap(overlap)
    try:
        x_buf = xs[0].clone()
        out = torch.empty(m, n, dtype=torch.float16, device="cuda")
        ops.gemm_fp16_q4f16(x_buf, pre, s, out=out)  # warm-up outside the capture (scratch exists)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ops.gemm_fp16_q4f16(x_buf, pre, s, out=out)
        for rep in range(12):
            i = rep % len(xs)
            x_buf.copy_(xs[i])
            out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, eager[i]), "replay %d differs from the eager result" % rep
        _check_status()
    finally:
        relax_b200.set_launch_overlap(False)
