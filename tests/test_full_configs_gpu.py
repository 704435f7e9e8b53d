"""The benchmark configurations at their full sizes, every one checked against the CPU oracle
(decode in fp16 ops, sequential fp32 accumulation, one rounding) - never against another kernel
of the library.  Where the full output would cost the oracle minutes, a sample of output rows /
columns is compared; the GPU always computes the whole problem."""
import numpy as np
import pytest
import torch

from relax_b200 import ops, synth
from tests.test_gemv_gpu import _check_status, _run_q4
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ configuration 1: all 12 (linear, M) pairs
@pytest.mark.parametrize("m", [1, 8, 32])
@pytest.mark.parametrize("name", [l[0] for l in synth.LLAMA7B_LINEARS])
def test_config1_every_linear_and_batch(oracle, name, m):
    case = synth.config1(name, m)
    got, exp = _run_q4(oracle, case)
    assert_close(got, exp)


# ------------------------------------------------------------------ configuration 2: full prefill shape
def test_config2_full_size_rows_against_oracle(oracle):
    """m 2048, k 4096, n 22016, group 128 with zero points: 24 batch rows x all 22016 columns of the
    tensor-core kernel's output against decode + sequential-fp32 matmul on those rows."""
    case = synth.config2()
    pre = ops.preprocess_weight_q4f16(u32_to_dev(case.w))
    out = ops.gemm_fp16_q4f16(to_dev(case.x), pre, to_dev(case.scales), to_dev(case.zeros), group_size=128)
    torch.cuda.synchronize()
    _check_status()
    rows = np.array([0, 1, 31, 32, 255, 256, 257, 511, 777, 1023, 1024, 1500, 1791, 1792, 2000, 2047,
                     100, 200, 300, 400, 500, 600, 700, 800])
    C = oracle.C()
    wq = C.decode_q4_nk(case.w, case.scales, case.zeros, 7.0, 128)
    exp = C.epilogue(C.matmul_f32(case.x[rows], wq))
    assert_close(out[torch.from_numpy(rows).cuda()].cpu().numpy(), exp)
    assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------ configuration 3: Llama-70B MLP, int8 per channel
@pytest.fixture(scope="module")
def c3_weights():
    """The unsharded int8 weights (gate_up 470 MB, down 235 MB) and their scales, drawn once."""
    g = synth.rng(3, 77)
    out = {}
    for name, k, n, axis in synth.LLAMA70B_MLP:
        w = g.integers(-127, 128, size=(k, n), dtype=np.int8)
        s = g.uniform(1e-4, 1e-3, size=(n,)).astype(np.float16)
        out[name] = (w, s, axis)
    return out


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("name", ["gate_up", "down"])
def test_config3_unsharded_and_rank0_shards(oracle, c3_weights, name, world):
    """gate_up (k 8192, n 57344) column-parallel and down (k 28672, n 8192) row-parallel: the
    unsharded layer and rank 0's shard at 2 / 4 / 8 ranks, m = 16 / 256 / 4096; a sample of 256
    output columns (and 256 batch rows at m = 4096) against the oracle on the same slice."""
    w, s, axis = c3_weights[name]
    k, n = w.shape
    if axis == "n":
        wl, sl, kl, nl = np.ascontiguousarray(w[:, :n // world]), s[:n // world].copy(), k, n // world
    else:
        wl, sl, kl, nl = np.ascontiguousarray(w[:k // world]), s, k // world, n
    pre = ops.preprocess_weight_ft(to_dev(wl), False)
    sd = to_dev(sl)
    g = synth.rng(3, 1000 + world)
    cols = np.sort(g.choice(nl, size=256, replace=False))
    C = oracle.C()
    wq_cols = C.decode_ft_kn(np.ascontiguousarray(wl[:, cols]), sl[cols].copy(), 8, -1)  # [kl, 256]
    for m in (16, 256, 4096):
        x = g.standard_normal((m, kl), dtype=np.float32).astype(np.float16)
        out = ops.gemm_fp16_ft(to_dev(x), pre, sd, 8)
        torch.cuda.synchronize()
        _check_status()
        rows = np.arange(m) if m <= 256 else np.sort(g.choice(m, size=256, replace=False))
        exp = C.epilogue(C.matmul_f32(x[rows], wq_cols, False))
        got = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
        assert_close(got, exp)
        del out


# ------------------------------------------------------------------ configuration 4: Mixtral expert layer, full width
def test_config4_full_ffn_width_against_oracle(oracle):
    """512 tokens, top-2 of 8 experts, hidden 4096, expert FFN 14336, W4 group 128: the grouped
    kernel's output on up to 6 rows of every expert x all 14336 columns against the oracle's
    per-expert decode + sequential-fp32 matmul."""
    case = synth.config4()
    pre = ops.preprocess_weight_ft(to_dev(case.w), True)
    out = ops.moe_gemm_ft(to_dev(case.x), pre, to_dev(case.scales), torch.from_numpy(case.indptr).cuda())
    torch.cuda.synchronize()
    _check_status()
    C = oracle.C()
    r0 = 0
    for e in range(case.w.shape[0]):
        r1 = int(case.indptr[e])
        if r1 > r0:
            rows = np.unique(np.clip(np.array([r0, r0 + 1, (r0 + r1) // 2, r1 - 2, r1 - 1, r0 + 37]), r0, r1 - 1))
            wq = C.decode_ft_kn(case.w[e], case.scales[e], 4, case.group)  # [K, N]
            exp = C.epilogue(C.matmul_f32(case.x[rows], wq, False))
            assert_close(out[torch.from_numpy(rows).cuda()].cpu().numpy(), exp)
        r0 = r1
    assert int(case.indptr[-1]) == case.x.shape[0]
