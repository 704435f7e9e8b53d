"""Row-parallel decode matmul with the all-reduce fused into its epilogue
(`rb200_gemm_fp16_intx_allreduce`): one process per GPU over CUDA IPC workspaces.  Every rank
holds a K-shard of the same seeded layer; the result on every rank must be bit-identical and
agree with the oracle run on the unsharded layer (decode, sequential fp32 matmul, epilogue).
Needs at least two GPUs; with one GPU only the world-size-1 form (the plain matmul) runs."""
import ctypes
import os

import numpy as np
import pytest
import torch

from relax_b200 import _lib, ops, synth
from tests.util import assert_close, to_dev, u32_to_dev

pytestmark = pytest.mark.gpu

# (m, k, n, kind): q4 = q4f16_1 group 32; i8 = FT int8 per channel
SHAPES = [(1, 4096, 4096, "q4"), (8, 11008, 4096, "q4"), (32, 4096, 4096, "q4"), (16, 2048, 8192, "i8"),
          (5, 1024, 4224, "q4")]


def _layer(m, k, n, kind, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    if kind == "q4":
        c = synth.q4_case(g, m, k, n, 32)
        return c.x, c.w, c.scales
    x = g.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    w = g.integers(-127, 128, size=(k, n), dtype=np.int8)
    s = g.uniform(1e-4, 1e-3, size=(n,)).astype(np.float16)
    return x, w, s


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from relax_b200 import sharding
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rp = sharding.RowParallelLinear(8192)
    ok, msgs = True, []
    for si, (m, k, n, kind) in enumerate(SHAPES):
        if (k // world) % 64:
            continue
        x, w, s = _layer(m, k, n, kind, 100 + si)
        rs = np.random.RandomState(si)
        bias = rs.randn(n).astype(np.float16)
        res = rs.randn(m, n).astype(np.float16)
        if kind == "q4":
            sh = sharding.shard_q4f16(w, s, rank, world, "k", 32)
            pre = ops.preprocess_weight_q4f16(u32_to_dev(np.ascontiguousarray(sh.w)))
        else:
            sh = sharding.shard_ft(w, s, rank, world, "k", 8)
            pre = ops.preprocess_weight_ft(to_dev(np.ascontiguousarray(sh.w)), False)
        sd = to_dev(np.ascontiguousarray(sh.scales))
        xd = to_dev(np.ascontiguousarray(x[:, sh.x_slice[0]:sh.x_slice[1]]))
        bd, rd = to_dev(bias), to_dev(res)
        out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")

        def call():
            if kind == "q4":
                rp.gemm_q4f16(xd, pre, sd, out, bias=bd, residual=rd, activation=2)
            else:
                rp.gemm_ft(xd, pre, sd, 8, out, bias=bd)

        for _ in range(3):  # call numbers advance, the two data regions alternate
            out.fill_(float("nan"))
            call()
            torch.cuda.synchronize()
        got = out.cpu()
        # CUDA-graph replay of the same launch
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            call()
        for _ in range(3):
            out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
        if not torch.equal(out.cpu(), got):
            ok = False
            msgs.append("shape %d: graph replay differs from the eager result" % si)
        # every rank holds the same bits
        gathered = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(gathered, got)
        if not all(torch.equal(gathered[0], t) for t in gathered):
            ok = False
            msgs.append("shape %d: ranks disagree" % si)
        if rank == 0:
            from oracle import oracle as orc
            C = orc.C()
            if kind == "q4":
                acc = C.matmul_f32(x, C.decode_q4_nk(w, s, None, 7.0, 32))
                exp = C.epilogue(acc, bias, res, "silu", "plus")
            else:
                acc = C.matmul_f32(x, C.decode_ft_kn(w, s, 8, -1), False)
                exp = C.epilogue(acc, bias)
            try:
                assert_close(got.numpy(), exp, tight=False)
            except AssertionError as e:
                ok = False
                msgs.append("shape %d: differs from the oracle: %s" % (si, e))
    st = ctypes.c_int(0)
    _lib.load().rb200_check_async_error(None, ctypes.byref(st))
    if st.value != 0:
        ok = False
        msgs.append("a bounded wait gave up (status %d)" % st.value)
    dist.barrier()
    rp.close()
    dist.destroy_process_group()
    results[rank] = (ok, msgs)


def _run(world, port):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("worker did not finish")
    assert all(results.get(r, (False, ["no result"]))[0] for r in range(world)), dict(results)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks():
    _run(2, 29541)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_four_ranks():
    _run(4, 29542)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs eight GPUs")
def test_eight_ranks():
    _run(8, 29543)


def test_world_of_one_is_the_plain_matmul(oracle):
    m, k, n = 4, 1024, 4224
    x, w, s = _layer(m, k, n, "q4", 7)
    pre = ops.preprocess_weight_q4f16(u32_to_dev(w))
    xd, sd = to_dev(x), to_dev(s)
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    d = _lib.GemmDesc()
    d.struct_size = ctypes.sizeof(_lib.GemmDesc)
    d.weight_bits = 4
    d.x, d.w, d.scales, d.out = xd.data_ptr(), pre.data_ptr(), sd.data_ptr(), out.data_ptr()
    d.m, d.n, d.k, d.ldx, d.ldo = m, n, k, k, n
    d.group_size, d.scale_stride_n, d.scale_stride_g, d.zero_const = 32, k // 32, 1, 7.0
    lib = _lib.load()
    _lib.check(lib.rb200_gemm_fp16_intx_allreduce(ctypes.byref(d), None, 0, 1, 8192, None))
    torch.cuda.synchronize()
    C = oracle.C()
    assert_close(out.cpu().numpy(), C.epilogue(C.matmul_f32(x, C.decode_q4_nk(w, s, None, 7.0, 32))))
    assert lib.rb200_gemm_fp16_intx_allreduce(ctypes.byref(d), None, 1, 1, 8192, None) == -1


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m,k,n,kind", [(1, 4096, 4096, "q4"), (8, 2048, 4096, "q4"), (32, 1024, 4224, "q4"),
                                        (16, 2048, 8192, "i8")])
def test_all_ranks_in_one_launch_on_one_gpu(oracle, world, m, k, n, kind):
    """The exchange of the fused epilogue on a single GPU: `world` ranks inside one cooperative
    launch (all CTAs resident together), every rank on its share of the SMs with its own
    workspace and split-k scratch.  All ranks compute the same matmul, so every rank's block of
    rows must be epilogue(world * (x @ wq^T)) - exact in fp32 for a power-of-two world - and the
    blocks must agree bit for bit.  Called three times: the call number advances and the two data
    regions alternate."""
    lib = _lib.load()
    x, w, s = _layer(m, k, n, kind, 7 + world)
    rs = np.random.RandomState(world)
    bias = rs.randn(n).astype(np.float16)
    if kind == "q4":
        pre = ops.preprocess_weight_q4f16(u32_to_dev(w))
    else:
        pre = ops.preprocess_weight_ft(to_dev(w), False)
    sd, xd, bd = to_dev(s), to_dev(x), to_dev(bias)
    out = torch.full((world * m, n), float("nan"), dtype=torch.float16, device="cuda")
    nbytes = lib.rb200_gemm_allreduce_workspace_bytes(8192)
    spaces = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in spaces])
    d = _lib.GemmDesc()
    d.struct_size = ctypes.sizeof(_lib.GemmDesc)
    d.weight_bits = 4 if kind == "q4" else 8
    d.x, d.w, d.scales, d.out, d.bias = xd.data_ptr(), pre.data_ptr(), sd.data_ptr(), out.data_ptr(), bd.data_ptr()
    d.m, d.n, d.k, d.ldx, d.ldo = m, n, k, k, n
    if kind == "q4":
        d.group_size, d.scale_stride_n, d.scale_stride_g, d.zero_const = 32, k // 32, 1, 7.0
    else:
        d.group_size, d.scale_stride_n, d.scale_stride_g, d.zero_const = k, 1, 0, 128.0
    for _ in range(3):
        out.fill_(float("nan"))
        _lib.check(lib.rb200_gemm_fp16_intx_allreduce_selftest(ctypes.byref(d), ptrs, world, 8192, None))
        torch.cuda.synchronize()
        st = ctypes.c_int(0)
        assert lib.rb200_check_async_error(None, ctypes.byref(st)) == 0 and st.value == 0
        got = out.cpu().numpy().reshape(world, m, n)
        for r in range(1, world):
            assert np.array_equal(got[0].view(np.uint16), got[r].view(np.uint16)), "rank %d differs from rank 0" % r
    C = oracle.C()
    if kind == "q4":
        acc = C.matmul_f32(x, C.decode_q4_nk(w, s, None, 7.0, 32))
    else:
        acc = C.matmul_f32(x, C.decode_ft_kn(w, s, 8, -1), False)
    exp = C.epilogue(acc * np.float32(world), bias)
    assert_close(got[0], exp, tight=False)
