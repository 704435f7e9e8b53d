"""The one-shot all-reduce kernel.  On one GPU all ranks run inside a single cooperative launch
(the kernel's self-test entry); with two or more GPUs the real path runs as one process per GPU
over CUDA IPC workspaces, including CUDA-graph replay."""
import ctypes
import os

import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import _lib
from tests.test_gemv_gpu import _check_status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("count", [8, 1000, 4096, 32 * 4096 + 3])
def test_selftest_all_ranks_in_one_launch(world, count):
    lib = _lib.load()
    max_count = 32 * 4096 + 8
    nbytes = lib.rb200_allreduce_workspace_bytes(max_count)
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(world * 1000 + count)
    outs = [torch.empty(count, dtype=torch.float16, device="cuda") for _ in range(world)]
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
    for call in range(5):  # the call counters and the two data regions cycle
        ins = [torch.randn(count, device="cuda", generator=gen).half() for _ in range(world)]
        _lib.check(lib.rb200_allreduce_oneshot_selftest(arr(ws), arr(ins), arr(outs), world, count, max_count, None))
        torch.cuda.synchronize()
        _check_status()
        acc = torch.zeros(count, dtype=torch.float32, device="cuda")
        for t in ins:  # rank order, fp32, one rounding: the kernel's own order
            acc += t.float()
        exp = acc.half()
        for o in outs:
            assert torch.equal(o, exp)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from relax_b200.sharding import OneShotAllReduce
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ar = OneShotAllReduce(32 * 4096)
    ok = True
    gen = torch.Generator(device="cuda")
    for count in (8, 4096, 1000, 32 * 4096):
        parts = []
        for r in range(world):  # every rank can rebuild every rank's input
            gen.manual_seed(1234 + r * 17 + count)
            parts.append(torch.randn(count, device="cuda", generator=gen).half())
        acc = torch.zeros(count, dtype=torch.float32, device="cuda")
        for t in parts:
            acc += t.float()
        exp = acc.half()
        for _ in range(3):
            out = ar(parts[rank].clone())
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(out, exp))
        # CUDA-graph replay of the same launch
        buf = parts[rank].clone()
        res = torch.empty_like(buf)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            ar(buf, out=res)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(res, exp))
    lib = _lib.load()
    st = ctypes.c_int(0)
    lib.rb200_check_async_error(None, ctypes.byref(st))
    ok = ok and st.value == 0
    dist.barrier()
    ar.close()
    dist.destroy_process_group()
    results[rank] = ok


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_ipc():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, 29533, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("worker did not finish")
    assert all(results.get(r) for r in range(world)), dict(results)
