"""World-size-2 CPU (gloo) checks of the multi-GPU host logic: shard slicing for column- and
row-parallel layers, the all-reduce after a row-parallel layer, expert ranges.  Each rank computes
its shard with the CPU oracle (the GPU kernels need a GPU; what is tested here is that the slices
and the collective reassemble the unsharded result)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        from relax_b200 import sharding, synth
        C = orc.C()
        ok = True
        # ---- q4f16_1, group 32: column-parallel then row-parallel
        case = synth.q4_case(np.random.Generator(np.random.PCG64(7)), 4, 512, 64, 32)
        full = C.matmul_f32(case.x, C.decode_q4_nk(case.w, case.scales, None, 7.0, 32))
        sh = sharding.shard_q4f16(case.w, case.scales, rank, world, "n", 32)
        part = C.matmul_f32(case.x, C.decode_q4_nk(np.ascontiguousarray(sh.w), np.ascontiguousarray(sh.scales), None, 7.0, 32))
        gathered = [torch.zeros(4, 64 // world) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        ok &= np.array_equal(torch.cat(gathered, dim=1).numpy(), full)
        assert not sh.needs_allreduce and sh.n == 64 // world
        sh = sharding.shard_q4f16(case.w, case.scales, rank, world, "k", 32)
        xs = np.ascontiguousarray(case.x[:, sh.x_slice[0]:sh.x_slice[1]])
        part = C.matmul_f32(xs, C.decode_q4_nk(np.ascontiguousarray(sh.w), np.ascontiguousarray(sh.scales), None, 7.0, 32))
        t = torch.from_numpy(part.copy())
        sharding.allreduce_sum_(t)
        ok &= np.allclose(t.numpy(), full, rtol=1e-5, atol=1e-5)
        assert sh.needs_allreduce and sh.k == 512 // world
        # ---- FT int8 per channel (Llama-70B MLP style): gate_up columns, down rows
        c3 = synth.config3("down", 16, k=256, n=64)
        fullw = C.decode_ft_kn(c3.w, c3.scales, 8, -1)
        full = C.matmul_f32(c3.x, fullw, False)
        sh = sharding.shard_ft(c3.w, c3.scales, rank, world, "k", 8)
        xs = np.ascontiguousarray(c3.x[:, sh.x_slice[0]:sh.x_slice[1]])
        part = C.matmul_f32(xs, C.decode_ft_kn(np.ascontiguousarray(sh.w), sh.scales, 8, -1), False)
        t = torch.from_numpy(part.copy())
        sharding.allreduce_sum_(t)
        ok &= np.allclose(t.numpy(), full, rtol=1e-5, atol=1e-5)
        sh = sharding.shard_ft(c3.w, c3.scales, rank, world, "n", 8)
        part = C.matmul_f32(c3.x, C.decode_ft_kn(np.ascontiguousarray(sh.w), np.ascontiguousarray(sh.scales), 8, -1), False)
        ok &= np.array_equal(part, full[:, rank * (64 // world):(rank + 1) * (64 // world)])
        # ---- experts
        assert sharding.expert_range(8, rank, world) == (rank * 4, rank * 4 + 4)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_world_size_2_shards_reassemble():
    port = 29500 + (os.getpid() % 1000)
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def _leaving_worker(rank, world, port, store_port, ret):
    """Step 1 with both ranks; rank 1 then leaves between steps.  Rank 0 must learn of it on the
    host before its next launch, and a collective it started anyway must end with an error, not
    hang."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from relax_b200 import sharding
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    mon = sharding.RankMonitor(store, rank, world)
    t = torch.ones(8) * (rank + 1)
    assert mon.all_present()
    sharding.allreduce_sum_(t)  # step 1: everyone is there
    ok = bool(torch.all(t == 3))
    if rank == 1:
        mon.leave("shutting down")  # between steps, nothing in flight
        ret[rank] = ok
        store.wait(["rb200/test/seen"])  # keep the store's client alive until rank 0 has looked
        dist.destroy_process_group()
        return
    deadline = time.time() + 20
    while mon.all_present() and time.time() < deadline:
        time.sleep(0.05)
    ok &= mon.departed() == [1]  # learnt on the host: the survivor launches nothing for step 2
    store.set("rb200/test/seen", "1")
    # what would have happened without the check: the collective fails within the group's timeout
    time.sleep(0.5)
    t0 = time.time()
    failed = False
    try:
        dist.all_reduce(torch.ones(8))
    except Exception:
        failed = True
    ok &= failed and (time.time() - t0) < 15
    ret[rank] = ok
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host():
    port = 30500 + (os.getpid() % 1000)
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_leaving_worker, args=(2, port, port + 1500, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True, dict(ret)


def test_shard_validation():
    sys.path.insert(0, ROOT)
    from relax_b200 import sharding
    w = np.zeros((48, 8), dtype=np.uint32)
    s = np.zeros((48, 2), dtype=np.float16)
    with pytest.raises(ValueError):
        sharding.shard_q4f16(w, s, 0, 5, "n")      # 48 rows over 5 ranks
    with pytest.raises(ValueError):
        sharding.shard_q4f16(w, s, 0, 2, "k")      # K/2 = 32 is not a whole 64-k fragment
    with pytest.raises(ValueError):
        sharding.shard_q4f16(w, s, 0, 2, "x")
