"""Parameter cache (ndarray-cache.json + params_shard_*.bin, the reference's on-disk form) and the
per-rank loader: the ranks' slices, put back together, reproduce the full product."""
import json
import os

import numpy as np
import pytest

from relax_b200 import param_cache, synth


def _make_cache(tmp_path, oracle):
    g = np.random.Generator(np.random.PCG64(21))
    k, n = 256, 128
    y = g.normal(0, 0.002, size=(n, k)).astype(np.float16)
    packed4, s4 = oracle.np_encode_ft(y, 4, 64)
    packed8, s8 = oracle.np_encode_ft(y, 8, -1)
    q = synth.q4_case(g, 1, k, n, 32, asymmetric=True)
    params = {"l0.w": packed4, "l0.s": s4, "l1.w": packed8, "l1.s": s8,
              "l2.w": q.w, "l2.s": q.scales, "l2.z": q.zeros}
    param_cache.write_cache(str(tmp_path), params, shard_bytes=20000)
    return params, k, n


def test_cache_roundtrip_and_format(tmp_path, oracle):
    params, k, n = _make_cache(tmp_path, oracle)
    meta = json.load(open(os.path.join(tmp_path, "ndarray-cache.json")))
    assert len(meta["records"]) > 1  # several shard files
    for f in meta["records"]:
        assert f["format"] == "raw-shard" and os.path.getsize(os.path.join(tmp_path, f["dataPath"])) == f["nbytes"]
        for r in f["records"]:
            assert set(r) >= {"name", "shape", "dtype", "format", "nbytes", "byteOffset"}
    recs = param_cache.load_metadata(str(tmp_path))
    for name, arr in params.items():
        got = param_cache.read_param(str(tmp_path), recs[name])
        assert got.dtype == arr.dtype and np.array_equal(got, arr)


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_load_reassembles_the_product(tmp_path, oracle, world):
    params, k, n = _make_cache(tmp_path, oracle)
    C = oracle.C()
    x = np.random.RandomState(0).randn(3, k).astype(np.float16)
    specs = {
        "ft4_col": param_cache.LinearSpec("l0.w", "l0.s", "ft", 4, 64, "n"),
        "ft4_row": param_cache.LinearSpec("l0.w", "l0.s", "ft", 4, 64, "k"),
        "ft8_row": param_cache.LinearSpec("l1.w", "l1.s", "ft", 8, -1, "k"),
        "q4_col": param_cache.LinearSpec("l2.w", "l2.s", "q4f16", 4, 32, "n", "l2.z"),
        "q4_row": param_cache.LinearSpec("l2.w", "l2.s", "q4f16", 4, 32, "k", "l2.z"),
    }

    def product(spec, w, s, z, xs):
        if spec.layout == "ft":
            return C.matmul_f32(xs, C.decode_ft_kn(w, s, spec.bits, spec.group), False)
        return C.matmul_f32(xs, C.decode_q4_nk(w, s, z, 7.0, spec.group))

    for name, spec in specs.items():
        full = param_cache.ShardedLoader(str(tmp_path), 0, 1).load(spec)
        ref = product(spec, full.w, full.scales, full.zeros, x)
        parts = [param_cache.ShardedLoader(str(tmp_path), r, world).load(spec) for r in range(world)]
        if spec.axis == "n":
            got = np.concatenate([product(spec, p.w, p.scales, p.zeros, x) for p in parts], axis=1)
            assert not any(p.needs_allreduce for p in parts)
            np.testing.assert_array_equal(got, ref)
        else:
            got = sum(product(spec, p.w, p.scales, p.zeros, x[:, p.x_slice[0]:p.x_slice[1]]) for p in parts)
            assert all(p.needs_allreduce for p in parts)
            np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_loader_repacks_on_the_gpu(tmp_path, oracle):
    import torch
    from relax_b200 import ops
    from tests.util import assert_close, to_dev
    params, k, n = _make_cache(tmp_path, oracle)
    x = np.random.RandomState(1).randn(5, k).astype(np.float16)
    spec = param_cache.LinearSpec("l0.w", "l0.s", "ft", 4, 64, "n")
    C = oracle.C()
    ref = C.epilogue(C.matmul_f32(x, C.decode_ft_kn(params["l0.w"], params["l0.s"], 4, 64), False))
    outs = []
    for r in range(2):
        lin = param_cache.ShardedLoader(str(tmp_path), r, 2, device="cuda").load(spec)
        outs.append(ops.gemm_fp16_ft(to_dev(x), lin.w, lin.scales, 4, group_size=64).cpu().numpy())
    torch.cuda.synchronize()
    assert_close(np.concatenate(outs, axis=1), ref)
