"""Parameter cache on disk and per-rank loading of quantised linears (host logic).

The on-disk form is the reference's NDArray cache: ``ndarray-cache.json`` listing shard files
``params_shard_<i>.bin`` of format ``raw-shard``, each with parameter records ``name, shape, dtype,
format ("raw"), nbytes, byteOffset`` (include/tvm/runtime/relax_vm/ndarray_cache_support.h:36-87,
src/runtime/relax_vm/ndarray_cache_support.cc:75-131).  :class:`ShardedLoader` plays the role of
``runtime.disco.ShardLoader`` (src/runtime/disco/loader.cc:46-165,409-447) for this path: every
rank reads the parameters it needs, keeps its Megatron slice (:mod:`relax_b200.sharding`) and
repacks the weight slice once with the preprocess entry point, so that the repack is per shard
and never sees the full matrix on one GPU.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional

import numpy as np

from . import sharding

_DTYPES = {"int8": np.int8, "uint8": np.uint8, "int32": np.int32, "uint32": np.uint32, "int64": np.int64,
           "float16": np.float16, "float32": np.float32}


@dataclass
class ParamRecord:
    name: str
    shape: tuple
    dtype: str
    nbytes: int
    byte_offset: int
    data_path: str


def write_cache(directory: str, params: Dict[str, np.ndarray], shard_bytes: int = 32 << 20) -> None:
    """Writes ``params`` as ``ndarray-cache.json`` + ``params_shard_<i>.bin`` (format "raw-shard",
    records of format "raw"); a parameter never straddles two shard files."""
    os.makedirs(directory, exist_ok=True)
    files: List[dict] = []
    cur: List[dict] = []
    blob = bytearray()

    def flush():
        nonlocal cur, blob
        if not cur:
            return
        path = "params_shard_%d.bin" % len(files)
        with open(os.path.join(directory, path), "wb") as f:
            f.write(bytes(blob))
        files.append({"dataPath": path, "format": "raw-shard", "nbytes": len(blob), "records": cur})
        cur, blob = [], bytearray()

    for name, arr in params.items():
        arr = np.ascontiguousarray(arr)
        if arr.dtype.name not in _DTYPES:
            raise ValueError("unsupported dtype %s for %s" % (arr.dtype, name))
        raw = arr.tobytes()
        if blob and len(blob) + len(raw) > shard_bytes:
            flush()
        cur.append({"name": name, "shape": list(arr.shape), "dtype": arr.dtype.name, "format": "raw",
                    "nbytes": len(raw), "byteOffset": len(blob)})
        blob += raw
    flush()
    with open(os.path.join(directory, "ndarray-cache.json"), "w") as f:
        json.dump({"metadata": {"ParamSize": len(params)}, "records": files}, f)


def load_metadata(directory: str) -> Dict[str, ParamRecord]:
    with open(os.path.join(directory, "ndarray-cache.json")) as f:
        meta = json.load(f)
    out: Dict[str, ParamRecord] = {}
    for frec in meta["records"]:
        if frec.get("format", "raw-shard") != "raw-shard":
            raise ValueError("only the raw-shard file format is supported, got %r" % frec.get("format"))
        for r in frec["records"]:
            if r.get("format", "raw") != "raw":
                raise ValueError("parameter %s: only the raw record format is supported" % r["name"])
            out[r["name"]] = ParamRecord(r["name"], tuple(r["shape"]), r["dtype"], int(r["nbytes"]),
                                         int(r["byteOffset"]), frec["dataPath"])
    return out


def read_param(directory: str, rec: ParamRecord) -> np.ndarray:
    """One parameter, memory-mapped from its shard file (only the bytes that get sliced are read)."""
    mm = np.memmap(os.path.join(directory, rec.data_path), dtype=np.uint8, mode="r", offset=rec.byte_offset,
                   shape=(rec.nbytes,))
    return mm.view(_DTYPES[rec.dtype]).reshape(rec.shape)


@dataclass
class LinearSpec:
    """How one quantised linear is stored and split.  ``layout``: "ft" (weight int8 [K, N/2] or
    [K, N], scales [N] or [K/group, N]) or "q4f16" (weight uint32 [N, K/8], scales [N, K/group]);
    ``axis``: "n" column-parallel, "k" row-parallel, None replicated."""
    weight: str
    scales: str
    layout: str
    bits: int = 4
    group: int = -1
    axis: Optional[str] = None
    zeros: Optional[str] = None


@dataclass
class LoadedLinear:
    w: object            # preprocessed weight (torch CUDA tensor) or the raw numpy slice
    scales: object
    zeros: object
    k: int
    n: int
    x_slice: Optional[tuple]
    needs_allreduce: bool


class ShardedLoader:
    """Per-rank loading: ``load(spec)`` returns this rank's slice of a linear, repacked on the GPU
    when ``device`` is a CUDA device (``device=None`` keeps numpy slices - what the CPU tests use)."""

    def __init__(self, directory: str, rank: int, world: int, device=None):
        self.directory = directory
        self.rank = rank
        self.world = world
        self.device = device
        self.meta = load_metadata(directory)

    def names(self) -> Iterable[str]:
        return self.meta.keys()

    def _get(self, name: str) -> np.ndarray:
        if name not in self.meta:
            raise KeyError("parameter %s is not in the cache" % name)
        return read_param(self.directory, self.meta[name])

    def load(self, spec: LinearSpec) -> LoadedLinear:
        w, s = self._get(spec.weight), self._get(spec.scales)
        z = self._get(spec.zeros) if spec.zeros else None
        if spec.axis is None or self.world == 1:
            k = w.shape[0] if spec.layout == "ft" else w.shape[1] * 8
            n = (w.shape[1] * (2 if spec.bits == 4 else 1)) if spec.layout == "ft" else w.shape[0]
            sh = sharding.Shard(w, s, z, k, n, None, False)
        elif spec.layout == "ft":
            sh = sharding.shard_ft(w, s, self.rank, self.world, spec.axis, spec.bits, spec.group, z)
        elif spec.layout == "q4f16":
            sh = sharding.shard_q4f16(w, s, self.rank, self.world, spec.axis, spec.group, z)
        else:
            raise ValueError("unknown layout %r" % spec.layout)
        wv, sv = np.ascontiguousarray(sh.w), np.ascontiguousarray(sh.scales)
        zv = None if sh.zeros is None else np.ascontiguousarray(sh.zeros)
        if self.device is None:
            return LoadedLinear(wv, sv, zv, sh.k, sh.n, sh.x_slice, sh.needs_allreduce)
        import torch
        from . import ops
        dev = torch.device(self.device)
        if spec.layout == "ft":
            pre = ops.preprocess_weight_ft(torch.from_numpy(wv.view(np.int8)).to(dev), spec.bits == 4)
        else:
            pre = ops.preprocess_weight_q4f16(torch.from_numpy(wv.view(np.int32)).to(dev))
        st = torch.from_numpy(sv).to(dev)
        zt = None if zv is None else torch.from_numpy(zv).to(dev)
        return LoadedLinear(pre, st, zt, sh.k, sh.n, sh.x_slice, sh.needs_allreduce)
