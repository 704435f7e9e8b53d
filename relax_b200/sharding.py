"""Megatron-style sharding of weight-only quantised linears (host logic, no kernels).

Mirrors what the reference's tests do by hand when they place ``W[:, shard]`` / ``W[shard, :]`` on
each Disco worker (tests/python/disco/test_ccl.py:190-198,240-241) and finish a row-parallel layer
with ``runtime.disco.allreduce`` (src/runtime/disco/nccl/nccl.cc:90-98):

* column-parallel: rank r owns output columns [r*N/g, (r+1)*N/g) with their scales; x is
  replicated; no collective; the output stays sharded along N;
* row-parallel: rank r owns reduction rows [r*K/g, (r+1)*K/g) and the matching slice of x;
  per-channel scales are replicated, group scales / zeros are sliced along the group axis
  (K/g must be a multiple of the group size); partial outputs are summed with an all-reduce.

All functions take and return numpy arrays or torch tensors in the layouts the operators accept,
BEFORE ``preprocess_weight`` (the repack is per shard).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass
class Shard:
    w: Any
    scales: Any
    zeros: Optional[Any]
    k: int
    n: int
    x_slice: Optional[Tuple[int, int]]   # columns of x this rank consumes (row-parallel), else None
    needs_allreduce: bool


def _check(total: int, world: int, what: str, multiple: int = 1) -> int:
    if total % world != 0:
        raise ValueError("%s=%d is not divisible by the %d ranks" % (what, total, world))
    part = total // world
    if part % multiple != 0:
        raise ValueError("%s/ranks=%d must be a multiple of %d" % (what, part, multiple))
    return part


def shard_ft(w, scales, rank: int, world: int, axis: str, bits: int, group: int = -1, zeros=None) -> Shard:
    """FT layout: w int8 [K, N/2] (int4) or [K, N] (int8); scales [N] or [K/group, N]."""
    k = w.shape[0]
    n = w.shape[1] * (2 if bits == 4 else 1)
    per_channel = group <= 0 or group >= k
    if axis == "n":
        nl = _check(n, world, "N", 16)
        c0, c1 = rank * nl, (rank + 1) * nl
        wc0, wc1 = (c0 // 2, c1 // 2) if bits == 4 else (c0, c1)
        s = scales[c0:c1] if per_channel else scales[:, c0:c1]
        z = None if zeros is None else (zeros[c0:c1] if per_channel else zeros[:, c0:c1])
        return Shard(w[:, wc0:wc1], s, z, k, nl, None, False)
    if axis != "k":
        raise ValueError("axis must be 'n' (column-parallel) or 'k' (row-parallel)")
    kl = _check(k, world, "K", (64 if bits == 4 else 32) if per_channel else max(group, 64 if bits == 4 else 32))
    r0, r1 = rank * kl, (rank + 1) * kl
    if per_channel:
        s, z = scales, zeros
    else:
        s = scales[r0 // group:r1 // group]
        z = None if zeros is None else zeros[r0 // group:r1 // group]
    return Shard(w[r0:r1], s, z, kl, n, (r0, r1), True)


def shard_q4f16(w, scales, rank: int, world: int, axis: str, group: int = 32, zeros=None) -> Shard:
    """q4f16_1 layout: w uint32 [N, K/8]; scales (and zeros) [N, K/group]."""
    n = w.shape[0]
    k = w.shape[1] * 8
    if axis == "n":
        nl = _check(n, world, "N", 16)
        r0, r1 = rank * nl, (rank + 1) * nl
        return Shard(w[r0:r1], scales[r0:r1], None if zeros is None else zeros[r0:r1], k, nl, None, False)
    if axis != "k":
        raise ValueError("axis must be 'n' (column-parallel) or 'k' (row-parallel)")
    kl = _check(k, world, "K", max(group, 64))
    c0, c1 = rank * kl, (rank + 1) * kl
    return Shard(w[:, c0 // 8:c1 // 8], scales[:, c0 // group:c1 // group],
                 None if zeros is None else zeros[:, c0 // group:c1 // group], kl, n, (c0, c1), True)


def expert_range(num_experts: int, rank: int, world: int) -> Tuple[int, int]:
    """MoE: experts [r*E/g, (r+1)*E/g) live on rank r (one expert per GPU at g = E)."""
    per = _check(num_experts, world, "experts")
    return rank * per, (rank + 1) * per


def allreduce_sum_(t, group=None):
    """Sum all-reduce of a row-parallel partial output over the ranks (NCCL on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
