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


class RankMonitor:
    """Host-side membership for the ranks of one job: a rank that stops taking part (shutdown,
    preemption, an exception in its serving loop) says so through a key-value store before it
    goes, and the others look before their next launch.  A kernel that waits for a peer which is
    gone would sit out its bounded wait (``rb200_set_wait_limit_ms``) and report through the status
    word; with this check the survivors never launch it.  The reference has no counterpart: its
    collectives abort the process on any NCCL error (src/runtime/disco/nccl/nccl_context.h:50-56)
    and its customized all-reduce spins without a bound
    (3rdparty/tensorrt_llm/custom_allreduce_kernels.cu:94-113).

    ``store`` is any ``torch.distributed`` store (``TCPStore``, ``FileStore``, the default store of
    an initialised process group)."""

    def __init__(self, store, rank: int, world: int, prefix: str = "rb200/left/"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def leave(self, reason: str = "") -> None:
        """Call between steps, with none of this rank's kernels or collectives in flight."""
        self.store.set(self.prefix + str(self.rank), reason or "left")

    def departed(self):
        """Ranks that have announced their departure (cheap: one store query per peer)."""
        return [r for r in range(self.world) if r != self.rank and self.store.check([self.prefix + str(r)])]

    def all_present(self) -> bool:
        return not self.departed()


class PeerWorkspace:
    """A zero-filled device buffer of this rank that every rank of the group can address: allocated
    with ``rb200_peer_alloc``, its CUDA IPC handle exchanged over ``torch.distributed`` (host bytes
    only, any backend) and the peers' handles mapped - what
    src/runtime/disco/cuda_ipc/cuda_ipc_memory.cc does over Disco's channel.  ``ptrs[p]`` is this
    process's address of rank p's buffer."""

    def __init__(self, nbytes: int, group=None):
        import ctypes
        import torch.distributed as dist
        from . import _lib
        self._lib = _lib
        lib = _lib.load()
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        own = ctypes.c_void_p()
        _lib.check(lib.rb200_peer_alloc(nbytes, ctypes.byref(own)))
        self._own = own
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.rb200_peer_export(own, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self._imported = []
        self.ptrs = (ctypes.c_void_p * self.world)()
        for p in range(self.world):
            if p == self.rank:
                self.ptrs[p] = own.value
            else:
                q = ctypes.c_void_p()
                _lib.check(lib.rb200_peer_import(ctypes.create_string_buffer(handles[p], 64), ctypes.byref(q)))
                self._imported.append(q)
                self.ptrs[p] = q.value
        dist.barrier(group=group)  # every workspace exists and is zero before the first use

    def close(self):
        lib = self._lib.load()
        for q in self._imported:
            lib.rb200_peer_close(q)
        self._imported = []
        if self._own is not None:
            lib.rb200_peer_free(self._own)
            self._own = None


class RowParallelLinear:
    """Row-parallel decode matmul whose epilogue is the all-reduce (``rb200_gemm_fp16_intx_allreduce``):
    one kernel per rank instead of the reference's matmul followed by ``runtime.disco.allreduce``
    (src/runtime/disco/nccl/nccl.cc:90-98).  One object serves every row-parallel layer of a model
    whose output width is at most ``max_n``; calls must be issued in the same order on all ranks."""

    def __init__(self, max_n: int, group=None):
        from . import _lib
        self._lib = _lib
        self.max_n = int(max_n)
        self.ws = PeerWorkspace(_lib.load().rb200_gemm_allreduce_workspace_bytes(self.max_n), group)
        self.rank, self.world = self.ws.rank, self.ws.world

    def _call(self, d):
        import ctypes
        import torch
        lib = self._lib.load()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._lib.check(lib.rb200_gemm_fp16_intx_allreduce(ctypes.byref(d), self.ws.ptrs, self.rank, self.world,
                                                           self.max_n, stream))

    def bind_q4f16(self, x, w_pre, scales, out, group_size: int = 32, zero_const: float = 7.0):
        """The call of :meth:`gemm_q4f16` with its descriptor built once: returns a zero-argument
        callable for serving loops that pass the same buffers on every step."""
        import ctypes
        import torch
        d = self._lib.GemmDesc()
        d.struct_size = ctypes.sizeof(self._lib.GemmDesc)
        d.weight_bits = 4
        k = x.shape[-1]
        d.x, d.w, d.scales, d.out = x.data_ptr(), w_pre.data_ptr(), scales.data_ptr(), out.data_ptr()
        d.m, d.n, d.k = x.numel() // k, w_pre.shape[0], k
        d.ldx, d.ldo = k, w_pre.shape[0]
        d.group_size = group_size
        d.scale_stride_n, d.scale_stride_g = k // group_size, 1
        d.zero_const = zero_const
        fn = self._lib.load().rb200_gemm_fp16_intx_allreduce
        ref, ptrs, rank, world, max_n, check = ctypes.byref(d), self.ws.ptrs, self.rank, self.world, self.max_n, self._lib.check
        keep = (d, x, w_pre, scales, out)

        def call():
            rc = fn(ref, ptrs, rank, world, max_n, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            if rc != 0:
                check(rc)
            return keep[4]

        return call

    def gemm_q4f16(self, x, w_pre, scales, out, group_size: int = 32, zero_const: float = 7.0, bias=None,
                   residual=None, activation: int = 0):
        """``out = epilogue(sum over ranks of x_shard @ decode(w_shard)^T)`` for q4f16_1 shards
        (:func:`shard_q4f16` with ``axis="k"``), every rank receiving the full result."""
        import ctypes
        d = self._lib.GemmDesc()
        d.struct_size = ctypes.sizeof(self._lib.GemmDesc)
        d.weight_bits = 4
        k = x.shape[-1]
        d.x, d.w, d.scales, d.out = x.data_ptr(), w_pre.data_ptr(), scales.data_ptr(), out.data_ptr()
        d.m, d.n, d.k = x.numel() // k, w_pre.shape[0], k
        d.ldx, d.ldo = k, w_pre.shape[0]
        d.group_size = group_size
        d.scale_stride_n, d.scale_stride_g = k // group_size, 1
        d.zero_const = zero_const
        d.activation = activation
        if bias is not None:
            d.bias = bias.data_ptr()
        if residual is not None:
            d.residual, d.binary_op = residual.data_ptr(), 1
        self._call(d)
        return out

    def gemm_ft(self, x, w_pre, scales, weight_bits: int, out, bias=None):
        """The same for FT-layout shards with per-channel scales (:func:`shard_ft` with ``axis="k"``)."""
        import ctypes
        d = self._lib.GemmDesc()
        d.struct_size = ctypes.sizeof(self._lib.GemmDesc)
        d.weight_bits = weight_bits
        k = x.shape[-1]
        n = w_pre.shape[-1] * (2 if weight_bits == 4 else 1)
        d.x, d.w, d.scales, d.out = x.data_ptr(), w_pre.data_ptr(), scales.data_ptr(), out.data_ptr()
        d.m, d.n, d.k = x.numel() // k, n, k
        d.ldx, d.ldo = k, n
        d.group_size = k
        d.scale_stride_n, d.scale_stride_g = 1, 0
        d.zero_const = 8.0 if weight_bits == 4 else 128.0
        if bias is not None:
            d.bias = bias.data_ptr()
        self._call(d)
        return out

    def close(self):
        self.ws.close()


class OneShotAllReduce:
    """Low-latency sum all-reduce of small fp16 tensors between the GPUs of one node
    (``rb200_allreduce_oneshot``): the counterpart of ``runtime.disco.cuda_ipc.custom_allreduce``
    with its one-shot strategy (src/runtime/disco/cuda_ipc/custom_allreduce.cc:65-105).  Each rank
    allocates a peer-visible workspace, the ranks exchange its CUDA IPC handle over
    ``torch.distributed`` (any backend - only host bytes travel) and map one another's
    (src/runtime/disco/cuda_ipc/cuda_ipc_memory.cc does the same with Disco's channel).

    ``max_count`` bounds the tensor size in elements; larger tensors go through
    :func:`allreduce_sum_` (NCCL), as the reference falls back to ``ncclAllReduce``.
    All ranks must call with the same sequence of tensor sizes."""

    def __init__(self, max_count: int, group=None):
        import torch
        from . import _lib
        self._lib = _lib
        self.group = group
        self.max_count = int(max_count)
        self.ws = PeerWorkspace(_lib.load().rb200_allreduce_workspace_bytes(self.max_count), group)
        self.rank, self.world = self.ws.rank, self.ws.world
        self._ptrs = self.ws.ptrs
        self._torch = torch

    def fits(self, t) -> bool:
        return t.dtype == self._torch.float16 and t.is_contiguous() and t.numel() <= self.max_count

    def __call__(self, t, out=None):
        """In place by default.  ``t``: contiguous fp16 CUDA tensor of at most ``max_count`` elements."""
        import ctypes
        if not self.fits(t):
            raise ValueError("tensor does not fit the one-shot all-reduce (fp16, contiguous, <= %d elements)"
                             % self.max_count)
        out = t if out is None else out
        stream = self._torch.cuda.current_stream().cuda_stream
        self._lib.check(self._lib.load().rb200_allreduce_oneshot(
            self._ptrs, self.rank, self.world, ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(out.data_ptr()),
            t.numel(), self.max_count, ctypes.c_void_p(stream)))
        return out

    def close(self):
        self.ws.close()
