"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No public dataset or model weights are involved: the layer sizes are those of Llama-2-7B,
Llama-70B and Mixtral-8x7B linears, the values are drawn from ``numpy.random.Generator(PCG64(seed))``
with ``seed = 1000 * config + index``.  Everything is returned as numpy arrays on the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

# (name, K, N) of the Llama-2-7B decode linears (config 1)
LLAMA7B_LINEARS: List[Tuple[str, int, int]] = [
    ("qkv", 4096, 12288), ("o", 4096, 4096), ("gate_up", 4096, 22016), ("down", 11008, 4096),
]
# Llama-70B MLP (config 3): (name, K, N, sharded axis)
LLAMA70B_MLP = [("gate_up", 8192, 57344, "n"), ("down", 28672, 8192, "k")]


def rng(config: int, index: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(1000 * config + index))


@dataclass
class Q4Case:
    """W4A16 group-quantised case in the q4f16_1 layout."""
    x: np.ndarray                 # fp16 [M, K]
    w: np.ndarray                 # uint32 [N, K/8]
    scales: np.ndarray            # fp16 [N, K/g]
    zeros: Optional[np.ndarray]   # fp16 [N, K/g] or None (constant zero point 7)
    group: int
    zero_const: float = 7.0


def pack_q4_nk(codes: np.ndarray) -> np.ndarray:
    """codes uint8 [N, K] (values 0..15) -> uint32 [N, K/8], nibble j of a word = element 8w+j."""
    n, k = codes.shape
    c = codes.reshape(n, k // 8, 8).astype(np.uint32)
    sh = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    return np.bitwise_or.reduce(c << sh, axis=2).astype(np.uint32)


def q4_case(g: np.random.Generator, m: int, k: int, n: int, group: int = 32,
            asymmetric: bool = False) -> Q4Case:
    x = g.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    codes = g.integers(0, 16, size=(n, k), dtype=np.uint8)
    scales = g.uniform(0.001, 0.01, size=(n, k // group)).astype(np.float16)
    zeros = None
    if asymmetric:
        zeros = g.integers(0, 16, size=(n, k // group)).astype(np.float16)
    return Q4Case(x, pack_q4_nk(codes), scales, zeros, group)


def config0(m: int = 1) -> Q4Case:
    """x [1,4096], W uint32 [4096,512], scales [4096,128] ~U(0.001,0.01), dequant (code-7)*scale."""
    return q4_case(rng(0), m, 4096, 4096, 32)


def config1(name: str, m: int) -> Q4Case:
    idx = [l[0] for l in LLAMA7B_LINEARS].index(name)
    _, k, n = LLAMA7B_LINEARS[idx]
    return q4_case(rng(1, idx * 100 + m), m, k, n, 32)


def config2(m: int = 2048, k: int = 4096, n: int = 22016) -> Q4Case:
    """Prefill W4A16: group-128 asymmetric, fp16 scales and integer-valued fp16 zero points."""
    return q4_case(rng(2), m, k, n, 128, asymmetric=True)


@dataclass
class Int8Case:
    """W8A16 per-output-channel case in the FT layout (codes int8 [K, N], scales fp16 [N])."""
    x: np.ndarray
    w: np.ndarray
    scales: np.ndarray


def config3(name: str, m: int, shard: Tuple[int, int] = (0, 1), k: Optional[int] = None,
            n: Optional[int] = None) -> Int8Case:
    """Llama-70B MLP linear, optionally only rank ``shard[0]`` of ``shard[1]`` (column-parallel
    for gate_up, row-parallel for down).  The shard is generated directly (seeded per rank) so a
    rank never materialises the full matrix."""
    idx = [l[0] for l in LLAMA70B_MLP].index(name)
    _, k0, n0, axis = LLAMA70B_MLP[idx]
    k = k or k0
    n = n or n0
    rank, world = shard
    g = rng(3, idx * 1000 + m * 10 + 0)
    x = g.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    scales = g.uniform(1e-4, 1e-3, size=(n,)).astype(np.float16)
    gw = rng(3, 500000 + idx * 1000 + rank * 16 + world)
    if axis == "n":
        nl = n // world
        w = gw.integers(-127, 128, size=(k, nl), dtype=np.int8)
        return Int8Case(x, w, scales[rank * nl:(rank + 1) * nl].copy())
    kl = k // world
    w = gw.integers(-127, 128, size=(kl, n), dtype=np.int8)
    return Int8Case(x[:, rank * kl:(rank + 1) * kl].copy(), w, scales)


@dataclass
class MoECase:
    """Mixtral-shaped MoE layer input: tokens already gathered and sorted by expert."""
    x: np.ndarray          # fp16 [sum_rows, K] rows sorted by expert
    w: np.ndarray          # int8 [E, K, N/2] FT int4 layout (signed nibbles)
    scales: np.ndarray     # fp16 [E, K/g, N]
    indptr: np.ndarray     # int64 [E], END row of each expert's block
    token_of_row: np.ndarray
    gate_of_row: np.ndarray
    group: int


def config4(tokens: int = 512, hidden: int = 4096, experts: int = 8, ffn: int = 14336,
            top_k: int = 2, group: int = 128) -> MoECase:
    g = rng(4)
    logits = g.standard_normal((tokens, experts), dtype=np.float32)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :top_k]     # ties -> lower index first
    xt = g.standard_normal((tokens, hidden), dtype=np.float32).astype(np.float16)
    flat_expert = order.reshape(-1)
    flat_token = np.repeat(np.arange(tokens), top_k)
    flat_gate = np.take_along_axis(p, order, axis=1).reshape(-1)
    perm = np.argsort(flat_expert, kind="stable")
    counts = np.bincount(flat_expert, minlength=experts)
    indptr = np.cumsum(counts).astype(np.int64)
    x = xt[flat_token[perm]]
    w = g.integers(-128, 128, size=(experts, hidden, ffn // 2), dtype=np.int8)
    scales = g.uniform(0.001, 0.01, size=(experts, hidden // group, ffn)).astype(np.float16)
    return MoECase(x, w, scales, indptr, flat_token[perm], flat_gate[perm].astype(np.float32), group)


def algorithmic_bytes(m: int, n: int, k: int, bits: int, group: int, zeros: bool = False) -> int:
    """Each operand once: packed weight + scales (+ zeros) + x + out."""
    per_col = group <= 0 or group >= k
    sc = n * (1 if per_col else k // group) * 2
    return n * k * bits // 8 + sc * (2 if zeros else 1) + m * k * 2 + m * n * 2
