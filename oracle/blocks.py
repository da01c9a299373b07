"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (test infrastructure, not product code).

They stand in for the real GGUF checkpoint the reference's tests and benchmarks read
(tests/test_mmq.py:12-35, bench/mmq_benchmark_common.py:14-19): every bit pattern of the
non-fp16 fields of the five supported block types is a valid block, so "random valid
super-block" = uniform random bytes with the fp16 super-scales overwritten by finite
positive values |N(0,1)| * scale.
"""
from __future__ import annotations

import numpy as np

from .ref import BLOCK_BYTES, IQ2_S, Q3_K, Q4_K, Q5_K, Q6_K

# byte offsets of the fp16 fields (csrc/vendor/llama_cpp/common.cuh:78-127)
_FP16_FIELDS = {Q4_K: (0, 2), Q5_K: (0, 2), Q6_K: (208,), Q3_K: (108,), IQ2_S: (0,)}
_DEFAULT_SCALE = {Q4_K: 2e-3, Q5_K: 2e-3, Q6_K: 2e-3, Q3_K: 2e-3, IQ2_S: 1e-3}


def random_blocks(qtype: int, n_blocks: int, seed: int, scale: float | None = None) -> np.ndarray:
    """uint8 [n_blocks, block_bytes] of valid super-blocks drawn from ``seed``."""
    rng = np.random.Generator(np.random.PCG64(seed))
    bb = BLOCK_BYTES[qtype]
    blocks = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
    s = _DEFAULT_SCALE[qtype] if scale is None else scale
    for off in _FP16_FIELDS[qtype]:
        d = (np.abs(rng.standard_normal(n_blocks)) * s).astype(np.float16)
        blocks[:, off:off + 2] = d.view(np.uint8).reshape(n_blocks, 2)
    return blocks


def dense_weight(qtype: int, out_features: int, in_features: int, seed: int,
                 scale: float | None = None) -> np.ndarray:
    """Packed dense weight as a flat uint8 array of N*(K/256) blocks."""
    return random_blocks(qtype, out_features * (in_features // 256), seed, scale).reshape(-1)


def expert_weights(qtype: int, experts: int, out_features: int, in_features: int, seed: int,
                   scale: float | None = None) -> np.ndarray:
    """Packed grouped weight uint8 [E, N, (K/256)*block_bytes]."""
    nb = in_features // 256
    blocks = random_blocks(qtype, experts * out_features * nb, seed, scale)
    return blocks.reshape(experts, out_features, nb * BLOCK_BYTES[qtype])


def extreme_blocks(qtype: int) -> np.ndarray:
    """A few hand-built blocks: all-zero payload, all-ones payload, alternating bytes, and
    walking bytes, each with d (and dmin) = 1.0, so every field hits its extremes."""
    bb = BLOCK_BYTES[qtype]
    pats = [np.zeros(bb, np.uint8), np.full(bb, 0xFF, np.uint8),
            np.tile(np.array([0xAA, 0x55], np.uint8), bb // 2 + 1)[:bb],
            (np.arange(bb) * 37 % 256).astype(np.uint8),
            (255 - np.arange(bb) * 11 % 256).astype(np.uint8)]
    blocks = np.stack(pats)
    one = np.array([1.0], np.float16).view(np.uint8)
    for off in _FP16_FIELDS[qtype]:
        blocks[:, off:off + 2] = one
    return blocks


def gaussian_bf16(shape, seed: int):
    """bf16 N(0,1) torch tensor on the CPU from a fixed generator."""
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(torch.bfloat16)


def topk_routing(tokens: int, experts: int, top_k: int, seed: int, sigma: float = 2.0):
    """Top-k routing from softmax of Gaussian logits (softmax is monotone, so top-k of the
    logits).  Returns (topk_ids int32 [tokens, top_k])."""
    rng = np.random.Generator(np.random.PCG64(seed))
    logits = rng.standard_normal((tokens, experts), dtype=np.float32) * np.float32(sigma)
    # a fixed per-expert popularity bias makes the counts skewed, as real routers are
    bias = rng.standard_normal(experts, dtype=np.float32) * np.float32(sigma) * np.float32(0.25)
    logits += bias
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :top_k]
    return ids.astype(np.int32)


def sort_by_expert(topk_ids: np.ndarray, experts: int):
    """Host statement of the routing prefix-sum: stable sort of the flattened (token, slot)
    pairs by expert id.  Returns (perm, expert_indices int64, expert_offsets int32) with one
    entry per expert (empty groups included, as the device helper emits them)."""
    flat = topk_ids.reshape(-1)
    perm = np.argsort(flat, kind="stable").astype(np.int64)
    counts = np.bincount(flat, minlength=experts)
    offsets = np.cumsum(counts).astype(np.int32)
    return perm, np.arange(experts, dtype=np.int64), offsets
