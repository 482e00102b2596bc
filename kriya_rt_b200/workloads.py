"""Seeded synthetic workloads shaped like the benchmark configurations.

The reference measures through a whole model on text prompts; this path is measured on synthetic
activations instead: fp32 N(0,1) draws rounded once to the storage dtype, block tables drawn as a seeded
permutation of the pool.  The rounded values are the inputs of both the CUDA kernels and the CPU oracle.
Everything here is host-side numpy; nothing touches the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

BF16, FP16 = 0, 1


def to_storage(x: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 -> 16-bit storage bit patterns (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == FP16:
        return x.astype(np.float16).view(np.uint16)
    u = x.view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def from_storage(b: np.ndarray, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    if dtype == FP16:
        return b.view(np.float16).astype(np.float32)
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass
class AttnShape:
    name: str
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    dtype: int
    num_layers: int = 1
    block_size: int = 16
    rope_theta: float = 10000.0

    @property
    def kv_bytes_per_token(self) -> int:  # K and V, one layer
        return 2 * self.num_kv_heads * self.head_dim * 2


SMOLLM2_135M = AttnShape("SmolLM2-135M", 9, 3, 64, FP16, num_layers=30)
QWEN25_3B = AttnShape("Qwen2.5-3B", 16, 2, 128, BF16, num_layers=36, rope_theta=1000000.0)
QWEN25_1P5B = AttnShape("Qwen2.5-1.5B", 12, 2, 128, BF16, num_layers=28, rope_theta=1000000.0)


@dataclass
class DecodeBatch:
    """One decode step's plan: each row holds `context[i]` cached tokens and receives one new token."""

    shape: AttnShape
    num_blocks: int
    context: np.ndarray  # int [B] tokens already cached (= position of the new token)
    page_indptr: np.ndarray  # int32 [B+1], tables AFTER reserving the new token's slot
    page_indices: np.ndarray  # int32
    last_page_len: np.ndarray  # int32 [B], after the append
    positions: np.ndarray  # uint32 [B]
    tiles: np.ndarray = field(default_factory=lambda: np.zeros((0, 4), np.uint32))

    @property
    def cta_work_tiles(self) -> np.ndarray:  # same field name as FlashInferSchedulePlan
        return self.tiles

    @property
    def batch(self) -> int:
        return int(self.context.size)

    @property
    def attended_tokens(self) -> int:
        return int((self.context + 1).sum())

    @property
    def kv_bytes_per_layer(self) -> int:
        return self.attended_tokens * self.shape.kv_bytes_per_token


def reference_tiles(page_indptr: np.ndarray, max_blocks_per_cta: int = 8) -> np.ndarray:
    """CtaWorkTile rows as build_schedule_plan cuts them (crates/kriya-kv/src/bsr_paged.rs:522-532)."""
    out = []
    cap = max(max_blocks_per_cta, 1)
    for r in range(page_indptr.size - 1):
        nb = int(page_indptr[r + 1] - page_indptr[r])
        for start in range(0, nb, cap):
            out.append((r, start, min(nb - start, cap), 1 if nb > cap else 0))
    return np.asarray(out, dtype=np.uint32).reshape(-1, 4)


def make_decode_batch(shape: AttnShape, context: np.ndarray, num_blocks: int, seed: int,
                      step: int = 0) -> DecodeBatch:
    """Block tables are the leading entries of a seeded permutation of the pool, dealt to rows in order.
    Every row is given enough blocks for `context + step + 1` tokens, so the same table serves a run of
    decode steps; `step` selects how many tokens are counted as present."""
    rng = np.random.default_rng(seed)
    bs = shape.block_size
    ctx = np.asarray(context, dtype=np.int64) + step
    nblk = (ctx + 1 + bs - 1) // bs
    total = int(nblk.sum())
    if total > num_blocks:
        raise ValueError(f"workload needs {total} blocks, pool has {num_blocks}")
    perm = rng.permutation(num_blocks).astype(np.int32)
    indptr = np.zeros(ctx.size + 1, np.int32)
    indptr[1:] = np.cumsum(nblk)
    indices = perm[:total].copy()
    last = ((ctx % bs) + 1).astype(np.int32)
    b = DecodeBatch(shape, num_blocks, ctx, indptr, indices, last, ctx.astype(np.uint32))
    b.tiles = reference_tiles(indptr, 8)
    return b


def growing_decode_tables(shape: AttnShape, context: np.ndarray, num_blocks: int, seed: int, steps: int):
    """Tables for a run of `steps` decode steps over fixed physical blocks: row i owns a fixed list of blocks
    long enough for context[i] + steps tokens; step t uses the first ceil((context[i]+t+1)/16) of them."""
    rng = np.random.default_rng(seed)
    bs = shape.block_size
    ctx = np.asarray(context, dtype=np.int64)
    cap = (ctx + steps + bs - 1) // bs
    total = int(cap.sum())
    if total > num_blocks:
        raise ValueError(f"workload needs {total} blocks, pool has {num_blocks}")
    perm = rng.permutation(num_blocks).astype(np.int32)
    starts = np.zeros(ctx.size + 1, np.int64)
    starts[1:] = np.cumsum(cap)
    owned = [perm[starts[i]:starts[i + 1]] for i in range(ctx.size)]

    def at_step(t: int) -> DecodeBatch:
        c = ctx + t
        nblk = (c + 1 + bs - 1) // bs
        indptr = np.zeros(ctx.size + 1, np.int32)
        indptr[1:] = np.cumsum(nblk)
        indices = np.concatenate([owned[i][:nblk[i]] for i in range(ctx.size)]).astype(np.int32)
        last = ((c % bs) + 1).astype(np.int32)
        b = DecodeBatch(shape, num_blocks, c, indptr, indices, last, c.astype(np.uint32))
        b.tiles = reference_tiles(indptr, 8)
        return b

    return at_step


def normal16(rng: np.random.Generator, shape, dtype: int) -> np.ndarray:
    return to_storage(rng.standard_normal(shape, dtype=np.float32), dtype)


def config1(seed_tensors: int = 1001, seed_tables: int = 2001, dtype: Optional[int] = None):
    """SmolLM2-135M attention shape, batch 4, contexts {64,128,200,255}, 64-block pool, one layer."""
    shape = AttnShape(**{**SMOLLM2_135M.__dict__, "num_layers": 1})
    if dtype is not None:
        shape.dtype = dtype
    batch = make_decode_batch(shape, np.array([64, 128, 200, 255]), 64, seed_tables)
    rng = np.random.default_rng(seed_tensors)
    B, Hq, Hkv, D = 4, shape.num_q_heads, shape.num_kv_heads, shape.head_dim
    data = {
        "q": normal16(rng, (B, Hq, D), shape.dtype),
        "k": normal16(rng, (B, Hkv, D), shape.dtype),
        "v": normal16(rng, (B, Hkv, D), shape.dtype),
        "cache_k": normal16(rng, (64, 16, Hkv, D), shape.dtype),
        "cache_v": normal16(rng, (64, 16, Hkv, D), shape.dtype),
    }
    return shape, batch, data


def config2_contexts(seed_tables: int = 2002, batch: int = 32, lo: int = 512, hi: int = 4096) -> np.ndarray:
    rng = np.random.default_rng(seed_tables)
    return rng.integers(lo, hi + 1, size=batch)
