"""Seeded synthetic inputs for the paged decode path, shaped like the benchmark configurations.

No dataset is involved: contexts, block tables and values all come from a seed.  Block tables
are slices of one seeded permutation of the pool's block ids, so a sequence's blocks are
scattered over the pool the way a long-running allocator leaves them.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Shape:
    """One configuration of the path."""
    name: str
    heads: int
    kv_heads: int
    head_dim: int
    block_tokens: int
    dtype: str            # "f32" | "bf16" | "f16"
    batch: int
    ctx_lo: int
    ctx_hi: int
    layers: int = 1
    steps: int = 1
    scaled: bool = True   # values ~ N(0,1) / sqrt(head_dim); False: N(0,1)

    @property
    def kv_out(self) -> int:
        return self.kv_heads * self.head_dim

    @property
    def elem(self) -> int:
        return 4 if self.dtype == "f32" else 2


# The reference-runnable case: 1 layer, f32, 8 q / 2 kv heads of 64, block 16, prompts 37/128/255/512.
C1 = Shape("c1-f32-gqa4", 8, 2, 64, 16, "f32", 4, 0, 0, layers=1, steps=64, scaled=False)
# MoE-decoder shape: 48 layers, 32 q / 4 kv heads of 128, bf16, block 16, batch 64, ctx U[1024, 4096].
C2 = Shape("c2-bf16-b64-ctx1k-4k", 32, 4, 128, 16, "bf16", 64, 1024, 4096, layers=48, steps=128)
# Long context with a shared prefix: batch 16 x 32768, 8 sequences share 8192 tokens.
C3 = Shape("c3-bf16-b16-ctx32k-prefix8k", 32, 4, 128, 16, "bf16", 16, 32768, 32768, layers=1, steps=256)
# Churn + compaction: 32 q / 8 kv heads of 128, bf16, block 32, pool 65536 blocks at 90 %.
C4 = Shape("c4-bf16-b32-churn", 32, 8, 128, 32, "bf16", 0, 256, 8192, layers=1, steps=1)
# Head-sharded over 8 GPUs: 64 q / 8 kv heads of 128, bf16, block 16, batch 256, ctx U[1024, 16384].
C5 = Shape("c5-bf16-b256-ctx1k-16k-headshard", 64, 8, 128, 16, "bf16", 256, 1024, 16384, layers=1, steps=64)

C1_PROMPTS = (37, 128, 255, 512)


def contexts(shape: Shape, seed: int) -> np.ndarray:
    """Context length per sequence, uniform in [ctx_lo, ctx_hi]."""
    if shape is C1 or shape.name == C1.name:
        return np.array(C1_PROMPTS, dtype=np.int64)
    rng = np.random.default_rng([seed, 0x51])
    return rng.integers(shape.ctx_lo, shape.ctx_hi + 1, size=shape.batch, dtype=np.int64)


def permutation(pool_blocks: int, seed: int) -> np.ndarray:
    return np.random.default_rng([seed, 0x52]).permutation(pool_blocks).astype(np.uint32)


@dataclass
class Tables:
    pos: np.ndarray        # u32[s]: the position of each sequence's newest token
    table_at: np.ndarray   # u32[s]
    blocks: np.ndarray     # u32[sum of table lengths]
    lengths: np.ndarray = field(default=None)


def tables_for(lengths: np.ndarray, block_tokens: int, perm: np.ndarray, offset: int = 0, reserve: int = 0) -> Tables:
    """Tables for sequences holding `lengths` positions (newest token at lengths - 1), blocks
    taken from `perm[offset:]` in order; `reserve` more positions of room per sequence."""
    lengths = np.asarray(lengths, dtype=np.int64)
    nb = (lengths + reserve + block_tokens - 1) // block_tokens
    table_at = np.zeros(len(lengths), dtype=np.uint32)
    table_at[1:] = np.cumsum(nb)[:-1]
    total = int(nb.sum())
    if offset + total > len(perm):
        raise ValueError(f"the pool has {len(perm)} blocks, the tables need {offset + total}")
    return Tables((lengths - 1).astype(np.uint32), table_at, perm[offset:offset + total].copy(), lengths)


def normal(rng: np.random.Generator, shape, scale: float) -> np.ndarray:
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def value_scale(shape: Shape) -> float:
    return 1.0 / float(np.sqrt(shape.head_dim)) if shape.scaled else 1.0


def algorithmic_bytes(shape: Shape, lengths: np.ndarray, unique_positions: int | None = None) -> int:
    """Bytes one decode-attention op must move for one layer: every distinct filled position's
    key and value rows once, the queries in, the f32 outputs out, the block tables and positions."""
    lengths = np.asarray(lengths, dtype=np.int64)
    s = len(lengths)
    positions = int(lengths.sum()) if unique_positions is None else unique_positions
    kv = positions * 2 * shape.kv_out * shape.elem
    qo = s * shape.heads * shape.head_dim * (4 + 4)
    tables = 4 * int(((lengths + shape.block_tokens - 1) // shape.block_tokens).sum()) + 8 * s
    return kv + qo + tables
