"""CPU restatement (NumPy float64) of the reference's indexer functions in front of the top-k selection.

TEST INFRASTRUCTURE: only tests/ may import this.  It follows
  crates/breccia-kernels/src/qsa/cpu.rs:159-195  pool_keys      pooled[b] = rope(rmsnorm(mean(raw[4b..4b+3])), pos = 4b);
                                                                the mean accumulates raw / 4 in f32, cell after cell
  crates/breccia-kernels/src/qsa/cpu.rs:97-121   indexer_score  (1/sqrt(idx_dim)) * sum_h relu(q_h . pooled_b) in f64,
                                                                -inf for a block that starts after the query's position
  crates/breccia-kernels/src/qsa/mod.rs:1673-1687 blocks_completed
and, for rows of a chunk, the GPU path's stricter mask (shaders/qsa_idx_score.comp:74-81: a block whose LAST cell
lies beyond the row's position is dead), selected with `mask="last"`.  Parity unpinned: the reference holds no
golden vectors for these functions (its tests compare its GPU with this same arithmetic within 1e-5 and id for id).
"""
from __future__ import annotations

import numpy as np

from .prepare_ref import rmsnorm, rope_apply


def blocks_completed(pos0: int, tokens: int, idx_block: int = 4):
    if tokens == 0:
        return 0, 0
    last = pos0 + tokens - 1
    if last < idx_block - 1:
        return 0, 0
    b0 = pos0 // idx_block
    b_last = (last - (idx_block - 1)) // idx_block
    if b_last < b0:
        return b0, 0
    return b0, b_last - b0 + 1


def pool_keys(raw, cells: int, gamma, table, idx_dim: int = 128, idx_block: int = 4, n_rot: int = 64, eps: float = 1e-6) -> np.ndarray:
    """raw [cells, idx_dim] f32 (the whole sequence's raw keys) -> pooled [cells // idx_block, idx_dim] f32."""
    raw = np.asarray(raw, np.float32).reshape(-1, idx_dim)
    n_blocks = cells // idx_block
    mean = np.zeros((n_blocks, idx_dim), np.float32)
    for k in range(idx_block):   # f32 accumulation of raw / idx_block, cell after cell, as the reference's loop
        mean += raw[k:n_blocks * idx_block:idx_block] / np.float32(idx_block)
    normed = rmsnorm(mean, idx_dim, gamma, eps)
    return rope_apply(normed, idx_dim, n_rot, table, np.arange(n_blocks) * idx_block)


def indexer_score(q, pooled, n_blocks: int, pos: int, idx_n_head: int = 4, idx_dim: int = 128, idx_block: int = 4,
                  mask: str = "first") -> np.ndarray:
    """q [idx_n_head, idx_dim], pooled [>= n_blocks, idx_dim] -> scores [n_blocks] f64 (-inf = dead block)."""
    q64 = np.asarray(q, np.float32).astype(np.float64).reshape(idx_n_head, idx_dim)
    p64 = np.asarray(pooled, np.float32).astype(np.float64).reshape(-1, idx_dim)[:n_blocks]
    dots = p64 @ q64.T                                   # [n_blocks, heads]
    out = np.maximum(dots, 0.0).sum(axis=1) * (1.0 / np.sqrt(np.float64(idx_dim)))
    b = np.arange(n_blocks)
    dead = b * idx_block > pos if mask == "first" else b * idx_block + idx_block - 1 > pos
    out[dead] = -np.inf
    return out
