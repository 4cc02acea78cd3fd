"""CPU restatement (NumPy float64) of the steps in front of the cache in the reference's Qsa::forward:
per-head RMSNorm of q and k and the partial NEOX rotary, as the reference's own CPU code computes them.

TEST INFRASTRUCTURE: only tests/ may import this.  It follows, function by function,
  crates/breccia-kernels/src/ops/cpu.rs:52-88    rmsnorm     (f64 sum of squares, inv = 1/sqrt(ss/cols + eps),
                                                              out = x * inv * gamma cast to f32)
  crates/breccia-kernels/src/ops/cpu.rs:103-117  rope_table  (inv = base^(-2i/n_rot), ang = pos * inv in f64,
                                                              (cos, sin) rounded to f32)
  crates/breccia-kernels/src/ops/cpu.rs:124-153  rope_apply  (pairs (j, j + n_rot/2); position clamped into the
                                                              table; dims [n_rot, head_dim) copied)
and the order of Qsa::forward (crates/breccia-kernels/src/qsa/mod.rs:1607-1617): q_norm, k_norm, rope_q, rope_k,
kv_append.  Parity unpinned: the reference holds no golden vectors for these steps (its tests compare its GPU
with this same f64 arithmetic within a bar).
"""
from __future__ import annotations

import numpy as np


def rmsnorm(x, cols: int, gamma, eps: float) -> np.ndarray:
    """Rows of `cols` elements; one gamma vector for all rows (wgroups = 1)."""
    x64 = np.asarray(x, np.float32).astype(np.float64).reshape(-1, cols)
    ss = (x64 * x64).sum(axis=1, keepdims=True)
    inv = 1.0 / np.sqrt(ss / cols + np.float64(np.float32(eps)))
    return (x64 * inv * np.asarray(gamma, np.float32).astype(np.float64)[None, :]).astype(np.float32)


def rope_table(freq_base: float, n_rot: int, max_pos: int) -> np.ndarray:
    """[max_pos][n_rot/2][2] f32 (cos, sin)."""
    half = n_rot // 2
    inv = np.float64(freq_base) ** (-2.0 * np.arange(half, dtype=np.float64) / n_rot)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def rope_apply(x, head_dim: int, n_rot: int, table, positions) -> np.ndarray:
    """x: rows of head_dim; positions: one per row."""
    x32 = np.asarray(x, np.float32).reshape(-1, head_dim)
    t = np.asarray(table, np.float32).astype(np.float64)
    half = n_rot // 2
    p = np.clip(np.asarray(positions, np.int64), 0, t.shape[0] - 1)
    a = x32[:, :half].astype(np.float64)
    b = x32[:, half:n_rot].astype(np.float64)
    c, s = t[p, :, 0], t[p, :, 1]
    out = x32.copy()
    out[:, :half] = (a * c - b * s).astype(np.float32)
    out[:, half:n_rot] = (a * s + b * c).astype(np.float32)
    return out


def prepare(q_full, k_cur, v_cur, q_gamma, k_gamma, eps: float, table, n_rot: int, positions, n_head: int, n_kv_head: int,
            head_dim: int, q_head_stride: int):
    """q_full [T, n_head, q_head_stride], k_cur / v_cur [T, n_kv * hd], positions [T]
    -> (q [T, n_head, hd] f32, k [T, n_kv * hd] f32 to append, v unchanged)."""
    T = np.asarray(positions).size
    q = np.asarray(q_full, np.float32).reshape(T, n_head, q_head_stride)[:, :, :head_dim]
    q = rmsnorm(q, head_dim, q_gamma, eps)
    q = rope_apply(q, head_dim, n_rot, table, np.repeat(np.asarray(positions), n_head))
    k = rmsnorm(np.asarray(k_cur, np.float32).reshape(T * n_kv_head, head_dim), head_dim, k_gamma, eps)
    k = rope_apply(k, head_dim, n_rot, table, np.repeat(np.asarray(positions), n_kv_head))
    return q.reshape(T, n_head, head_dim), k.reshape(T, n_kv_head * head_dim), np.asarray(v_cur, np.float32)
