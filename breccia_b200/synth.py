"""Seeded synthetic inputs for the benchmark workloads (host-side, NumPy only).

One generator feeds the GPU path, the oracle and the CPU baseline so all three see identical bits:
splitmix64 (counter mode) -> Box-Muller in float64 -> float32.  Block tables are slices of one seeded
permutation of the pool, i.e. pages scattered at random.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """n outputs of splitmix64 started at `seed`, skipping `offset` outputs."""
    with np.errstate(over="ignore"):
        i = np.arange(1 + offset, n + 1 + offset, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform01(seed: int, n: int, offset: int = 0) -> np.ndarray:
    """float64 in (0, 1]."""
    return ((splitmix64(seed, n, offset) >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740992.0)


def normal(seed: int, n: int, std: float = 1.0) -> np.ndarray:
    """n float32 samples of N(0, std^2) (Box-Muller on two uniform streams)."""
    m = (n + 1) // 2
    u1 = uniform01(seed, m)
    u2 = uniform01(seed ^ 0x5DEECE66D, m)
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2.0 * np.pi * u2), r * np.sin(2.0 * np.pi * u2)])[:n]
    return (z * std).astype(np.float32)


def permutation(seed: int, n: int) -> np.ndarray:
    """Seeded permutation of 0..n-1 (argsort of a splitmix64 stream)."""
    return np.argsort(splitmix64(seed, n), kind="stable").astype(np.uint32)


def uniform_ints(seed: int, n: int, lo: int, hi: int) -> np.ndarray:
    """n integers uniform in [lo, hi]."""
    return (lo + (splitmix64(seed, n) % np.uint64(hi - lo + 1))).astype(np.int64)


def scattered_tables(seed: int, seq_lens, page_tokens: int = 16, pool_factor: float = 1.25, extra_tokens: int = 0,
                     min_stride: int = 0):
    """Block tables for sequences of the given lengths (+ room for `extra_tokens` appended later):
    disjoint slices of one seeded permutation of a pool sized ceil(pool_factor x pages needed).
    Returns (tables [n_seqs, stride] uint32, n_pool_pages)."""
    seq_lens = np.asarray(seq_lens, np.int64)
    need = (seq_lens + extra_tokens + page_tokens - 1) // page_tokens
    total = int(need.sum())
    n_pool = int(np.ceil(pool_factor * total))
    perm = permutation(seed, n_pool)
    stride = max(int(need.max()), min_stride)
    tables = np.zeros((seq_lens.size, stride), np.uint32)
    at = 0
    for s, n in enumerate(need):
        tables[s, :n] = perm[at:at + n]
        at += int(n)
    return tables, n_pool
