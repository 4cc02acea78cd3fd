"""Shared builders for the GPU parity tests: seeded pools, tables and oracle-side mirrors."""
from __future__ import annotations

import numpy as np
import torch

import oracle
from breccia_b200 import synth
from breccia_b200.qsa import KvPool


def fill_pool_from_host(pool: KvPool, layer: int, seed: int, std: float = 0.5):
    """Write seeded N(0, std^2) values, encoded by the reference store rule, into one layer's K and V
    pools; return the uint16 host copies."""
    n = pool.n_pages * pool.n_kv_head * pool.page_tokens * pool.head_dim
    k = oracle.f32_to_f16_bits_np(synth.normal(seed, n, std))
    v = oracle.f32_to_f16_bits_np(synth.normal(seed + 1, n, std))
    pool.write(0, layer, k)
    pool.write(1, layer, v)
    return k, v


def dev_u32(a, device=0) -> torch.Tensor:
    return torch.as_tensor(np.ascontiguousarray(a, np.uint32).astype(np.int32), device=f"cuda:{device}")


def attention_errors(got: np.ndarray, want: np.ndarray):
    """(max abs, max rel as the target defines it, reference measure max|g-w|/max(|w|,1))."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    diff = np.abs(got - want)
    max_abs = float(diff.max()) if diff.size else 0.0
    # relative error where the reference value is not tiny; tiny values are covered by the abs bar
    big = np.abs(want) > 2e-2
    max_rel = float((diff[big] / np.abs(want[big])).max()) if big.any() else 0.0
    ref_measure = float((diff / np.maximum(np.abs(want), 1.0)).max()) if diff.size else 0.0
    return max_abs, max_rel, ref_measure


ATTN_MAX_ABS = 2e-3   # target: max-abs 2e-3
ATTN_MAX_REL = 1e-2   # target: max-rel 1e-2
