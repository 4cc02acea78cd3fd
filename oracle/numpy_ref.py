"""Second, independent restatement of the reference attention in NumPy float64.

TEST INFRASTRUCTURE: exists only to catch transcription mistakes in
``breccia_oracle.c`` (the two are compared on random cases by the CPU tests).
Follows crates/breccia-kernels/src/qsa/cpu.rs:197-246 (`attend`) written as
array algebra instead of loops.
"""
from __future__ import annotations

import numpy as np


def attend(q, k, v, cells, pos: int, n_head: int, n_kv_head: int, head_dim: int, gate=None) -> np.ndarray:
    q = np.asarray(q, np.float64).reshape(n_head, head_dim)
    k = np.asarray(k, np.float64).reshape(-1, n_kv_head, head_dim)
    v = np.asarray(v, np.float64).reshape(-1, n_kv_head, head_dim)
    cells = np.asarray(cells, np.int64)
    live = cells[cells <= pos]
    out = np.zeros((n_head, head_dim), np.float64)
    for h in range(n_head):
        kvh = h * n_kv_head // n_head
        logits = (k[live, kvh, :] @ q[h]) / np.sqrt(float(head_dim))
        p = np.exp(logits - logits.max())
        p /= p.sum()
        out[h] = p @ v[live, kvh, :]
    if gate is not None:
        g = np.asarray(gate, np.float64).reshape(n_head, head_dim)
        out = out / (1.0 + np.exp(-g))
    return out.astype(np.float32)


def paged_view(pool_u16, block_table, n_cells: int, n_kv_head: int, head_dim: int, page_cells: int = 16):
    """Logical [cell][kv_head][d] uint16 view of a pool laid out
    [page][kv_head][cell_in_page][d] (crates/breccia-kernels/src/qsa/mod.rs:22-28)."""
    pool = np.asarray(pool_u16, np.uint16).reshape(-1, n_kv_head, page_cells, head_dim)
    bt = np.asarray(block_table, np.int64)
    n_pages = (n_cells + page_cells - 1) // page_cells
    pages = pool[bt[:n_pages]]                      # [p, kvh, c, d]
    logical = pages.transpose(0, 2, 1, 3).reshape(n_pages * page_cells, n_kv_head, head_dim)
    return logical[:n_cells]
