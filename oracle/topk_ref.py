"""Top-k block selection on the CPU — TEST INFRASTRUCTURE, never the product.

Follows cpu::topk_blocks (crates/breccia-kernels/src/qsa/cpu.rs:129-151) with the dead-block rule of the shader
that ships (crates/breccia-kernels/shaders/qsa_topk.comp:62, 131-133: a score <= -1e29 ends the selection; NaN never
compares greater): descending score, equal scores towards the lower block index, at most k blocks, then the row's
own block unless already present.  Pinned by the reference's two unit tests of that function (qsa/cpu.rs:518-534),
restated in tests/test_topk_cpu.py."""
from __future__ import annotations

import numpy as np

DEAD = -1.0e29


def topk_blocks(scores, k: int, own_block=None, max_ids: int | None = None) -> list[int]:
    scores = np.asarray(scores, np.float32)
    live = [i for i in range(scores.size) if scores[i] > DEAD]        # NaN fails the comparison
    live.sort(key=lambda i: (-float(scores[i]), i))
    out = live[:min(k, scores.size)]
    if own_block is not None and own_block not in out and (max_ids is None or len(out) < max_ids):
        out.append(int(own_block))
    return out


def dense_blocks(n_blocks: int, own_block: int, max_ids: int) -> list[int]:
    """qsa_topk.comp:76-93: every block up to the row's own, ascending."""
    n = min(n_blocks, own_block + 1, max_ids)
    out = list(range(n))
    if own_block >= n_blocks and n < max_ids:
        out.append(own_block)
    return out
