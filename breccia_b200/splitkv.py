"""Long single-stream decode split along the KV length across GPUs (BASELINE config 3).

One process per GPU (torch.distributed, NCCL over NVLink).  Rank r of n holds the cells
[r * L / n, (r + 1) * L / n) of the sequence (page-aligned) in its own pool, under a local block table
whose cell 0 is the first cell of its range.  A decode step per layer is
    local split-KV attention -> un-normalised (acc, m, l) per head   brc_decode_partial
    all-gather of the 16 512-byte partials over NVLink               ncclAllGather
    log-sum-exp merge of the n partials, gate, output                brc_decode_combine
This is the only collective on the whole path (batched decode shards by sequence and needs none).
The reference has no counterpart: its split-K partials never leave one device
(crates/breccia-kernels/src/qsa/mod.rs:1491-1521).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ._lib import DTYPE_F16
from .qsa import DecodeBatch, KvPool, decode_combine, decode_partial_bytes


def kv_range(rank: int, world: int, n_tokens: int, page_tokens: int = 16) -> tuple[int, int]:
    """Cells [begin, end) of rank `rank`: contiguous, page-aligned cuts, the remainder spread over the
    first ranks; the last range ends at n_tokens."""
    n_pages = (n_tokens + page_tokens - 1) // page_tokens
    base, extra = divmod(n_pages, world)
    first = rank * base + min(rank, extra)
    last = first + base + (1 if rank < extra else 0)
    return min(first * page_tokens, n_tokens), min(last * page_tokens, n_tokens)


class SplitKvDecode:
    """This rank's share of one long sequence and the machinery of a split-KV decode step."""

    def __init__(self, pool: KvPool, n_head: int, local_table: np.ndarray, local_len: int, group=None,
                 q_dtype: int = DTYPE_F16):
        self.pool, self.n_head, self.group = pool, n_head, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.batch = DecodeBatch(pool, n_head, np.asarray(local_table, np.uint32)[None, :], [local_len], q_dtype=q_dtype)
        self.part_bytes = decode_partial_bytes(1, n_head, pool.head_dim)
        dev = f"cuda:{pool.device}"
        self.partial = torch.zeros(self.part_bytes, dtype=torch.uint8, device=dev)
        self.gathered = torch.zeros(self.world * self.part_bytes, dtype=torch.uint8, device=dev)

    def attend(self, layer: int, q: torch.Tensor, out: torch.Tensor, gate=None, gate_head_stride: int = 0) -> None:
        """q [1, n_head, hd] (the same on every rank) -> out [1, n_head, hd] f32 (the same on every rank)."""
        self.batch.partial(layer, q, self.partial)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.partial, group=self.group)
        else:
            self.gathered.copy_(self.partial)
        decode_combine(self.pool.device, self.gathered, self.world, self.part_bytes, 1, self.n_head, self.pool.head_dim, out,
                       gate=gate, gate_head_stride=gate_head_stride)
