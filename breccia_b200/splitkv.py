"""Long single-stream decode split along the KV length across GPUs (the long-context single-stream workload).

One process per GPU (torch.distributed, NCCL over NVLink).  Rank r of n holds the cells
[r * L / n, (r + 1) * L / n) of the sequence (page-aligned) in its own pool, under a local block table
whose cell 0 is the first cell of its range.  A decode step per layer is
    local split-KV attention -> un-normalised (acc, m, l) per head   brc_decode_partial
    exchange of the 16 512-byte partials over NVLink + merge + gate  one kernel (brc_splitkv_attend)
The exchange kernel stores this rank's partial into a receive buffer of every peer (mapped once
through CUDA IPC; the 64-byte handles travel by torch.distributed at set-up), releases a flag, waits
with a time limit for the peers' flags and merges.  `exchange="nccl"` keeps the plain composition
brc_decode_partial -> ncclAllGather -> brc_decode_combine as the baseline to compare against.
This is the only exchange on the whole path (batched decode shards by sequence and needs none).
The reference has no counterpart: its split-K partials never leave one device
(crates/breccia-kernels/src/qsa/mod.rs:1491-1521).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from ._lib import DTYPE_F16
from .qsa import DecodeBatch, KvPool, _ptr, _stream_ptr, decode_combine, decode_partial_bytes

IPC_HANDLE_BYTES = 64


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
                 q_dtype: int = DTYPE_F16, exchange: str = "p2p", max_layers: int = 1):
        """`max_layers` sizes the exchange buffers for `step`, which moves the partials of that many
        layers with one kernel."""
        if exchange not in ("p2p", "nccl"):
            raise ValueError("exchange is 'p2p' or 'nccl'")
        self.pool, self.n_head, self.group, self.exchange = pool, n_head, group, exchange
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.batch = DecodeBatch(pool, n_head, np.asarray(local_table, np.uint32)[None, :], [local_len], q_dtype=q_dtype)
        self.part_bytes = decode_partial_bytes(1, n_head, pool.head_dim)
        dev = f"cuda:{pool.device}"
        self.comm = None
        if exchange == "nccl":
            self.partial = torch.zeros(self.part_bytes, dtype=torch.uint8, device=dev)
            self.gathered = torch.zeros(self.world * self.part_bytes, dtype=torch.uint8, device=dev)
            return
        comm = C.c_void_p()
        self.max_layers = max_layers
        _lib.call("brc_comm_create", pool.handle, self.world, self.rank, max_layers, n_head, C.byref(comm))
        self.comm = comm
        if self.world > 1:
            mine = (C.c_uint8 * IPC_HANDLE_BYTES)()
            _lib.call("brc_comm_ipc_handle", comm, C.cast(mine, C.c_void_p))
            handles = self._all_gather_bytes(bytes(mine), dev)
            buf = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
            _lib.call("brc_comm_connect_ipc", comm, C.cast(buf, C.c_void_p), self.world)
            dist.barrier(group=self.group)   # every rank has mapped every buffer before the first store

    def _all_gather_bytes(self, payload: bytes, dev: str) -> bytes:
        """The same-sized byte strings of all ranks, in rank order (through the process group's backend)."""
        cpu = dist.get_backend(self.group) == "gloo"
        mine = torch.frombuffer(bytearray(payload), dtype=torch.uint8).to("cpu" if cpu else dev)
        out = torch.empty(self.world * len(payload), dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(out, mine, group=self.group)
        return out.cpu().numpy().tobytes()

    def attend(self, layer: int, q: torch.Tensor, out: torch.Tensor, gate=None, gate_head_stride: int = 0) -> None:
        """q [1, n_head, hd] (the same on every rank) -> out [1, n_head, hd] f32 (the same on every rank)."""
        b = self.batch
        if self.comm is not None:
            _lib.call("brc_splitkv_attend", self.comm, layer, _ptr(q), b.q_dtype, _ptr(gate) if gate is not None else None,
                      gate_head_stride, _ptr(b.block_tables), b.table_stride, _ptr(b.seq_lens), 1, b.capacity, b.scale,
                      _ptr(out), _ptr(b.scratch), b.scratch.numel(), _stream_ptr())
            return
        b.partial(layer, q, self.partial)
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.partial, group=self.group)
            parts = self.gathered
        else:
            parts = self.partial
        decode_combine(self.pool.device, parts, self.world, self.part_bytes, 1, self.n_head, self.pool.head_dim, out,
                       gate=gate, gate_head_stride=gate_head_stride)

    def step(self, q: torch.Tensor, out: torch.Tensor, layer0: int = 0) -> None:
        """One decode token over the layers q carries, the layers' attention calls being independent of
        one another: q [L, 1, n_head, hd] -> out [L, 1, n_head, hd] f32 (contiguous).  One launch streams the
        local cells of all layers, pushes the merged partials to the peers and merges theirs (brc_splitkv_step)."""
        b = self.batch
        if self.comm is None:
            for i in range(q.shape[0]):
                self.attend(layer0 + i, q[i], out[i])
            return
        if not out.is_contiguous():
            raise ValueError("out must be contiguous")
        _lib.call("brc_splitkv_step", self.comm, layer0, q.shape[0], _ptr(q), b.q_dtype, q.stride(0) * q.element_size(), None, 0,
                  _ptr(b.block_tables), b.table_stride, _ptr(b.seq_lens), 1, b.capacity, b.scale, _ptr(out), _ptr(b.scratch),
                  b.scratch.numel(), _stream_ptr())

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (all ranks, after their last step)."""
        if self.comm is not None:
            if self.world > 1:
                torch.cuda.synchronize()
                dist.barrier(group=self.group)   # nobody unmaps while a peer may still store
            _lib.call("brc_comm_destroy", self.comm)
            self.comm = None
