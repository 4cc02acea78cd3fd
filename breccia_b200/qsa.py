"""Host-side mirror of the reference's `breccia-kernels::qsa` operator surface over libbreccia_kv.

Same names, argument meaning and error behaviour as the reference's `QsaState` / `QsaWorkspace` /
`Qsa` (crates/breccia-kernels/src/qsa/mod.rs:294-311, 606-650, 1107-1156, 1365-1580), so tests read
like the reference's own; the difference is that ONE pool per GPU is shared by all sequences and a
sequence is a block table into it.  `DecodeBatch` is the batched form the engine's decode loop uses.

torch is used for device buffers and streams only; every operator is a call through the C ABI.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from . import _lib
from ._lib import BrcError, DTYPE_F16, DTYPE_F32

PAGE_CELLS = 16  # crates/breccia-kernels/src/qsa/mod.rs:114


def _ptr(t) -> C.c_void_p:
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream_ptr(stream=None) -> C.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _u32_array(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


class KvPool:
    """Paged f16 K/V pools of all layers on one GPU plus the page allocator (brc_pool).  v_q8: V page bodies
    as q8_0 blocks (the reference's VLayout::Q8_0, qsa/mod.rs:245-349): K stays binary16, append quantises
    from f32, and every operator reads the blocks."""

    def __init__(self, device: int, n_layers: int, n_kv_head: int, head_dim: int, n_pages: int,
                 page_tokens: int = PAGE_CELLS, bookkeeping_only: bool = False, v_q8: bool = False):
        self._h = C.c_void_p()
        self.v_q8 = v_q8
        if v_q8:
            _lib.call("brc_pool_create_q8v", device, n_layers, n_kv_head, head_dim, page_tokens, n_pages, C.byref(self._h))
        elif bookkeeping_only:
            _lib.call("brc_pool_create_bookkeeping", n_layers, n_kv_head, head_dim, page_tokens, n_pages,
                      C.byref(self._h))
        else:
            _lib.call("brc_pool_create", device, n_layers, n_kv_head, head_dim, page_tokens, n_pages,
                      C.byref(self._h))
        self.device = device
        self.n_layers, self.n_kv_head, self.head_dim = n_layers, n_kv_head, head_dim
        self.n_pages, self.page_tokens = n_pages, page_tokens
        self.half_page_bytes = n_kv_head * page_tokens * head_dim * 2

    # -- lifetime
    @property
    def handle(self) -> C.c_void_p:
        if not self._h:
            raise BrcError(_lib.ERR_INVALID, "pool already released")
        return self._h

    def release(self) -> None:
        if self._h:
            _lib.call("brc_pool_destroy", self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def bytes(self) -> int:
        out = C.c_uint64()
        _lib.call("brc_pool_bytes", self.handle, C.byref(out))
        return out.value

    def zero(self, stream=None) -> None:
        _lib.call("brc_pool_zero", self.handle, _stream_ptr(stream))

    def poison_nan(self, stream=None) -> None:
        _lib.call("brc_pool_poison_nan", self.handle, _stream_ptr(stream))

    def check(self, stream=None) -> None:
        """Synchronise and raise if any kernel refused an index or gave up a wait."""
        _lib.call("brc_pool_check", self.handle, _stream_ptr(stream))

    def k_ptr(self, layer: int) -> int:
        out = C.c_void_p()
        _lib.call("brc_pool_k_ptr", self.handle, layer, C.byref(out))
        return out.value

    def v_ptr(self, layer: int) -> int:
        out = C.c_void_p()
        _lib.call("brc_pool_v_ptr", self.handle, layer, C.byref(out))
        return out.value

    def read(self, which: int, layer: int) -> np.ndarray:
        """Whole K (0) or V (1) pool of a layer as uint16 [n_pages, n_kv, page_tokens, head_dim]."""
        if which == 1 and self.v_q8:   # raw q8_0 rows: [n_pages * n_kv * page_tokens, head_dim / 32 * 36] bytes
            out = np.empty((self.n_pages * self.n_kv_head * self.page_tokens, self.head_dim // 32 * 36), np.uint8)
        else:
            out = np.empty((self.n_pages, self.n_kv_head, self.page_tokens, self.head_dim), np.uint16)
        _lib.call("brc_pool_read", self.handle, which, layer, 0, out.ctypes.data_as(C.c_void_p), out.nbytes,
                  _stream_ptr())
        return out

    def write(self, which: int, layer: int, data: np.ndarray, byte_offset: int = 0) -> None:
        data = np.ascontiguousarray(data)
        _lib.call("brc_pool_write", self.handle, which, layer, byte_offset, data.ctypes.data_as(C.c_void_p),
                  data.nbytes, _stream_ptr())

    # -- allocator
    def alloc(self, n: int) -> np.ndarray:
        ids = np.empty(n, np.uint32)
        _lib.call("brc_pages_alloc", self.handle, n, ids.ctypes.data_as(C.POINTER(C.c_uint32)))
        return ids

    def retain(self, ids) -> None:
        ids = _u32_array(ids)
        _lib.call("brc_pages_retain", self.handle, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size)

    def release_pages(self, ids) -> None:
        ids = _u32_array(ids)
        _lib.call("brc_pages_release", self.handle, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size)

    def refcount(self, page: int) -> int:
        out = C.c_uint32()
        _lib.call("brc_page_refcount", self.handle, page, C.byref(out))
        return out.value

    def free_count(self) -> int:
        out = C.c_uint32()
        _lib.call("brc_pages_free_count", self.handle, C.byref(out))
        return out.value

    # -- page movers
    def copy_pages(self, src_ids, dst_ids, stream=None) -> None:
        src = torch.as_tensor(_u32_array(src_ids).astype(np.int32), device=f"cuda:{self.device}")
        dst = torch.as_tensor(_u32_array(dst_ids).astype(np.int32), device=f"cuda:{self.device}")
        _lib.call("brc_page_copy", self.handle, _ptr(src), _ptr(dst), src.numel(), _stream_ptr(stream))
        torch.cuda.current_stream().synchronize()  # src/dst tensors die with this frame

    def fork(self, parent_table, n_tokens: int, stream=None):
        """Copy-on-write fork -> (child table, id of the private last page or None)."""
        parent = _u32_array(parent_table)
        n_pages = (n_tokens + self.page_tokens - 1) // self.page_tokens
        child = np.zeros(max(n_pages, 1), np.uint32)
        fresh = C.c_uint32()
        _lib.call("brc_seq_fork", self.handle, parent.ctypes.data_as(C.POINTER(C.c_uint32)), n_tokens,
                  child.ctypes.data_as(C.POINTER(C.c_uint32)), C.byref(fresh), _stream_ptr(stream))
        return child[:n_pages], (None if fresh.value == 0xFFFFFFFF else fresh.value)

    def gather(self, layer: int, block_table_dev: torch.Tensor, n_tokens: int, stream=None):
        """Cells 0..n_tokens-1 of one sequence -> (K, V) tensors [n_tokens, n_kv, head_dim] holding binary16
        bits; on a q8_0 V pool V is the stored rows, uint8 [n_tokens, n_kv, head_dim / 32 * 36]."""
        dev = f"cuda:{self.device}"
        k = torch.empty((n_tokens, self.n_kv_head, self.head_dim), dtype=torch.float16, device=dev)
        v = torch.empty((n_tokens, self.n_kv_head, self.head_dim // 32 * 36), dtype=torch.uint8, device=dev) if self.v_q8 else torch.empty_like(k)
        _lib.call("brc_page_gather", self.handle, layer, _ptr(block_table_dev), block_table_dev.numel(), n_tokens,
                  _ptr(k), _ptr(v), _stream_ptr(stream))
        return k, v


class QsaState:
    """One sequence's view of one layer: a block table into the shared pool
    (reference: per-layer, per-sequence pools behind an identity page table, qsa/mod.rs:294-311)."""

    def __init__(self, pool: KvPool, capacity_cells: int, layer: int = 0, block_table=None):
        self.pool = pool
        self.layer = layer
        n_pages = (capacity_cells + PAGE_CELLS - 1) // PAGE_CELLS
        self.capacity_cells = n_pages * PAGE_CELLS  # rounded up to whole pages like the reference
        self._owned = block_table is None
        self.page_table = pool.alloc(n_pages) if block_table is None else _u32_array(block_table)[:n_pages].copy()
        if self.page_table.size != n_pages:
            raise BrcError(_lib.ERR_INVALID, f"block table of {self.page_table.size} pages for {n_pages} needed")
        self.page_table_dev = torch.as_tensor(self.page_table.astype(np.int32), device=f"cuda:{pool.device}")

    def bytes(self) -> int:
        return self.page_table.size * 2 * self.pool.half_page_bytes

    def release(self) -> None:
        if self._owned and self.page_table is not None:
            self.pool.release_pages(self.page_table)
        self.page_table = None


class QsaWorkspace:
    """Device buffers of one call (reference: qsa/mod.rs:606-650): k_cur / v_cur [T, n_kv*hd] f32,
    q [T, n_head, hd] (f32, or f16 when q_dtype says so), q_full [T, n_head*2*hd] f32 whose second
    half per head is the gate, attn_out [T, n_head, hd] f32."""

    def __init__(self, pool: KvPool, tokens: int, n_head: int, q_dtype: int = DTYPE_F32):
        dev = f"cuda:{pool.device}"
        hd, nkv = pool.head_dim, pool.n_kv_head
        self.tokens, self.n_head, self.q_dtype = tokens, n_head, q_dtype
        self.k_cur = torch.zeros((tokens, nkv * hd), dtype=torch.float32, device=dev)
        self.v_cur = torch.zeros_like(self.k_cur)
        self.q = torch.zeros((tokens, n_head, hd), dtype=torch.float32 if q_dtype == DTYPE_F32 else torch.float16,
                             device=dev)
        self.q_full = None  # set to a [T, n_head*2*hd] f32 tensor to enable the gate
        self.attn_out = torch.zeros((tokens, n_head, hd), dtype=torch.float32, device=dev)
        self.seq_lens = torch.zeros(tokens, dtype=torch.int32, device=dev)
        self.pos0 = torch.zeros(1, dtype=torch.int32, device=dev)
        ws_bytes = C.c_uint64()
        _lib.call("brc_decode_workspace_bytes", pool.handle, tokens, n_head, C.byref(ws_bytes))
        self.scratch = torch.empty(ws_bytes.value, dtype=torch.uint8, device=dev)
        self.tables = None


class Qsa:
    """Operator object (reference: `Qsa`, qsa/mod.rs:746-1580) — stateless here."""

    def __init__(self, pool: KvPool, n_head: int):
        self.pool, self.n_head = pool, n_head
        self.scale = 1.0 / math.sqrt(pool.head_dim)

    def workspace(self, tokens: int, q_dtype: int = DTYPE_F32) -> QsaWorkspace:
        return QsaWorkspace(self.pool, tokens, self.n_head, q_dtype)

    def kv_append(self, state: QsaState, ws: QsaWorkspace, pos0: int) -> None:
        """Append ws.tokens cells at pos0.. (reference: Qsa::kv_append, qsa/mod.rs:1107-1156)."""
        if pos0 + ws.tokens > state.capacity_cells:
            raise BrcError(_lib.ERR_CAPACITY,
                           f"kv_append would write cells {pos0}..{pos0 + ws.tokens} but the cache holds "
                           f"{state.capacity_cells} (a write past the page table reads an unmapped page index "
                           "and can scribble over live cells)")
        ws.pos0.fill_(pos0)
        _lib.call("brc_kv_append", self.pool.handle, state.layer, _ptr(state.page_table_dev),
                  state.page_table_dev.numel(), _ptr(ws.pos0), 1, ws.tokens, None, ws.tokens, pos0 + ws.tokens,
                  _ptr(ws.k_cur), _ptr(ws.v_cur), DTYPE_F32, _stream_ptr())

    def topk_dense(self, ws: QsaWorkspace, pos0: int) -> None:
        """Dense selection: every cell 0..=pos0+t for row t (reference: qsa/mod.rs:1365-1376).  The
        selection is carried as per-row lengths instead of an id list."""
        ws.seq_lens.copy_(torch.arange(pos0 + 1, pos0 + 1 + ws.tokens, dtype=torch.int32))

    def attend_apply(self, state: QsaState, ws: QsaWorkspace, pos0: int) -> None:
        """Scores, softmax, probability-weighted V and gate in one pass (reference: Qsa::attend then
        Qsa::apply, qsa/mod.rs:1382-1580).  Row t sees cells <= pos0 + t."""
        if pos0 + ws.tokens > state.capacity_cells:
            raise BrcError(_lib.ERR_CAPACITY, f"attend at cells {pos0}..{pos0 + ws.tokens} but the cache holds "
                                              f"{state.capacity_cells}")
        hd = self.pool.head_dim
        if ws.tables is None or ws.tables.shape[1] != state.page_table_dev.numel():
            ws.tables = state.page_table_dev.unsqueeze(0).repeat(ws.tokens, 1).contiguous()
        else:
            ws.tables.copy_(state.page_table_dev.unsqueeze(0).expand_as(ws.tables))
        gate, stride = None, 0
        if ws.q_full is not None:
            gate, stride = ws.q_full.view(-1)[hd:], 2 * hd
        _lib.call("brc_paged_decode_attn", self.pool.handle, state.layer, _ptr(ws.q), ws.q_dtype, self.n_head,
                  _ptr(gate), stride, _ptr(ws.tables), ws.tables.shape[1], _ptr(ws.seq_lens), ws.tokens,
                  pos0 + ws.tokens, self.scale, _ptr(ws.attn_out), _ptr(ws.scratch), ws.scratch.numel(),
                  _stream_ptr())

    # The reference splits the work into `attend` (scores + softmax) and `apply` (weighted V + gate);
    # the fused kernel does both, so `attend` runs it and `apply` is the completed second half.
    def attend(self, state: QsaState, ws: QsaWorkspace, pos0: int) -> None:
        self.attend_apply(state, ws, pos0)

    def apply(self, state: QsaState, ws: QsaWorkspace, pos0: int) -> None:
        return None


class DecodeBatch:
    """A batch of sequences decoding together from one shared pool: block tables [n_seqs, stride],
    lengths, and the workspace of the split-KV kernel.  One `append` + `attend` per layer per step."""

    def __init__(self, pool: KvPool, n_head: int, block_tables: np.ndarray, seq_lens: np.ndarray,
                 q_dtype: int = DTYPE_F16):
        dev = f"cuda:{pool.device}"
        self.pool, self.n_head, self.q_dtype = pool, n_head, q_dtype
        bt = _u32_array(block_tables)
        self.n_seqs, self.table_stride = bt.shape
        self.capacity = self.table_stride * pool.page_tokens
        self.seq_lens_host = np.asarray(seq_lens, np.int64).copy()
        self.block_tables = torch.as_tensor(bt.astype(np.int32), device=dev)
        self.seq_lens = torch.as_tensor(self.seq_lens_host.astype(np.int32), device=dev)
        self.pos0 = torch.empty_like(self.seq_lens)
        ws_bytes = C.c_uint64()
        _lib.call("brc_decode_workspace_bytes", pool.handle, self.n_seqs, n_head, C.byref(ws_bytes))
        # partial slots for every layer: brc_decode_step covers all layers of a step in one launch
        self.scratch = torch.empty(pool.n_layers * ws_bytes.value, dtype=torch.uint8, device=dev)
        self.scale = 1.0 / math.sqrt(pool.head_dim)

    def begin_step(self) -> None:
        """One new token per sequence: cells seq_len .. are about to be appended in every layer."""
        if int(self.seq_lens_host.max()) + 1 > self.capacity:
            raise BrcError(_lib.ERR_CAPACITY, f"kv_append would write cell {int(self.seq_lens_host.max())} but each "
                                              f"block table holds {self.capacity}")
        self.pos0.copy_(self.seq_lens)
        self.seq_lens_host += 1
        self.seq_lens.add_(1)

    def append(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, src_dtype: int = DTYPE_F32) -> None:
        """k_new / v_new: [n_seqs, n_kv*hd] at cell pos0[s] of each sequence."""
        _lib.call("brc_kv_append", self.pool.handle, layer, _ptr(self.block_tables), self.table_stride,
                  _ptr(self.pos0), self.n_seqs, 1, None, self.n_seqs, int(self.seq_lens_host.max()), _ptr(k_new),
                  _ptr(v_new), src_dtype, _stream_ptr())

    def attend(self, layer: int, q: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None,
               gate_head_stride: int = 0) -> None:
        _lib.call("brc_paged_decode_attn", self.pool.handle, layer, _ptr(q), self.q_dtype, self.n_head, _ptr(gate),
                  gate_head_stride, _ptr(self.block_tables), self.table_stride, _ptr(self.seq_lens), self.n_seqs,
                  int(self.seq_lens_host.max()), self.scale, _ptr(out), _ptr(self.scratch), self.scratch.numel(),
                  _stream_ptr())

    def step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, out: torch.Tensor, layer0: int = 0,
             kv_dtype: int = DTYPE_F32) -> None:
        """One decode step over the layers q carries: q [L, n_seqs, n_head, hd], k_new / v_new
        [L, n_seqs, n_kv*hd], out [L, n_seqs, n_head, hd] f32.  Positions advance on the device; one
        call into the library (brc_decode_step), asynchronous on the current stream."""
        n_layers = q.shape[0]
        if int(self.seq_lens_host.max()) + 1 > self.capacity:
            raise BrcError(_lib.ERR_CAPACITY, f"decode step would write cell {int(self.seq_lens_host.max())} but each "
                                              f"block table holds {self.capacity}")
        self.seq_lens_host += 1
        _lib.call("brc_decode_step", self.pool.handle, layer0, n_layers, _ptr(self.block_tables), self.table_stride,
                  _ptr(self.seq_lens), _ptr(self.pos0), self.n_seqs, int(self.seq_lens_host.max()), _ptr(q),
                  self.q_dtype, q.stride(0) * q.element_size(), self.n_head, _ptr(k_new), _ptr(v_new), kv_dtype,
                  k_new.stride(0) * k_new.element_size(), None, 0, 0, self.scale, _ptr(out),
                  out.stride(0) * out.element_size(), _ptr(self.scratch), self.scratch.numel(), _stream_ptr())

    def step_part(self, first: int, count: int, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                  out: torch.Tensor, layer0: int = 0, kv_dtype: int = DTYPE_F32) -> None:
        """Layers [first, first + count) of the step `step` would run on the same tensors
        (brc_decode_step_part); the part with first == 0 advances the positions."""
        if first == 0:
            if int(self.seq_lens_host.max()) + 1 > self.capacity:
                raise BrcError(_lib.ERR_CAPACITY, f"decode step would write cell {int(self.seq_lens_host.max())} but "
                                                  f"each block table holds {self.capacity}")
            self.seq_lens_host += 1
        _lib.call("brc_decode_step_part", self.pool.handle, layer0, q.shape[0], first, count, _ptr(self.block_tables),
                  self.table_stride, _ptr(self.seq_lens), _ptr(self.pos0), self.n_seqs, int(self.seq_lens_host.max()),
                  _ptr(q), self.q_dtype, q.stride(0) * q.element_size(), self.n_head, _ptr(k_new), _ptr(v_new), kv_dtype,
                  k_new.stride(0) * k_new.element_size(), None, 0, 0, self.scale, _ptr(out),
                  out.stride(0) * out.element_size(), _ptr(self.scratch), self.scratch.numel(), _stream_ptr())

    def host_staging(self, n_layers: int, kv_dtype: int = DTYPE_F32) -> torch.Tensor:
        """The device buffer step_host needs for steps of n_layers layers."""
        need = C.c_uint64()
        _lib.call("brc_decode_step_host_staging_bytes", self.pool.handle, n_layers, self.n_seqs, self.n_head, self.q_dtype,
                  kv_dtype, C.byref(need))
        return torch.empty(need.value, dtype=torch.uint8, device=self.seq_lens.device)

    def step_host(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor, out_host: torch.Tensor,
                  staging: torch.Tensor | None, layer0: int = 0, parts: int = 1, kv_dtype: int = DTYPE_F32,
                  download: bool = False, upload: bool = False) -> None:
        """The same step for a caller whose activations live in host memory, one call into the library
        (brc_decode_step_host).  Pinned q / k / v are read by the kernels where they lie and the attention
        output is stored straight into a pinned out_host; pageable buffers (or `upload` / `download`) go
        through `staging` (from host_staging()).  `parts` > 1 uploads the layers in groups on a second
        stream; on the machines measured the hand-over between the streams cost more than the hidden copy
        saved, so one part is the default.  Returns when out_host is complete."""
        for t in (q_host, k_host, v_host, out_host):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("step_host takes contiguous host tensors")
        if int(self.seq_lens_host.max()) + 1 > self.capacity:
            raise BrcError(_lib.ERR_CAPACITY, f"decode step would write cell {int(self.seq_lens_host.max())} but each "
                                              f"block table holds {self.capacity}")
        self.seq_lens_host += 1
        _lib.call("brc_decode_step_host", self.pool.handle, layer0, q_host.shape[0], parts,
                  (1 if download else 0) | (2 if upload else 0),
                  _ptr(self.block_tables),
                  self.table_stride, _ptr(self.seq_lens), _ptr(self.pos0), self.n_seqs, int(self.seq_lens_host.max()),
                  _ptr(q_host), self.q_dtype, self.n_head, _ptr(k_host), _ptr(v_host), kv_dtype, self.scale, _ptr(out_host),
                  _ptr(staging), staging.numel() if staging is not None else 0, _ptr(self.scratch), self.scratch.numel(),
                  _stream_ptr())

    def reset_lengths(self, seq_lens) -> None:
        self.seq_lens_host = np.asarray(seq_lens, np.int64).copy()
        self.seq_lens.copy_(torch.as_tensor(self.seq_lens_host.astype(np.int32)))

    def partial(self, layer: int, q: torch.Tensor, partial_out: torch.Tensor) -> None:
        _lib.call("brc_decode_partial", self.pool.handle, layer, _ptr(q), self.q_dtype, self.n_head,
                  _ptr(self.block_tables), self.table_stride, _ptr(self.seq_lens), self.n_seqs,
                  int(self.seq_lens_host.max()), self.scale, _ptr(partial_out), _ptr(self.scratch),
                  self.scratch.numel(), _stream_ptr())


def sparse_attend(pool: KvPool, layer: int, q: torch.Tensor, n_head: int, block_tables: torch.Tensor, pos0: torch.Tensor,
                  rows_per_seq: int, ids: torch.Tensor, counts: torch.Tensor, max_pos_end: int, out: torch.Tensor,
                  gate: torch.Tensor | None = None, gate_head_stride: int = 0) -> None:
    """Attention over selected 4-cell blocks (reference: Qsa::attend + Qsa::apply over the `ids` / `counts` lists of
    its top-k stage, qsa/mod.rs:620-625, 1382-1580).  q [rows, n_head, hd] f32 or f16; ids [rows, max_ids] int32;
    counts [rows]; block_tables [n_seqs, stride]; pos0 [n_seqs]; out [rows, n_head, hd] f32."""
    q_dtype = DTYPE_F32 if q.dtype == torch.float32 else DTYPE_F16
    _lib.call("brc_paged_sparse_attn", pool.handle, layer, _ptr(q), q_dtype, n_head, _ptr(gate), gate_head_stride,
              _ptr(block_tables), block_tables.shape[1], _ptr(pos0), block_tables.shape[0], rows_per_seq, _ptr(ids),
              ids.shape[1], _ptr(counts), max_pos_end, 1.0 / math.sqrt(pool.head_dim), _ptr(out), _stream_ptr())


def topk_blocks(pool: KvPool, scores: torch.Tensor, pos0: torch.Tensor, rows_per_seq: int, topk: int = 512,
                dense: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """The selection lists sparse_attend takes, from indexer scores [rows, n_blocks] f32 (reference: Qsa::topk,
    shaders/qsa_topk.comp): per row the `topk` best blocks in descending score order (ties towards the lower
    block, scores <= -1e29 never), then the row's own block.  Returns (ids [rows, min(n_blocks, topk) + 1] int32,
    counts [rows] int32)."""
    rows, n_blocks = scores.shape
    max_ids = min(n_blocks, topk) + 1
    ids = torch.empty((rows, max_ids), dtype=torch.int32, device=scores.device)
    counts = torch.empty((rows,), dtype=torch.int32, device=scores.device)
    _lib.call("brc_topk_blocks", pool.handle, _ptr(scores), pos0.numel(), rows_per_seq, n_blocks, topk, max_ids, _ptr(pos0),
              1 if dense else 0, _ptr(ids), _ptr(counts), _stream_ptr())
    return ids, counts


IDX_DIM, IDX_BLOCK, IDX_N_HEAD = 128, 4, 4   # crates/breccia-kernels/src/qsa/mod.rs:77-81


class IndexerState:
    """The indexer's key cache of a batch of sequences (reference: `QsaState::idx_pooled` / `idx_tail`, one per
    sequence, qsa/mod.rs:294-311, 353-386): one pooled key per completed 4-cell block and the raw keys of the
    block being filled."""

    def __init__(self, pool: KvPool, n_seqs: int, capacity_cells: int):
        dev = f"cuda:{pool.device}"
        self.pool, self.n_seqs = pool, n_seqs
        self.max_blocks = capacity_cells // IDX_BLOCK + 1          # sizes::max_blocks, qsa/mod.rs:384-387
        self.pooled = torch.zeros((n_seqs, self.max_blocks, IDX_DIM), dtype=torch.float32, device=dev)
        self.tail = torch.zeros((n_seqs, IDX_BLOCK - 1, IDX_DIM), dtype=torch.float32, device=dev)

    def append(self, raw: torch.Tensor, pos0: torch.Tensor, max_pos_end: int, gamma: torch.Tensor, rope_table: torch.Tensor,
               n_rot: int, eps: float = 1e-6) -> None:
        """raw [n_seqs, tokens, 128] f32: this call's raw indexer keys at positions pos0[s] ..: pools every block
        the call completes, then stores the new incomplete block's keys in the tail (Qsa::idx_pool then
        Qsa::idx_tail, the order of Qsa::forward)."""
        n_seqs, tokens = raw.shape[0], raw.shape[1]
        _lib.call("brc_idx_pool", self.pool.handle, _ptr(raw), _ptr(self.tail), _ptr(gamma), _ptr(rope_table), n_rot,
                  rope_table.shape[0], eps, _ptr(pos0), n_seqs, tokens, max_pos_end, IDX_DIM, IDX_BLOCK, _ptr(self.pooled),
                  self.max_blocks, _stream_ptr())
        _lib.call("brc_idx_tail", self.pool.handle, _ptr(raw), _ptr(pos0), n_seqs, tokens, IDX_DIM, IDX_BLOCK, _ptr(self.tail),
                  _stream_ptr())

    def score(self, q: torch.Tensor, pos0: torch.Tensor, rows_per_seq: int, n_blocks: int) -> torch.Tensor:
        """q [rows, idx_n_head, 128] f32 -> scores [rows, n_blocks] f32 (Qsa::idx_score), ready for topk_blocks."""
        rows = q.shape[0]
        scores = torch.empty((rows, n_blocks), dtype=torch.float32, device=q.device)
        _lib.call("brc_idx_score", self.pool.handle, _ptr(q), q.shape[1], _ptr(self.pooled), self.max_blocks, _ptr(pos0),
                  rows // rows_per_seq, rows_per_seq, n_blocks, IDX_DIM, IDX_BLOCK, 1.0 / math.sqrt(IDX_DIM), _ptr(scores),
                  _stream_ptr())
        return scores


def decode_partial_bytes(n_seqs: int, n_head: int, head_dim: int) -> int:
    out = C.c_uint64()
    _lib.call("brc_decode_partial_bytes", n_seqs, n_head, head_dim, C.byref(out))
    return out.value


def decode_combine(device: int, parts: torch.Tensor, n_parts: int, part_stride_bytes: int, n_seqs: int, n_head: int,
                   head_dim: int, out: torch.Tensor, gate: torch.Tensor | None = None,
                   gate_head_stride: int = 0) -> None:
    _lib.call("brc_decode_combine", device, _ptr(parts), n_parts, part_stride_bytes, n_seqs, n_head, head_dim,
              _ptr(gate), gate_head_stride, _ptr(out), _stream_ptr())
