"""CPU oracle for the paged KV hot path — TEST INFRASTRUCTURE, never the product.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference arm may import this package.  It wraps ``breccia_oracle.c`` (a plain-C
restatement of the reference's CPU algorithm: crates/breccia-kernels/src/qsa/cpu.rs,
crates/breccia-kernels/shaders/f16_storage.glsl, qsa_kv_append.comp) through ctypes.

Parity pin status: codec / layout / sizes are pinned by the reference's own
known-answer tests; attention values are "parity unpinned" (the reference holds
no golden outputs, and it cannot be compiled here: Rust + GLSL).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "breccia_oracle.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_LIB = os.path.join(_OUT_DIR, "libbreccia_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement with gcc (OpenMP for the threaded baseline)."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-std=c11",
           "-Wall", "-Wextra", "-o", _LIB, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


_lib = None

_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u8p = C.POINTER(C.c_uint8)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        L = C.CDLL(_LIB)
        L.brc_ref_f32_to_f16_bits.restype = C.c_uint16
        L.brc_ref_f32_to_f16_bits.argtypes = [C.c_float]
        L.brc_ref_f16_bits_to_f32.restype = C.c_float
        L.brc_ref_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.brc_ref_to_f16.restype = C.c_float
        L.brc_ref_to_f16.argtypes = [C.c_float]
        L.brc_ref_pack_f16x2.restype = C.c_uint32
        L.brc_ref_pack_f16x2.argtypes = [C.c_float, C.c_float]
        L.brc_ref_to_q8_0.restype = C.c_int
        L.brc_ref_to_q8_0.argtypes = [_f32p, C.c_size_t, _f32p]
        for name in ("brc_ref_elem_index",):
            getattr(L, name).restype = C.c_uint64
            getattr(L, name).argtypes = [C.c_uint64] * 7
        for name in ("brc_ref_f16_pool_bytes", "brc_ref_q8v_pool_bytes"):
            getattr(L, name).restype = C.c_uint64
            getattr(L, name).argtypes = [C.c_uint64] * 4
        L.brc_ref_pool_rows.restype = C.c_uint64
        L.brc_ref_pool_rows.argtypes = [C.c_uint64] * 3
        L.brc_ref_page_bytes.restype = C.c_uint64
        L.brc_ref_page_bytes.argtypes = [C.c_uint64] * 3
        L.brc_ref_f16_row_words.restype = C.c_uint64
        L.brc_ref_f16_row_words.argtypes = [C.c_uint64]
        L.brc_ref_q8v_row_words.restype = C.c_uint64
        L.brc_ref_q8v_row_words.argtypes = [C.c_uint64]
        L.brc_ref_kv_append.restype = C.c_int
        L.brc_ref_kv_append.argtypes = [_u32p, _u32p, _u32p, _f32p, _f32p, C.c_uint32, C.c_uint32,
                                        C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64]
        L.brc_ref_gather.restype = None
        L.brc_ref_gather.argtypes = [_u16p, _u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                     _u16p, _f32p]
        L.brc_ref_attend.restype = C.c_int
        L.brc_ref_attend.argtypes = [_f32p, _f32p, _f32p, _u32p, C.c_size_t, C.c_size_t, C.c_size_t,
                                     C.c_size_t, C.c_size_t, _f32p, _f32p]
        L.brc_ref_cells_of.restype = None
        L.brc_ref_cells_of.argtypes = [_u32p, C.c_size_t, C.c_size_t, _u32p]
        L.brc_ref_softmax_rows.restype = None
        L.brc_ref_softmax_rows.argtypes = [_f32p, C.c_size_t, C.c_size_t, _f64p]
        L.brc_ref_decode_batch.restype = C.c_int
        L.brc_ref_decode_batch.argtypes = [_u16p, _u16p, _u32p, C.c_uint32, _u32p, C.c_uint32, _f32p,
                                           _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                           _f32p, C.c_int]
        L.brc_ref_prefill_chunk.restype = C.c_int
        L.brc_ref_prefill_chunk.argtypes = [_u16p, _u16p, _u32p, C.c_uint32, C.c_uint32, _f32p, _f32p,
                                            C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _f32p,
                                            C.c_int]
        L.brc_ref_partial_head.restype = None
        L.brc_ref_partial_head.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t,
                                           C.c_size_t, C.c_size_t, C.c_double, _f64p, _f64p, _f64p]
        L.brc_ref_lse_combine.restype = None
        L.brc_ref_lse_combine.argtypes = [_f64p, _f64p, _f64p, C.c_size_t, C.c_size_t, _f64p]
        L.brc_ref_page_copy.restype = None
        L.brc_ref_page_copy.argtypes = [_u8p, _u8p, C.c_uint64, C.c_uint64, C.c_uint64, _u32p, _u32p,
                                        C.c_size_t]
        L.brc_ref_normalish.restype = None
        L.brc_ref_normalish.argtypes = [C.c_uint64, C.c_size_t, _f32p]
        L.brc_ref_max_rel.restype = C.c_double
        L.brc_ref_max_rel.argtypes = [_f32p, _f64p, C.c_size_t]
        L.brc_ref_f16_rule_mismatches.restype = C.c_uint64
        L.brc_ref_f16_rule_mismatches.argtypes = [C.c_uint32, C.c_uint32, C.c_uint64]
        _lib = L
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t) if a is not None else None


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ----------------------------------------------------------------------------- codec

def f32_to_f16_bits(x) -> np.ndarray:
    """Reference store rule, vectorised over an f32 array -> uint16 bits."""
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    L = lib()
    xf, of = x.reshape(-1), out.reshape(-1)
    for i in range(xf.size):
        of[i] = L.brc_ref_f32_to_f16_bits(float(xf[i]))
    return out


def f32_to_f16_bits_np(x) -> np.ndarray:
    """Same rule in NumPy integer arithmetic (fast path for large test arrays);
    held equal to the C functions by the CPU tests."""
    b = _c(x, np.float32).view(np.uint32)
    sign = (b >> 16) & np.uint32(0x8000)
    mag = b & np.uint32(0x7FFFFFFF)
    e = ((mag >> 23) & np.uint32(0xFF)).astype(np.int64) - 127
    m = mag & np.uint32(0x7FFFFF)
    q = (m >> 13) | np.uint32(0x400)
    rem = m & np.uint32(0x1FFF)
    up = (rem > 0x1000) | ((rem == 0x1000) & ((q & 1) == 1))
    q = q + up.astype(np.uint32)
    carry = q >= 0x800
    q = np.where(carry, q >> 1, q)
    e = e + carry.astype(np.int64)
    body = ((e + 15).astype(np.uint32) << 10) | (q & np.uint32(0x3FF))
    inf = (mag >= 0x477FF000) | (e > 15)
    zero = (((mag >> 23) & np.uint32(0xFF)).astype(np.int64) - 127) < -14
    res = np.where(inf, np.uint32(0x7C00), np.where(zero, np.uint32(0), body))
    return (sign | res).astype(np.uint16)


def f16_bits_to_f32(h) -> np.ndarray:
    """Reference load rule in NumPy: exponent 0 reads as signed zero."""
    h = _c(h, np.uint16).astype(np.uint32)
    sign = (h & 0x8000) << 16
    e = (h >> 10) & 0x1F
    m = h & 0x3FF
    normal = sign | ((e + 112) << 23) | (m << 13)
    special = sign | np.uint32(0x7F800000) | (m << 13)
    out = np.where(e == 0, sign, np.where(e == 31, special, normal)).astype(np.uint32)
    return out.view(np.float32)


def to_f16(x) -> np.ndarray:
    return f16_bits_to_f32(f32_to_f16_bits_np(x))


def normalish(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().brc_ref_normalish(seed, n, _p(out, _f32p))
    return out


def max_rel(got, want) -> float:
    got = _c(got, np.float32).reshape(-1)
    want = _c(want, np.float64).reshape(-1)
    return float(lib().brc_ref_max_rel(_p(got, _f32p), _p(want, _f64p), got.size))


# ----------------------------------------------------------------------------- append / gather

def kv_append(k_pool_words: np.ndarray, v_pool_words: np.ndarray, page_table, k_cur, v_cur, pos0: int,
              n_kv_head: int, head_dim: int, page_cells: int = 16, capacity_cells: int | None = None) -> int:
    """In-place reference append into uint32-word pools of ONE layer."""
    assert k_pool_words.dtype == np.uint32 and v_pool_words.dtype == np.uint32
    pt = _c(page_table, np.uint32)
    k_cur = _c(k_cur, np.float32)
    v_cur = _c(v_cur, np.float32)
    tokens = k_cur.size // (n_kv_head * head_dim)
    if capacity_cells is None:
        capacity_cells = pt.size * page_cells
    return lib().brc_ref_kv_append(_p(k_pool_words, _u32p), _p(v_pool_words, _u32p), _p(pt, _u32p),
                                   _p(k_cur, _f32p), _p(v_cur, _f32p), tokens, pos0, n_kv_head,
                                   head_dim, page_cells, capacity_cells)


def gather(pool_u16: np.ndarray, block_table, n_cells: int, n_kv_head: int, head_dim: int,
           page_cells: int = 16):
    """-> (bits [n_cells, n_kv, hd] uint16, values f32) through the block table."""
    pool_u16 = _c(pool_u16, np.uint16)
    bt = _c(block_table, np.uint32)
    bits = np.empty((n_cells, n_kv_head, head_dim), np.uint16)
    vals = np.empty((n_cells, n_kv_head, head_dim), np.float32)
    lib().brc_ref_gather(_p(pool_u16, _u16p), _p(bt, _u32p), n_cells, n_kv_head, head_dim, page_cells,
                         _p(bits, _u16p), _p(vals, _f32p))
    return bits, vals


# ----------------------------------------------------------------------------- attention

def attend(q, k, v, cells, pos: int, n_head: int, n_kv_head: int, head_dim: int, gate=None) -> np.ndarray:
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    cells = _c(cells, np.uint32)
    g = _c(gate, np.float32) if gate is not None else None
    out = np.empty((n_head, head_dim), np.float32)
    rc = lib().brc_ref_attend(_p(q, _f32p), _p(k, _f32p), _p(v, _f32p), _p(cells, _u32p), cells.size, pos,
                              n_head, n_kv_head, head_dim, _p(g, _f32p), _p(out, _f32p))
    assert rc == 0
    return out


def cells_of(blocks, idx_block: int) -> np.ndarray:
    blocks = _c(blocks, np.uint32)
    out = np.empty(blocks.size * idx_block, np.uint32)
    lib().brc_ref_cells_of(_p(blocks, _u32p), blocks.size, idx_block, _p(out, _u32p))
    return out


def decode_batch(k_pool_u16, v_pool_u16, block_tables, seq_lens, q, n_head: int, n_kv_head: int,
                 head_dim: int, page_cells: int = 16, gate=None, n_threads: int = 0):
    """One layer's batched paged decode attention -> (out [n_seqs, n_head, hd], threads used)."""
    k_pool_u16 = _c(k_pool_u16, np.uint16)
    v_pool_u16 = _c(v_pool_u16, np.uint16)
    bt = _c(block_tables, np.uint32)
    sl = _c(seq_lens, np.uint32)
    q = _c(q, np.float32)
    g = _c(gate, np.float32) if gate is not None else None
    n_seqs = sl.size
    out = np.empty((n_seqs, n_head, head_dim), np.float32)
    used = lib().brc_ref_decode_batch(_p(k_pool_u16, _u16p), _p(v_pool_u16, _u16p), _p(bt, _u32p),
                                      bt.shape[1], _p(sl, _u32p), n_seqs, _p(q, _f32p), _p(g, _f32p),
                                      n_head, n_kv_head, head_dim, page_cells, _p(out, _f32p), n_threads)
    assert used > 0
    return out, used


def prefill_chunk(k_pool_u16, v_pool_u16, block_table, pos0: int, q, n_head: int, n_kv_head: int,
                  head_dim: int, page_cells: int = 16, gate=None, n_threads: int = 0):
    """Causal chunk attention: row t (position pos0+t) over cells 0..=pos0+t."""
    k_pool_u16 = _c(k_pool_u16, np.uint16)
    v_pool_u16 = _c(v_pool_u16, np.uint16)
    bt = _c(block_table, np.uint32)
    q = _c(q, np.float32)
    g = _c(gate, np.float32) if gate is not None else None
    chunk = q.size // (n_head * head_dim)
    out = np.empty((chunk, n_head, head_dim), np.float32)
    used = lib().brc_ref_prefill_chunk(_p(k_pool_u16, _u16p), _p(v_pool_u16, _u16p), _p(bt, _u32p), pos0,
                                       chunk, _p(q, _f32p), _p(g, _f32p), n_head, n_kv_head, head_dim,
                                       page_cells, _p(out, _f32p), n_threads)
    assert used > 0
    return out, used


def partial_head(q_head, k, v, cell_begin: int, cell_end: int, kvh: int, n_kv_head: int, head_dim: int,
                 scale: float):
    q_head = _c(q_head, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    m = C.c_double()
    l = C.c_double()
    acc = np.empty(head_dim, np.float64)
    lib().brc_ref_partial_head(_p(q_head, _f32p), _p(k, _f32p), _p(v, _f32p), cell_begin, cell_end, kvh,
                               n_kv_head, head_dim, scale, C.byref(m), C.byref(l), _p(acc, _f64p))
    return m.value, l.value, acc


def lse_combine(m, l, acc) -> np.ndarray:
    m = _c(m, np.float64)
    l = _c(l, np.float64)
    acc = _c(acc, np.float64)
    out = np.empty(acc.shape[-1], np.float64)
    lib().brc_ref_lse_combine(_p(m, _f64p), _p(l, _f64p), _p(acc, _f64p), m.size, acc.shape[-1],
                              _p(out, _f64p))
    return out


def page_copy(k_pool_bytes: np.ndarray, v_pool_bytes: np.ndarray, n_layers: int, n_pages: int,
              half_page_bytes: int, src_ids, dst_ids) -> None:
    src = _c(src_ids, np.uint32)
    dst = _c(dst_ids, np.uint32)
    assert k_pool_bytes.dtype == np.uint8 and v_pool_bytes.dtype == np.uint8
    lib().brc_ref_page_copy(_p(k_pool_bytes, _u8p), _p(v_pool_bytes, _u8p), n_layers, n_pages,
                            half_page_bytes, _p(src, _u32p), _p(dst, _u32p), src.size)
