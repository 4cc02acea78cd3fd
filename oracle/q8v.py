"""q8_0 V page bodies on the CPU — TEST INFRASTRUCTURE, never the product.

The reference's only shipped KV compression stores V rows as blocks of 32 values: one f32 scale and 32 signed
bytes, 36 B for 32 elements against 64 B for binary16 (crates/breccia-kernels/src/qsa/mod.rs:325-349).  Store rule:
crates/breccia-kernels/shaders/qsa_kv_append.comp:117-133 (scale = amax / 127, or 1 for an all-zero block; q =
round-half-away(clamp(x / scale, -127, 127)), from the f32 value, never through binary16; word 0 of a block is the
scale, words 1..8 hold four quanta each, lowest byte first).  Read rule: qsa_attn_apply.comp:69-77 (float(q) * scale).
The CPU statement is cpu::to_q8_0 (crates/breccia-kernels/src/qsa/cpu.rs:65-82).

Pinned by the reference's own tests of that function, restated in tests/test_q8v_cpu.py: exact zeros, error within
half a step of the block's scale, the block maximum on the grid (qsa/mod.rs:2072-2107), and the 36-byte / 0.5625x
size pins (qsa/mod.rs:1983, 2046)."""
from __future__ import annotations

import numpy as np

BLOCK_ELEMS = 32
BLOCK_BYTES = 36


def quantize(x) -> tuple[np.ndarray, np.ndarray]:
    """x [..., n] f32, n a multiple of 32 -> (scales [..., n/32] f32, quanta [..., n/32, 32] int8)."""
    x = np.ascontiguousarray(x, np.float32)
    if x.shape[-1] % BLOCK_ELEMS:
        raise ValueError(f"a q8_0 row is a whole number of {BLOCK_ELEMS}-element blocks")
    b = x.reshape(x.shape[:-1] + (x.shape[-1] // BLOCK_ELEMS, BLOCK_ELEMS))
    amax = np.abs(b).max(axis=-1)
    scale = np.where(amax > 0, amax / np.float32(127.0), np.float32(1.0)).astype(np.float32)
    r = np.clip(b / scale[..., None], np.float32(-127.0), np.float32(127.0)).astype(np.float32)
    # round half away from zero; the half is added in f64 so that it is exact
    q = np.sign(r) * np.floor(np.abs(r).astype(np.float64) + 0.5)
    return scale, q.astype(np.int8)


def dequantize(scale, q) -> np.ndarray:
    out = q.astype(np.float32) * np.asarray(scale, np.float32)[..., None]
    return out.reshape(out.shape[:-2] + (out.shape[-2] * BLOCK_ELEMS,))


def to_q8_0(x) -> np.ndarray:
    """What a q8_0 store followed by a load returns (cpu::to_q8_0)."""
    return dequantize(*quantize(x))


def pack_rows(x) -> np.ndarray:
    """x [rows, n] f32 -> the pool bytes of those rows, [rows, n/32 * 36] uint8."""
    scale, q = quantize(x)
    rows, nb = scale.shape
    out = np.empty((rows, nb, BLOCK_BYTES), np.uint8)
    out[:, :, :4] = scale.astype("<f4").view(np.uint8).reshape(rows, nb, 4)
    out[:, :, 4:] = q.view(np.uint8)
    return out.reshape(rows, nb * BLOCK_BYTES)


def unpack_rows(raw) -> np.ndarray:
    """The inverse of pack_rows: [rows, nb * 36] uint8 -> [rows, nb * 32] f32."""
    raw = np.ascontiguousarray(raw, np.uint8)
    rows = raw.shape[0]
    blocks = raw.reshape(rows, -1, BLOCK_BYTES)
    scale = np.ascontiguousarray(blocks[:, :, :4]).view("<f4").reshape(rows, -1)
    q = np.ascontiguousarray(blocks[:, :, 4:]).view(np.int8)
    return dequantize(scale, q)


def row_bytes(head_dim: int) -> int:
    return head_dim // BLOCK_ELEMS * BLOCK_BYTES


def v_append(v8_pool: np.ndarray, page_table, v_cur, pos0: int, n_kv_head: int, head_dim: int, page_cells: int = 16) -> None:
    """Store rows v_cur [T, n_kv_head * head_dim] f32 at cells pos0.. of the sequence `page_table` names.
    v8_pool: [n_pages * n_kv_head * page_cells, row_bytes] uint8, row (page * n_kv_head + kvh) * page_cells + cell
    (qsa_kv_append.comp:100-104)."""
    v_cur = np.asarray(v_cur, np.float32).reshape(-1, n_kv_head, head_dim)
    for t in range(v_cur.shape[0]):
        cell = pos0 + t
        page = int(page_table[cell // page_cells])
        for kvh in range(n_kv_head):
            row = (page * n_kv_head + kvh) * page_cells + cell % page_cells
            v8_pool[row] = pack_rows(v_cur[t, kvh][None, :])[0]


def gather_v(v8_pool: np.ndarray, page_table, n_cells: int, n_kv_head: int, head_dim: int, page_cells: int = 16) -> np.ndarray:
    """The dequantised V rows of cells 0..n_cells of a sequence, [n_cells, n_kv_head * head_dim] f32."""
    out = np.empty((n_cells, n_kv_head, head_dim), np.float32)
    for cell in range(n_cells):
        page = int(page_table[cell // page_cells])
        for kvh in range(n_kv_head):
            row = (page * n_kv_head + kvh) * page_cells + cell % page_cells
            out[cell, kvh] = unpack_rows(v8_pool[row][None, :])[0]
    return out.reshape(n_cells, n_kv_head * head_dim)
