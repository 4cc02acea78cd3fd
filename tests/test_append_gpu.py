"""KV append on the GPU through the C ABI, bit-exact against the oracle."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200.qsa import KvPool, Qsa, QsaState
from helpers import dev_u32
from test_oracle_cpu import layout_kat_inputs

pytestmark = pytest.mark.gpu


def test_layout_kat_cells_5_to_37_on_gpu(cuda_device):
    """The reference's `qsa_kv_cache_layout_and_f16_precision` through the mirror API: identity-ish
    table from the allocator, 33 single-token appends, every address and bit."""
    pool = KvPool(0, 1, 2, 256, 3)
    qsa = Qsa(pool, 16)
    state = QsaState(pool, 40)
    ws = qsa.workspace(1)
    want_k = np.zeros(3 * 2 * 16 * 256 // 2, np.uint32)
    want_v = np.zeros_like(want_k)
    for cell in range(5, 38):
        k, v = layout_kat_inputs(cell, 512)
        ws.k_cur.copy_(torch.from_numpy(k).view(1, -1))
        ws.v_cur.copy_(torch.from_numpy(v).view(1, -1))
        qsa.kv_append(state, ws, cell)
        assert oracle.kv_append(want_k, want_v, state.page_table, k, v, cell, 2, 256) == 0
    pool.check()
    assert np.array_equal(pool.read(0, 0).reshape(-1), want_k.view(np.uint16))
    assert np.array_equal(pool.read(1, 0).reshape(-1), want_v.view(np.uint16))
    with pytest.raises(_lib.BrcError, match="kv_append would write cells 48..49 but the cache holds 48"):
        qsa.kv_append(state, ws, 48)
    state.release()
    assert pool.free_count() == 3
    pool.release()


def test_f16_store_rule_on_hard_bit_patterns(cuda_device):
    """Bit patterns around every edge of the rule (flush threshold, ties, carries, overflow, NaN)
    plus a random sweep, appended as f32 tokens and compared word for word."""
    edges = []
    for base in (0x38000000, 0x387FE000, 0x38800000, 0x3F5FDBFC, 0x477FE000, 0x47800000, 0x7F800000, 0x7FC00000,
                 0x00000000, 0x00800000, 0x3F800000, 0x45000FFF):
        edges.append(np.arange(base - 2048 if base >= 2048 else 0, base + 2048, dtype=np.uint64))
    bits = np.concatenate(edges + [np.random.default_rng(3).integers(0, 1 << 32, 1 << 18, dtype=np.uint64)])
    bits = np.concatenate([bits, bits | 0x80000000]).astype(np.uint32)
    n_tok = (bits.size + 511) // 512
    bits = np.resize(bits, n_tok * 512)
    src = bits.view(np.float32).reshape(n_tok, 512)
    n_pages = (n_tok + 15) // 16
    pool = KvPool(0, 1, 2, 256, n_pages)
    table = synth.permutation(11, n_pages)
    k_dev = torch.from_numpy(src.copy()).cuda()
    v_dev = torch.from_numpy(src[::-1].copy()).cuda()
    table_dev, pos_dev = dev_u32(table), dev_u32([0])   # named: they must outlive the launch
    _lib.call("brc_kv_append", pool.handle, 0, C.c_void_p(table_dev.data_ptr()), n_pages,
              C.c_void_p(pos_dev.data_ptr()), 1, n_tok, None, n_tok, n_tok, C.c_void_p(k_dev.data_ptr()),
              C.c_void_p(v_dev.data_ptr()), _lib.DTYPE_F32, None)
    pool.check()
    want_k = np.zeros(n_pages * 2 * 16 * 256 // 2, np.uint32)
    want_v = np.zeros_like(want_k)
    assert oracle.kv_append(want_k, want_v, table, src, src[::-1].copy(), 0, 2, 256) == 0
    assert np.array_equal(pool.read(0, 0).reshape(-1), want_k.view(np.uint16))
    assert np.array_equal(pool.read(1, 0).reshape(-1), want_v.view(np.uint16))
    pool.release()


@pytest.mark.parametrize("head_dim,n_kv", [(256, 2), (128, 4)])
def test_batched_ragged_append_matches_oracle(cuda_device, head_dim, n_kv):
    """Several sequences in one call, ragged token counts (one of them zero), scattered tables,
    several layers; f32 and f16 sources."""
    rng = np.random.default_rng(21)
    n_layers = 3
    pos0 = np.array([0, 5, 31, 16, 100], np.uint32)
    counts = np.array([40, 1, 18, 0, 7], np.uint32)
    cu = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    tables, n_pool = synth.scattered_tables(4, pos0 + counts, pool_factor=1.5)
    pool = KvPool(0, n_layers, n_kv, head_dim, n_pool)
    total = int(cu[-1])
    row = n_kv * head_dim
    tables_dev, pos_dev, cu_dev = dev_u32(tables), dev_u32(pos0), dev_u32(cu)
    for layer in (0, 2):
        k = synth.normal(100 + layer, total * row, 0.5).reshape(total, row)
        v = synth.normal(200 + layer, total * row, 0.5).reshape(total, row)
        k_dev, v_dev = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        _lib.call("brc_kv_append", pool.handle, layer, C.c_void_p(tables_dev.data_ptr()), tables.shape[1],
                  C.c_void_p(pos_dev.data_ptr()), pos0.size, 0, C.c_void_p(cu_dev.data_ptr()), total,
                  int((pos0 + counts).max()), C.c_void_p(k_dev.data_ptr()), C.c_void_p(v_dev.data_ptr()),
                  _lib.DTYPE_F32, None)
        torch.cuda.synchronize()
        want_k = np.zeros(n_pool * n_kv * 16 * head_dim // 2, np.uint32)
        want_v = np.zeros_like(want_k)
        for s in range(pos0.size):
            if counts[s]:
                assert oracle.kv_append(want_k, want_v, tables[s], k[cu[s]:cu[s + 1]], v[cu[s]:cu[s + 1]], int(pos0[s]),
                                        n_kv, head_dim) == 0
        assert np.array_equal(pool.read(0, layer).reshape(-1), want_k.view(np.uint16))
        assert np.array_equal(pool.read(1, layer).reshape(-1), want_v.view(np.uint16))
    assert not pool.read(0, 1).any()      # untouched layer stays zero
    # f16 sources: stored as they are, subnormal bit patterns flushed to signed zero
    h = rng.integers(0, 1 << 16, (total, row), dtype=np.uint32).astype(np.uint16)
    hk = torch.from_numpy(h.view(np.int16)).cuda()
    _lib.call("brc_kv_append", pool.handle, 1, C.c_void_p(tables_dev.data_ptr()), tables.shape[1],
              C.c_void_p(pos_dev.data_ptr()), pos0.size, 0, C.c_void_p(cu_dev.data_ptr()), total,
              int((pos0 + counts).max()), C.c_void_p(hk.data_ptr()), C.c_void_p(hk.data_ptr()), _lib.DTYPE_F16, None)
    pool.check()
    flushed = np.where((h & 0x7C00) == 0, h & 0x8000, h).astype(np.uint16)
    got = pool.read(0, 1)
    for s in range(pos0.size):
        for t in range(int(counts[s])):
            cell = int(pos0[s]) + t
            page = tables[s, cell // 16]
            assert np.array_equal(got[page, :, cell % 16, :].reshape(-1), flushed[cu[s] + t])
    pool.release()


def test_append_host_and_device_refusals(cuda_device):
    pool = KvPool(0, 1, 2, 256, 4)
    k = torch.zeros((1, 512), device="cuda")
    table = dev_u32([0, 1, 2, 99])
    pos = dev_u32([63])
    L = _lib.load()
    # host: past the table
    rc = L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 1, None, 1, 65,
                         C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None)
    assert rc == _lib.ERR_CAPACITY and b"cells up to 65" in L.brc_last_error()
    # host: bad layer, bad dtype, inconsistent token count
    assert L.brc_kv_append(pool.handle, 1, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 1, None, 1, 64,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None) == _lib.ERR_INVALID
    assert L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 1, None, 1, 64,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 5, None) == _lib.ERR_INVALID
    assert L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 2, None, 1, 64,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None) == _lib.ERR_INVALID
    # device: the table names page 99 of 4 -> the kernel skips the write and the check reports it
    before = pool.read(0, 0).copy()
    assert L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 1, None, 1, 64,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None) == 0
    with pytest.raises(_lib.BrcError, match="page id >= n_pages"):
        pool.check()
    assert np.array_equal(pool.read(0, 0), before)
    pool.check()  # the word was cleared
    # device: a position beyond the caller's bound is skipped and reported
    assert L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 1, 1, None, 1, 32,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None) == 0
    with pytest.raises(_lib.BrcError, match="position past bound"):
        pool.check()
    # empty call
    assert L.brc_kv_append(pool.handle, 0, C.c_void_p(table.data_ptr()), 4, C.c_void_p(pos.data_ptr()), 0, 1, None, 0, 0,
                           C.c_void_p(k.data_ptr()), C.c_void_p(k.data_ptr()), 0, None) == 0
    pool.release()
