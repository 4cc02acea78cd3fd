"""Attention over selected 4-cell blocks (brc_paged_sparse_attn) against the oracle's `attend` over `cells_of`
(the reference's own CPU statement, crates/breccia-kernels/src/qsa/cpu.rs:197-257), with the shapes of the
reference's tests: the 2062-cell single-query case over a block list, and its 64-cell case with the id list
[0, 5, 9, 15] (crates/breccia-kernels/tests/attn_conformance.rs:897-1037, 1354-1439).

Bars: max-abs <= 2e-3, max-rel <= 1e-2 (target), and the reference's measure max|g-w|/max(|w|,1) <= 1e-5."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import KvPool
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32, fill_pool_from_host

pytestmark = pytest.mark.gpu
P = lambda x: C.c_void_p(x.data_ptr())


def run_sparse(pool, layer, q, n_head, tables, pos0s, rows_per_seq, ids, counts, q_dtype=DTYPE_F32, gate=None):
    rows = ids.shape[0]
    hd = pool.head_dim
    qd = torch.from_numpy(q).cuda()
    if q_dtype == DTYPE_F16:
        qd = qd.half()
    out = torch.full((rows, n_head, hd), float("nan"), device="cuda")
    t_dev, p_dev, i_dev, c_dev = dev_u32(tables), dev_u32(pos0s), dev_u32(ids), dev_u32(counts)
    g_dev = torch.from_numpy(gate).cuda() if gate is not None else None
    _lib.call("brc_paged_sparse_attn", pool.handle, layer, P(qd), q_dtype, n_head,
              C.c_void_p(g_dev.view(-1)[hd:].data_ptr()) if gate is not None else None, 2 * hd if gate is not None else 0,
              P(t_dev), tables.shape[1], P(p_dev), len(pos0s), rows_per_seq, P(i_dev), ids.shape[1], P(c_dev),
              int(max(pos0s) + rows_per_seq), 1.0 / np.sqrt(hd), P(out), None)
    pool.check()
    return out.cpu().numpy()


def want_row(k, v, table, pos, q_row, blocks, n_head, n_kv, hd, gate=None):
    n_cells = table.size * 16
    _, kf = oracle.gather(k, table, n_cells, n_kv, hd)
    _, vf = oracle.gather(v, table, n_cells, n_kv, hd)
    cells = oracle.cells_of(blocks, 4)
    return oracle.attend(q_row, kf, vf, cells, pos, n_head, n_kv, hd, gate=gate)


def check(got, want, what):
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    max_abs, max_rel, ref = attention_errors(got, want)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5, f"{what}: {max_abs:.2e} {max_rel:.2e} {ref:.2e}"


@pytest.mark.parametrize("n_head,n_kv,hd", [(24, 2, 256), (16, 2, 256), (8, 4, 128)])
def test_block_list_decode_row(cuda_device, n_head, n_kv, hd):
    """One query at position 2061 over 513 selected blocks scattered through the context (the last one its own,
    partly in the future), gate on, f32 query; the reference's head count 24 / 2 included."""
    pos, n_blocks_ctx = 2061, 2064 // 4
    n_pages = 2064 // 16
    pool = KvPool(0, 2, n_kv, hd, n_pages + 6)
    k, v = fill_pool_from_host(pool, 1, 300 + n_head)
    table = synth.permutation(31, n_pages + 6)[:n_pages].astype(np.uint32)
    picks = np.sort(synth.permutation(32, n_blocks_ctx - 1)[:400]).astype(np.uint32)
    ids = np.zeros((1, 513), np.uint32)
    ids[0, :400] = picks
    ids[0, 400] = pos // 4                                    # the row's own block (515, not among the picks): cells 2060, 2061 live, 2062.. masked
    ids[0, 401:] = 7                                          # beyond `counts`: never read
    counts = np.array([401], np.uint32)
    q = synth.normal(33, n_head * hd).reshape(1, n_head, hd).astype(np.float32)
    gate = synth.normal(34, n_head * 2 * hd).reshape(1, n_head, 2, hd).astype(np.float32)
    got = run_sparse(pool, 1, q, n_head, table[None, :], np.array([pos]), 1, ids, counts, gate=gate)
    want = want_row(k, v, table, pos, q[0], ids[0, :401], n_head, n_kv, hd, gate=gate[0, :, 1, :])
    check(got[0], want, f"{n_head}q/{n_kv}kv hd{hd}")
    pool.release()


def test_reference_id_list_shape_and_causal_rows(cuda_device):
    """ids [0, 5, 9, 15] over a 64-cell cache, three rows of two sequences (rows_per_seq = 3): row t sees cells up
    to pos0 + t only; f16 query; a row with an empty list yields zeros."""
    n_head, n_kv, hd = 16, 2, 256
    pool = KvPool(0, 1, n_kv, hd, 12)
    k, v = fill_pool_from_host(pool, 0, 310)
    tables = synth.permutation(35, 12)[:8].astype(np.uint32).reshape(2, 4)
    pos0s = np.array([37, 61])
    ids = np.zeros((6, 8), np.uint32)
    counts = np.zeros(6, np.uint32)
    for r in range(6):
        ids[r, :4] = [0, 5, 9, 15]
        counts[r] = 4
    counts[4] = 0                                               # second sequence, middle row: nothing selected
    q = oracle.to_f16(synth.normal(36, 6 * n_head * hd)).reshape(6, n_head, hd)
    got = run_sparse(pool, 0, q, n_head, tables, pos0s, 3, ids, counts, q_dtype=DTYPE_F16)
    for r in range(6):
        s, t = divmod(r, 3)
        if counts[r] == 0:
            assert not got[r].any()
            continue
        want = want_row(k, v, tables[s], int(pos0s[s]) + t, q[r], ids[r, :4], n_head, n_kv, hd)
        check(got[r], want, f"row {r}")
    pool.release()


def test_sparse_refusals(cuda_device):
    L = _lib.load()
    pool = KvPool(0, 1, 2, 256, 8)
    z = torch.zeros(24 * 256, device="cuda")
    t, p0, ids, cnt = dev_u32([[0, 1, 2, 3]]), dev_u32([10]), dev_u32([[0, 1]]), dev_u32([2])
    args = lambda **kw: [pool.handle, kw.get("layer", 0), P(z), kw.get("dt", 0), kw.get("nh", 24), None, 0, P(t), 4, P(p0), 1, 1, P(ids), 2,
                         P(cnt), kw.get("end", 11), 0.0625, P(z), None]
    assert L.brc_paged_sparse_attn(*args(end=65)) == _lib.ERR_CAPACITY
    assert L.brc_paged_sparse_attn(*args(layer=1)) == _lib.ERR_INVALID
    assert L.brc_paged_sparse_attn(*args(nh=5)) == _lib.ERR_INVALID
    assert L.brc_paged_sparse_attn(*args(dt=3)) == _lib.ERR_INVALID
    assert L.brc_paged_sparse_attn(*args()) == 0
    pool.check()
    pool.release()
