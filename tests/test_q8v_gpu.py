"""q8_0 V page bodies on the GPU: the append's store rule bit for bit against the oracle, and attention over selected
blocks with in-register dequantisation against the oracle's `attend` over the dequantised rows — the shape of the
reference's test (64 cells, block ids [0, 5, 9, 15], gate on; crates/breccia-kernels/tests/attn_conformance.rs:
1354-1452) and a longer ragged one.  Bars as for binary16 V: max-abs <= 2e-3, max-rel <= 1e-2, reference measure <= 1e-5."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from oracle import q8v
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import KvPool
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32

pytestmark = pytest.mark.gpu
P = lambda x: C.c_void_p(x.data_ptr())


def append(pool, layer, table, pos0, k_rows, v_rows):
    t_dev, p_dev = dev_u32(table[None, :]), dev_u32(np.array([pos0]))
    kd, vd = torch.from_numpy(k_rows).cuda(), torch.from_numpy(v_rows).cuda()
    n = k_rows.shape[0]
    _lib.call("brc_kv_append", pool.handle, layer, P(t_dev), table.size, P(p_dev), 1, n, None, n, pos0 + n, P(kd), P(vd),
              DTYPE_F32, None)
    pool.check()


def sparse(pool, layer, q, n_head, table, pos, ids, gate=None):
    hd = pool.head_dim
    qd = torch.from_numpy(q).cuda()
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    t_dev, p_dev = dev_u32(table[None, :]), dev_u32(np.array([pos]))
    i_dev, c_dev = dev_u32(np.asarray(ids, np.uint32)[None, :]), dev_u32(np.array([len(ids)]))
    g_dev = torch.from_numpy(gate).cuda() if gate is not None else None
    _lib.call("brc_paged_sparse_attn", pool.handle, layer, P(qd), DTYPE_F32, n_head,
              C.c_void_p(g_dev.view(-1)[hd:].data_ptr()) if gate is not None else None, 2 * hd if gate is not None else 0,
              P(t_dev), table.size, P(p_dev), 1, 1, P(i_dev), len(ids), P(c_dev), pos + 1, 1.0 / np.sqrt(hd), P(out), None)
    pool.check()
    return out.cpu().numpy()[0]


@pytest.mark.parametrize("n_head,n_kv,hd,cells,ids", [
    (24, 2, 256, 64, [0, 5, 9, 15]),                       # the reference's case
    (16, 2, 256, 1003, list(range(0, 251, 3)) + [250]),    # ragged: the last block holds the row's own cell and 1 future one
    (8, 4, 128, 200, list(range(50))),
])
def test_q8_0_v_append_bit_exact_and_sparse_attention(cuda_device, n_head, n_kv, hd, cells, ids):
    n_pages = (cells + 15) // 16
    pool = KvPool(0, 2, n_kv, hd, n_pages + 5, v_q8=True)
    layout = C.c_int32(-1)
    _lib.call("brc_pool_v_layout", pool.handle, C.byref(layout))
    assert layout.value == 1
    assert pool.bytes() == 2 * (n_pages + 5) * n_kv * 16 * hd * 2 * (1 + 0.5625)
    table = synth.permutation(91, n_pages + 5)[:n_pages].astype(np.uint32)
    dim = n_kv * hd
    k_all = oracle.normalish(0xF1, cells * dim).reshape(cells, dim)
    v_all = oracle.normalish(0xF2, cells * dim).reshape(cells, dim)
    v_all[7, :32] = 0.0                                     # an all-zero block keeps scale 1
    q = oracle.normalish(0xF3, n_head * hd).reshape(1, n_head, hd)
    q_full = oracle.normalish(0xF4, n_head * 2 * hd).reshape(1, n_head, 2, hd)
    first = min(cells, 40)
    append(pool, 1, table, 0, k_all[:first], v_all[:first])      # two calls, the second starting inside a page
    if cells > first:
        append(pool, 1, table, first, k_all[first:], v_all[first:])
    # the pool's V bytes are the oracle's, bit for bit; K stays binary16
    want_pool = np.zeros(((n_pages + 5) * n_kv * 16, q8v.row_bytes(hd)), np.uint8)
    q8v.v_append(want_pool, table, v_all, 0, n_kv, hd)
    assert np.array_equal(pool.read(1, 1), want_pool)
    assert not pool.read(1, 0).any()
    kw = np.zeros((n_pages + 5) * n_kv * 16 * hd // 2, np.uint32)
    assert oracle.kv_append(kw, kw.copy(), table, k_all, v_all, 0, n_kv, hd) == 0
    assert np.array_equal(pool.read(0, 1).reshape(-1), kw.view(np.uint16))
    # attention over the selected blocks
    got = sparse(pool, 1, q, n_head, table, cells - 1, ids, gate=q_full)
    kf = oracle.to_f16(k_all)
    vq = q8v.to_q8_0(v_all.reshape(cells * n_kv, hd)).reshape(cells, dim)
    want = oracle.attend(q[0], kf, vq, oracle.cells_of(ids, 4), cells - 1, n_head, n_kv, hd, gate=q_full[0, :, 1, :])
    max_abs, max_rel, ref = attention_errors(got, want)
    print(f"q8_0 V {n_head}q/{n_kv}kv hd{hd} {cells} cells: max_abs {max_abs:.2e} max_rel {max_rel:.2e} ref {ref:.2e}")
    assert np.isfinite(got).all()
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5
    # and it differs from the binary16 answer by no more than the storage loss allows
    want_f16 = oracle.attend(q[0], kf, oracle.to_f16(v_all), oracle.cells_of(ids, 4), cells - 1, n_head, n_kv, hd,
                             gate=q_full[0, :, 1, :])
    assert np.abs(got - want_f16).max() <= 0.05
    pool.release()


def test_q8_0_v_sparse_rows_of_two_sequences(cuda_device):
    """Three rows each of two sequences over a q8_0 V pool (rows_per_seq = 3, binary16 query): row t sees cells up to
    pos0 + t only; a list of 401 blocks (several CTAs per cluster, tiles interleaved between them, the last block partly
    in the future) beside short lists and a row with an empty list, which yields zeros."""
    n_head, n_kv, hd = 16, 2, 256
    lens, pages = [2064, 80], [129, 5]
    pool = KvPool(0, 1, n_kv, hd, 140, v_q8=True)
    perm = synth.permutation(93, 140).astype(np.uint32)
    tables = np.zeros((2, 129), np.uint32)
    tables[0], tables[1, :5] = perm[:129], perm[129:134]
    dim = n_kv * hd
    ks, vs = [], []
    for s in range(2):
        ks.append(oracle.normalish(0x101 + s, lens[s] * dim).reshape(lens[s], dim))
        vs.append(oracle.normalish(0x111 + s, lens[s] * dim).reshape(lens[s], dim))
        append(pool, 0, tables[s, :pages[s]].copy(), 0, ks[s], vs[s])
    pos0s = np.array([2059, 70])
    ids = np.zeros((6, 513), np.uint32)
    counts = np.zeros(6, np.uint32)
    for r in range(3):
        ids[r, :400] = np.sort(synth.permutation(94 + r, 514)[:400])
        ids[r, 400] = (2059 + r) // 4
        counts[r] = 401
        ids[3 + r, :5] = [0, 5, 9, 15, 17]                      # block 17 = cells 68 .. 71: partly in the future
        counts[3 + r] = 5
    counts[4] = 0
    q = oracle.to_f16(synth.normal(95, 6 * n_head * hd)).reshape(6, n_head, hd)
    qd = torch.from_numpy(q).cuda().half()
    out = torch.full((6, n_head, hd), float("nan"), device="cuda")
    t_dev, p_dev, i_dev, c_dev = dev_u32(tables), dev_u32(pos0s), dev_u32(ids), dev_u32(counts)
    _lib.call("brc_paged_sparse_attn", pool.handle, 0, P(qd), DTYPE_F16, n_head, None, 0, P(t_dev), tables.shape[1], P(p_dev), 2, 3,
              P(i_dev), ids.shape[1], P(c_dev), int(pos0s.max()) + 3, 1.0 / np.sqrt(hd), P(out), None)
    pool.check()
    got = out.cpu().numpy()
    for r in range(6):
        s, t = divmod(r, 3)
        if counts[r] == 0:
            assert not got[r].any()
            continue
        kf = oracle.to_f16(ks[s])
        vq = q8v.to_q8_0(vs[s].reshape(lens[s] * n_kv, hd)).reshape(lens[s], dim)
        want = oracle.attend(q[r], kf, vq, oracle.cells_of(ids[r, :counts[r]], 4), int(pos0s[s]) + t, n_head, n_kv, hd)
        max_abs, max_rel, ref = attention_errors(got[r], want)
        assert np.isfinite(got[r]).all()
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5, f"row {r}: {max_abs:.2e} {max_rel:.2e} {ref:.2e}"
    pool.release()


def test_binary16_sources_are_refused_on_a_q8_0_pool(cuda_device):
    pool = KvPool(0, 1, 2, 256, 8, v_q8=True)
    x = torch.zeros(4096, device="cuda")
    t = dev_u32(np.zeros((1, 2)))
    with pytest.raises(_lib.BrcError) as err:      # binary16 sources are refused: the rule quantises from f32
        _lib.call("brc_kv_append", pool.handle, 0, P(t), 2, P(t), 1, 1, None, 1, 1, P(x), P(x), _lib.DTYPE_F16, None)
    assert err.value.code == _lib.ERR_UNSUPPORTED
    assert pool.alloc(3).size == 3                  # the allocator works as on any pool
    pool.release()


def test_fork_copies_the_partial_last_page_of_a_q8_0_pool_as_it_is(cuda_device):
    """Copy-on-write fork on a q8_0 V pool: full pages shared, the partial last page copied in every layer, K as
    binary16 and V as its q8_0 bytes; the parent's pages and all other pages stay as they were."""
    n_kv, hd, n_layers, cells = 2, 256, 3, 21
    pool = KvPool(0, n_layers, n_kv, hd, 8, v_q8=True)
    parent = pool.alloc(2)
    for layer in range(n_layers):
        k_rows = oracle.normalish(0x51 + layer, cells * n_kv * hd).reshape(cells, n_kv * hd)
        v_rows = oracle.normalish(0x61 + layer, cells * n_kv * hd).reshape(cells, n_kv * hd)
        append(pool, layer, parent, 0, k_rows, v_rows)
    before = [(pool.read(0, layer), pool.read(1, layer)) for layer in range(n_layers)]
    child, fresh = pool.fork(parent, cells)
    torch.cuda.synchronize()
    pool.check()
    assert child[0] == parent[0] and fresh is not None and child[1] == fresh and fresh not in parent.tolist()
    rows = n_kv * 16
    for layer in range(n_layers):
        k_now, v_now = pool.read(0, layer), pool.read(1, layer)
        assert np.array_equal(k_now[fresh], before[layer][0][parent[1]])
        assert np.array_equal(v_now[fresh * rows:(fresh + 1) * rows], before[layer][1][parent[1] * rows:(parent[1] + 1) * rows])
        assert v_now[fresh * rows:(fresh + 1) * rows].any()
        keep = [p for p in range(8) if p != fresh]
        assert np.array_equal(k_now[keep], before[layer][0][keep])
        v_pages_now, v_pages_before = v_now.reshape(8, -1), before[layer][1].reshape(8, -1)
        assert np.array_equal(v_pages_now[keep], v_pages_before[keep])
    pool.release()


def test_gather_on_a_q8_0_pool_returns_k_rows_and_the_stored_v_rows(cuda_device):
    """brc_page_gather through a scattered block table: K as binary16 rows, V as the 36-byte blocks the append
    stored, in logical cell order."""
    from oracle import q8v

    n_kv, hd, cells = 2, 256, 37
    pool = KvPool(0, 1, n_kv, hd, 16, v_q8=True)
    table = np.array([9, 2, 14], np.uint32)
    pool.alloc(16)
    k = synth.normal(71, cells * n_kv * hd, 0.5).reshape(cells, n_kv * hd)
    v = synth.normal(72, cells * n_kv * hd, 0.5).reshape(cells, n_kv * hd)
    t_dev, pos0, k_dev, v_dev = dev_u32(table[None, :]), dev_u32([0]), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()   # kept alive
    _lib.call("brc_kv_append", pool.handle, 0, P(t_dev), 3, P(pos0), 1, cells, None, cells, cells, P(k_dev), P(v_dev), DTYPE_F32, None)
    k_out = torch.zeros((cells, n_kv, hd), dtype=torch.float16, device="cuda")
    v_out = torch.zeros((cells, n_kv, q8v.row_bytes(hd)), dtype=torch.uint8, device="cuda")
    _lib.call("brc_page_gather", pool.handle, 0, P(t_dev), 3, cells, P(k_out), P(v_out), None)
    pool.check()
    assert np.array_equal(k_out.view(torch.int16).cpu().numpy().view(np.uint16).reshape(cells, -1), oracle.f32_to_f16_bits_np(k.reshape(-1)).reshape(cells, -1))
    want_v = q8v.pack_rows(v.reshape(cells * n_kv, hd)).reshape(cells, n_kv, -1)
    assert np.array_equal(v_out.cpu().numpy(), want_v)
    pool.release()


@pytest.mark.parametrize("n_head,pos0,chunk", [(16, 100, 40), (24, 0, 21), (16, 1000, 130)])
def test_chunked_prefill_over_a_q8_0_v_pool(cuda_device, n_head, pos0, chunk):
    """The tensor-core prefill path on a q8_0 V pool: the loaders dequantise the blocks into the binary16 V tile
    (scale x quantum, rounded to binary16).  Oracle: f64 attention over K as binary16 and V as the q8_0 round
    trip (cpu::to_q8_0).  The binary16 rounding of the dequantised V adds up to 2^-11 |v| (about 4e-4 here) in
    absolute terms whatever the output's size, so the 2e-3 absolute bar holds everywhere and the 1 % relative bar
    is applied where |want| > 0.05 (0.02 on binary16 pools, whose V needs no rounding)."""
    n_kv, hd = 2, 256
    cells = pos0 + chunk
    dim = n_kv * hd
    n_pages = (cells + 15) // 16
    pool = KvPool(0, 1, n_kv, hd, n_pages + 5, v_q8=True)
    table = synth.permutation(41 + chunk, n_pages + 5)[:n_pages].astype(np.uint32)
    pool.alloc(n_pages + 5)
    k_all = synth.normal(42 + chunk, cells * dim, 0.5).reshape(cells, dim)
    v_all = synth.normal(43 + chunk, cells * dim, 0.5).reshape(cells, dim)
    t_dev, zero, k_dev, v_dev = dev_u32(table[None, :]), dev_u32([0]), torch.from_numpy(k_all).cuda(), torch.from_numpy(v_all).cuda()
    _lib.call("brc_kv_append", pool.handle, 0, P(t_dev), n_pages, P(zero), 1, cells, None, cells, cells, P(k_dev), P(v_dev), DTYPE_F32, None)
    q = oracle.to_f16(synth.normal(44 + chunk, chunk * n_head * hd)).reshape(1, chunk, n_head, hd)
    qd = torch.from_numpy(q).cuda().half()
    out = torch.full((1, chunk, n_head, hd), float("nan"), device="cuda")
    p_dev = dev_u32([pos0])
    _lib.call("brc_paged_prefill_attn", pool.handle, 0, P(qd), _lib.DTYPE_F16, n_head, None, 0, P(t_dev), n_pages, P(p_dev), 1, chunk,
              cells, 1.0 / np.sqrt(hd), P(out), None)
    pool.check()
    got = out.cpu().numpy()[0]
    kf, vq = oracle.to_f16(k_all), q8v.to_q8_0(v_all.reshape(cells * n_kv, hd)).reshape(cells, dim)
    worst = 0.0
    for t in range(chunk):
        want = oracle.attend(q[0, t], kf, vq, np.arange(cells, dtype=np.uint32), pos0 + t, n_head, n_kv, hd)
        diff = np.abs(got[t].astype(np.float64) - want)
        big = np.abs(want) > 0.05
        max_abs, max_rel = float(diff.max()), float((diff[big] / np.abs(want[big])).max()) if big.any() else 0.0
        worst = max(worst, max_abs)
        assert np.isfinite(got[t]).all() and max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL, f"row {t}: max_abs {max_abs:.2e} max_rel {max_rel:.2e}"
    print(f"prefill over q8_0 V, {n_head} heads, pos0 {pos0}, chunk {chunk}: worst max_abs {worst:.2e}")
    pool.release()
