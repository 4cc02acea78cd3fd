"""Chunked-prefill attention (tcgen05 path) through the C ABI against the oracle.

Tolerance (target): max-abs <= 2e-3, max-rel <= 1e-2 (fp32 accumulate over f16 K/V; the
probabilities enter the tensor cores as binary16)."""
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


def run_prefill(pool, layer, q, n_head, tables, pos0, chunk, q_dtype=DTYPE_F16, gate=None):
    n_seqs = len(pos0)
    hd = pool.head_dim
    qd = torch.from_numpy(q).cuda()
    if q_dtype == DTYPE_F16:
        qd = qd.half()
    out = torch.full((n_seqs, chunk, n_head, hd), float("nan"), device="cuda")
    t_dev, p_dev = dev_u32(tables), dev_u32(pos0)
    g_dev = torch.from_numpy(gate).cuda() if gate is not None else None
    _lib.call("brc_paged_prefill_attn", pool.handle, layer, C.c_void_p(qd.data_ptr()), q_dtype, n_head,
              C.c_void_p(g_dev.view(-1)[hd:].data_ptr()) if gate is not None else None, 2 * hd if gate is not None else 0,
              C.c_void_p(t_dev.data_ptr()), tables.shape[1], C.c_void_p(p_dev.data_ptr()), n_seqs, chunk,
              int(max(pos0) + chunk), 1.0 / np.sqrt(hd), C.c_void_p(out.data_ptr()), None)
    pool.check()
    return out.cpu().numpy()


def check(got, want, what):
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    max_abs, max_rel, ref = attention_errors(got, want)
    print(f"{what}: max_abs {max_abs:.2e} max_rel {max_rel:.2e} ref_measure {ref:.2e}")
    assert max_abs <= ATTN_MAX_ABS, f"{what}: max-abs {max_abs:.3e}"
    assert max_rel <= ATTN_MAX_REL, f"{what}: max-rel {max_rel:.3e}"


@pytest.mark.parametrize("n_head,n_kv,pos0s,chunk", [
    (16, 2, [0], 16),                 # one tile, nothing before it
    (16, 2, [64, 0, 37], 40),         # ragged starts, chunk not a multiple of the tile
    (16, 2, [1000], 256),             # a config-4 sized chunk after a long prefix
    (8, 2, [130, 5], 33),             # 4 query heads per kv head (half-empty tiles)
    (8, 1, [20], 17),
    # fewer rows than one 16-token tile: the reference's small path below 16 rows, causal per row
    # (speculative verify, shaders/qsa_attn_scores_small.comp:74-77)
    (16, 2, [100, 0], 2),
    (16, 2, [37], 3),
    (8, 2, [64, 1000], 15),
    # the reference model's own geometry: 12 query heads per kv head (shaders/qsa_attn_scores_gqa.comp:51-133), tiles of
    # 10 tokens x 12 heads; and 16 per kv head (8 tokens x 16)
    (24, 2, [70, 0], 40),
    (24, 2, [2048], 64),
    (16, 1, [33], 20),
])
def test_prefill_matches_oracle(cuda_device, n_head, n_kv, pos0s, chunk):
    hd = 256
    pos0s = np.asarray(pos0s)
    tables, n_pool = synth.scattered_tables(11 + chunk, pos0s + chunk, pool_factor=1.3)
    pool = KvPool(0, 2, n_kv, hd, n_pool)
    k, v = fill_pool_from_host(pool, 1, 1200 + chunk)
    q = oracle.to_f16(synth.normal(1300 + chunk, pos0s.size * chunk * n_head * hd)).reshape(pos0s.size, chunk, n_head, hd)
    got = run_prefill(pool, 1, q, n_head, tables, pos0s, chunk)
    for s in range(pos0s.size):
        want, _ = oracle.prefill_chunk(k, v, tables[s], int(pos0s[s]), q[s], n_head, n_kv, hd)
        check(got[s], want, f"{n_head}q/{n_kv}kv pos0 {pos0s[s]} chunk {chunk}")
    pool.release()


def test_prefill_shared_prefix_gate_f32_query_and_poisoned_tail(cuda_device):
    """Config-4 shape in small: sequences share the pages of a common prefix (the same physical pages in
    every block table), each with its own suffix pages; f32 query, gate; cells past the end of the cache
    and unowned pages hold NaN."""
    n_head, n_kv, hd, prefix, chunk, n_seqs = 16, 2, 256, 200, 48, 3
    n_prefix_pages = prefix // 16                     # 12 full shared pages; cells 192..199 are per sequence
    per_seq = (prefix + chunk + 15) // 16 - n_prefix_pages
    n_pool = n_prefix_pages + n_seqs * per_seq + 5
    perm = synth.permutation(77, n_pool)
    tables = np.zeros((n_seqs, n_prefix_pages + per_seq), np.uint32)
    tables[:, :n_prefix_pages] = perm[:n_prefix_pages]
    for s in range(n_seqs):
        tables[s, n_prefix_pages:] = perm[n_prefix_pages + s * per_seq: n_prefix_pages + (s + 1) * per_seq]
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    k, v = fill_pool_from_host(pool, 0, 1400)
    k = k.reshape(n_pool, n_kv, 16, hd).copy()
    v = v.reshape(n_pool, n_kv, 16, hd).copy()
    live = np.zeros((n_pool, 16), bool)
    for s in range(n_seqs):
        for c in range(prefix + chunk):
            live[tables[s, c // 16], c % 16] = True
    dead = np.broadcast_to(~live[:, None, :, None], k.shape)
    k[dead] = 0xFFFF
    v[dead] = 0xFFFF
    pool.write(0, 0, k)
    pool.write(1, 0, v)
    q = synth.normal(1500, n_seqs * chunk * n_head * hd).reshape(n_seqs, chunk, n_head, hd)
    gate = synth.normal(1501, n_seqs * chunk * n_head * 2 * hd).reshape(n_seqs, chunk, n_head, 2, hd)
    got = run_prefill(pool, 0, q, n_head, tables, np.full(n_seqs, prefix), chunk, q_dtype=DTYPE_F32, gate=gate)
    q16 = oracle.to_f16(q)   # the tensor-core path rounds the query to binary16
    for s in range(n_seqs):
        want, _ = oracle.prefill_chunk(k.reshape(-1), v.reshape(-1), tables[s], prefix, q16[s], n_head, n_kv, hd,
                                       gate=gate[s, :, :, 1, :])
        check(got[s], want, f"shared prefix, sequence {s}")
    pool.release()


def test_prefill_refusals(cuda_device):
    L = _lib.load()
    pool = KvPool(0, 1, 2, 256, 8)
    q = torch.zeros((1, 16, 16, 256), dtype=torch.half, device="cuda")
    out = torch.zeros((1, 16, 16, 256), device="cuda")
    t, p0 = dev_u32([[0, 1, 2, 3]]), dev_u32([0])
    args = lambda **kw: [pool.handle, kw.get("layer", 0), C.c_void_p(q.data_ptr()), kw.get("dt", 1), kw.get("nh", 16), None, 0,
                         C.c_void_p(t.data_ptr()), 4, C.c_void_p(p0.data_ptr()), 1, 16, kw.get("end", 16), 0.0625,
                         C.c_void_p(out.data_ptr()), None]
    assert L.brc_paged_prefill_attn(*args(end=65)) == _lib.ERR_CAPACITY
    assert L.brc_paged_prefill_attn(*args(layer=2)) == _lib.ERR_INVALID
    assert L.brc_paged_prefill_attn(*args(nh=80)) == _lib.ERR_UNSUPPORTED     # 40 query heads per kv head: a tile holds up to 32
    assert L.brc_paged_prefill_attn(*args(dt=7)) == _lib.ERR_INVALID
    p128 = KvPool(0, 1, 2, 128, 8)
    a = args()
    a[0] = p128.handle
    assert L.brc_paged_prefill_attn(*a) == _lib.ERR_UNSUPPORTED and b"head_dim 128" in L.brc_last_error()
    # a position beyond the caller's bound is caught on the device and the tile is skipped
    p0.fill_(40)
    assert L.brc_paged_prefill_attn(*args(end=16)) == 0
    with pytest.raises(_lib.BrcError, match="position past bound"):
        pool.check()
    p128.release()
    pool.release()
