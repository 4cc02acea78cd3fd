"""The radix-prefix + chunked-prefill workload as ONE pipeline on the GPU, through the C ABI:

    owner appends a 4088-token prefix (255 full pages + a last page holding 8 cells)
    brc_radix_insert of the prefix          -> the tree adopts the 255 full pages
    per sequence (64 of them):
        brc_radix_match                     -> the 255 shared pages, one more reference each
        brc_seq_fork of the owner's partial last page   -> a private copy (copy-on-write)
        brc_pages_alloc of the chunk's further pages
    brc_kv_append of every sequence's 256-token chunk at cell 4088 (the first 8 cells land in the fork)
    brc_paged_prefill_attn over prefix + chunk, causal

Checked: the whole pool bit for bit against the oracle's append + page copy on a host mirror (so the
owner's partial page is untouched by 64 forks and appends), refcounts 64 + 1 on the shared pages,
attention of three sequences against the oracle, and that releasing the sequences and evicting the
tree returns the pool to its start.  The reference has no code for this row (docs/BRIEF.md:287): the
semantics are those of its design note, the arithmetic that of its append and attention.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import KvPool
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32

pytestmark = pytest.mark.gpu
U32P = C.POINTER(C.c_uint32)


def _arr(a):
    a = np.ascontiguousarray(a, np.uint32)
    return a, a.ctypes.data_as(U32P)


def test_radix_match_fork_append_prefill_as_one_pipeline(cuda_device):
    n_head, n_kv, hd, prefix, chunk, n_seqs = 16, 2, 256, 4088, 256, 64
    full_pages = prefix // 16                      # 255
    chunk_pages = (prefix + chunk + 15) // 16 - full_pages - 1   # pages after the forked one: 16
    stride = full_pages + 1 + chunk_pages
    n_pool = full_pages + 1 + n_seqs * (1 + chunk_pages) + 16
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    pool.zero()
    free_at_start = pool.free_count()
    words = n_pool * n_kv * 16 * hd // 2
    kw, vw = np.zeros(words, np.uint32), np.zeros(words, np.uint32)      # host mirror of the one layer

    # ---- the owner: 256 pages, 4088 cells through the append kernel
    owner = pool.alloc(full_pages + 1)
    k_pre = synth.normal(2001, prefix * n_kv * hd, 0.5).reshape(prefix, n_kv * hd)
    v_pre = synth.normal(2002, prefix * n_kv * hd, 0.5).reshape(prefix, n_kv * hd)
    owner_dev, zero = dev_u32(owner), dev_u32([0])
    kd, vd = torch.from_numpy(k_pre).cuda(), torch.from_numpy(v_pre).cuda()
    _lib.call("brc_kv_append", pool.handle, 0, C.c_void_p(owner_dev.data_ptr()), owner.size, C.c_void_p(zero.data_ptr()), 1, prefix,
              None, prefix, prefix, C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), DTYPE_F32, None)
    assert oracle.kv_append(kw, vw, owner, k_pre, v_pre, 0, n_kv, hd) == 0

    # ---- the tree adopts the full pages; the owner keeps only its partial last page
    L = _lib.load()
    radix = C.c_void_p()
    _lib.call("brc_radix_create", pool.handle, C.byref(radix))
    tokens = (np.arange(prefix, dtype=np.uint32) * 7 + 3)
    _, tp = _arr(tokens)
    _, op = _arr(owner)
    new = C.c_uint32()
    _lib.call("brc_radix_insert", radix, tp, prefix, op, full_pages + 1, C.byref(new))
    assert new.value == full_pages
    pool.release_pages(owner[:full_pages])

    # ---- 64 sequences: match, fork the partial page, allocate the rest
    tables = np.zeros((n_seqs, stride), np.uint32)
    got, gp = _arr(np.zeros(300))
    n = C.c_uint32()
    forks = []
    for s in range(n_seqs):
        seq_tokens, sp = _arr(np.concatenate([tokens, np.arange(chunk, dtype=np.uint32) + 100000 * (s + 1)]))
        _lib.call("brc_radix_match", radix, sp, seq_tokens.size, gp, 300, C.byref(n))
        assert n.value == full_pages and np.array_equal(got[:full_pages], owner[:full_pages])
        tables[s, :full_pages] = got[:full_pages]
        child, fresh = pool.fork(owner[full_pages:], prefix - full_pages * 16)     # 8 cells: no full page, one copy
        assert fresh is not None and child.size == 1 and child[0] == fresh and fresh != owner[full_pages]
        tables[s, full_pages] = fresh
        forks.append(fresh)
        tables[s, full_pages + 1:] = pool.alloc(chunk_pages)
    half = pool.half_page_bytes
    kb, vb = kw.view(np.uint8), vw.view(np.uint8)
    oracle.page_copy(kb, vb, 1, n_pool, half, np.full(n_seqs, owner[full_pages], np.uint32), np.asarray(forks, np.uint32))
    for page in owner[:full_pages]:
        assert pool.refcount(int(page)) == n_seqs + 1          # 64 sequences + the tree
    assert pool.refcount(int(owner[full_pages])) == 1 and all(pool.refcount(int(f)) == 1 for f in forks)

    # ---- every sequence's chunk at cell 4088: the first 8 cells land in its fork, never in the owner's page
    k_ch = synth.normal(2003, n_seqs * chunk * n_kv * hd, 0.5).reshape(n_seqs, chunk, n_kv * hd)
    v_ch = synth.normal(2004, n_seqs * chunk * n_kv * hd, 0.5).reshape(n_seqs, chunk, n_kv * hd)
    t_dev, p_dev = dev_u32(tables), dev_u32(np.full(n_seqs, prefix))
    kcd, vcd = torch.from_numpy(k_ch).cuda(), torch.from_numpy(v_ch).cuda()
    _lib.call("brc_kv_append", pool.handle, 0, C.c_void_p(t_dev.data_ptr()), stride, C.c_void_p(p_dev.data_ptr()), n_seqs, chunk, None,
              n_seqs * chunk, prefix + chunk, C.c_void_p(kcd.data_ptr()), C.c_void_p(vcd.data_ptr()), DTYPE_F32, None)
    for s in range(n_seqs):
        assert oracle.kv_append(kw, vw, tables[s], k_ch[s], v_ch[s], prefix, n_kv, hd) == 0
    pool.check()
    k_pool, v_pool = pool.read(0, 0).reshape(-1), pool.read(1, 0).reshape(-1)
    assert np.array_equal(k_pool, kw.view(np.uint16)), "K pool differs from the oracle's append + fork"
    assert np.array_equal(v_pool, vw.view(np.uint16)), "V pool differs from the oracle's append + fork"

    # ---- chunked prefill over prefix + chunk, causal
    q = oracle.to_f16(synth.normal(2005, n_seqs * chunk * n_head * hd)).reshape(n_seqs, chunk, n_head, hd)
    qd = torch.from_numpy(q).cuda().half()
    out = torch.full((n_seqs, chunk, n_head, hd), float("nan"), device="cuda")
    _lib.call("brc_paged_prefill_attn", pool.handle, 0, C.c_void_p(qd.data_ptr()), DTYPE_F16, n_head, None, 0,
              C.c_void_p(t_dev.data_ptr()), stride, C.c_void_p(p_dev.data_ptr()), n_seqs, chunk, prefix + chunk, 1.0 / 16.0,
              C.c_void_p(out.data_ptr()), None)
    pool.check()
    res = out.cpu().numpy()
    assert np.isfinite(res).all()
    for s in (0, 17, 63):
        want, _ = oracle.prefill_chunk(k_pool, v_pool, tables[s], prefix, q[s], n_head, n_kv, hd)
        max_abs, max_rel, _ = attention_errors(res[s], want)
        print(f"pipeline, sequence {s}: max_abs {max_abs:.2e} max_rel {max_rel:.2e}")
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL

    # ---- tear down: sequences drop their references, the owner its page, the tree is evicted
    for s in range(n_seqs):
        matched, mp = _arr(tables[s, :full_pages])
        _lib.call("brc_radix_release", radix, mp, full_pages)      # what brc_radix_match handed out
        pool.release_pages(tables[s, full_pages:])                 # the fork and the chunk's pages
    pool.release_pages(owner[full_pages:])
    for page in owner[:full_pages]:
        assert pool.refcount(int(page)) == 1
    evicted = C.c_uint32()
    _lib.call("brc_radix_evict", radix, full_pages, C.byref(evicted))
    assert evicted.value == full_pages
    assert pool.free_count() == free_at_start
    _lib.call("brc_radix_destroy", radix)
    pool.release()
