"""Radix prefix tree + refcounts on a bookkeeping pool (host-side state machine, no GPU)."""
import ctypes as C

import numpy as np
import pytest

from breccia_b200 import _lib

U32P = C.POINTER(C.c_uint32)


def arr(a):
    a = np.ascontiguousarray(a, np.uint32)
    return a, a.ctypes.data_as(U32P)


@pytest.fixture()
def env():
    L = _lib.load()
    pool, radix = C.c_void_p(), C.c_void_p()
    assert L.brc_pool_create_bookkeeping(12, 2, 256, 16, 64, C.byref(pool)) == 0
    assert L.brc_radix_create(pool, C.byref(radix)) == 0
    yield L, pool, radix
    L.brc_radix_destroy(radix)
    L.brc_pool_destroy(pool)


def refcount(L, pool, page):
    rc = C.c_uint32()
    assert L.brc_page_refcount(pool, int(page), C.byref(rc)) == 0
    return rc.value


def free(L, pool):
    n = C.c_uint32()
    L.brc_pages_free_count(pool, C.byref(n))
    return n.value


def test_shared_prefix_of_64_sequences(env):
    """The shared-prefix workload's bookkeeping: one 4096-token prefix (256 pages), 64 sequences that match it:
    every prefix page ends with 1 (owner) + 1 (tree) + 64 references; releasing the sequences and the
    owner leaves the tree as the only holder, and eviction then frees everything."""
    L, pool, radix = env
    L2 = _lib.load()
    big, radix2 = C.c_void_p(), C.c_void_p()
    assert L2.brc_pool_create_bookkeeping(12, 2, 256, 16, 400, C.byref(big)) == 0
    assert L2.brc_radix_create(big, C.byref(radix2)) == 0
    prefix = np.arange(4096, dtype=np.uint32) * 7 + 3
    pages, pp = arr(np.zeros(256))
    assert L2.brc_pages_alloc(big, 256, pp) == 0
    toks, tp = arr(prefix)
    new = C.c_uint32()
    assert L2.brc_radix_insert(radix2, tp, 4096, pp, 256, C.byref(new)) == 0 and new.value == 256
    got, gp = arr(np.zeros(300))
    n = C.c_uint32()
    for s in range(64):
        q, qp = arr(np.concatenate([prefix, np.arange(256, dtype=np.uint32) + 100000 * (s + 1)]))
        assert L2.brc_radix_match(radix2, qp, q.size, gp, 300, C.byref(n)) == 0
        assert n.value == 256 and np.array_equal(got[:256], pages)
    assert refcount(L2, big, pages[0]) == 66 and refcount(L2, big, pages[255]) == 66
    for s in range(64):
        assert L2.brc_pages_release(big, pp, 256) == 0
    assert L2.brc_pages_release(big, pp, 256) == 0          # the original owner lets go
    assert refcount(L2, big, pages[17]) == 1 and free(L2, big) == 144
    ev = C.c_uint32()
    assert L2.brc_radix_evict(radix2, 1000, C.byref(ev)) == 0 and ev.value == 256
    assert free(L2, big) == 400
    L2.brc_radix_destroy(radix2)
    L2.brc_pool_destroy(big)


def test_match_stops_at_first_difference_and_ignores_partial_pages(env):
    L, pool, radix = env
    pages, pp = arr(np.zeros(4))
    assert L.brc_pages_alloc(pool, 4, pp) == 0
    a = np.arange(64, dtype=np.uint32)
    _, ap = arr(a)
    new = C.c_uint32()
    assert L.brc_radix_insert(radix, ap, 64, pp, 4, C.byref(new)) == 0 and new.value == 4
    got, gp = arr(np.zeros(8))
    n = C.c_uint32()
    b = a.copy()
    b[40] = 999                                   # third page differs
    _, bp = arr(b)
    assert L.brc_radix_match(radix, bp, 64, gp, 8, C.byref(n)) == 0 and n.value == 2
    assert got[:2].tolist() == pages[:2].tolist()
    assert L.brc_radix_match(radix, ap, 47, gp, 8, C.byref(n)) == 0 and n.value == 2   # 47 tokens = 2 full pages
    assert L.brc_radix_match(radix, ap, 64, gp, 3, C.byref(n)) == 0 and n.value == 3   # capped by max_pages
    assert L.brc_radix_match(radix, ap, 15, gp, 8, C.byref(n)) == 0 and n.value == 0
    assert refcount(L, pool, pages[0]) == 1 + 1 + 3 and refcount(L, pool, pages[2]) == 1 + 1 + 1
    # inserting a diverging branch adopts only the new pages; an existing node keeps its page
    other, op = arr(np.zeros(4))
    assert L.brc_pages_alloc(pool, 4, op) == 0
    assert L.brc_radix_insert(radix, bp, 64, op, 4, C.byref(new)) == 0 and new.value == 2
    assert refcount(L, pool, other[0]) == 1 and refcount(L, pool, other[2]) == 2
    nodes, hits, miss, evs = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
    assert L.brc_radix_stats(radix, C.byref(nodes), C.byref(hits), C.byref(miss), C.byref(evs)) == 0
    assert nodes.value == 6 and hits.value == 7


def test_eviction_is_lru_over_unreferenced_leaves(env):
    L, pool, radix = env
    new, n, ev = C.c_uint32(), C.c_uint32(), C.c_uint32()
    seqs = []
    for s in range(3):
        pages, pp = arr(np.zeros(2))
        assert L.brc_pages_alloc(pool, 2, pp) == 0
        toks, tp = arr(np.arange(32, dtype=np.uint32) + 1000 * s)
        assert L.brc_radix_insert(radix, tp, 32, pp, 2, C.byref(new)) == 0
        assert L.brc_pages_release(pool, pp, 2) == 0        # only the tree holds them now
        seqs.append((toks, tp, pages))
    got, gp = arr(np.zeros(2))
    assert L.brc_radix_match(radix, seqs[0][1], 32, gp, 2, C.byref(n)) == 0   # touches sequence 0; caller holds it
    assert L.brc_radix_evict(radix, 2, C.byref(ev)) == 0 and ev.value == 2
    # the oldest unreferenced leaf chain went first: sequence 1's leaf, then its parent (now a leaf)
    assert refcount(L, pool, seqs[1][2][1]) == 0 and refcount(L, pool, seqs[1][2][0]) == 0
    assert refcount(L, pool, seqs[2][2][0]) == 1
    assert L.brc_radix_evict(radix, 10, C.byref(ev)) == 0 and ev.value == 2   # sequence 2; sequence 0 is held
    assert refcount(L, pool, seqs[0][2][1]) == 2
    assert L.brc_pages_release(pool, gp, 2) == 0
    assert L.brc_radix_evict(radix, 10, C.byref(ev)) == 0 and ev.value == 2
    assert free(L, pool) == 64


def test_insert_refuses_pages_the_caller_does_not_hold(env):
    L, pool, radix = env
    bogus, bp = arr([5])
    _, tp = arr(np.arange(16))
    new = C.c_uint32()
    assert L.brc_radix_insert(radix, tp, 16, bp, 1, C.byref(new)) == _lib.ERR_INVALID
    assert b"not allocated" in L.brc_last_error()


def test_prefix_tags_name_a_page_by_everything_up_to_it():
    """brc_radix_prefix_tags: one tag per FULL page; equal prefixes give equal tags, a change in an earlier page
    changes every later tag; the values are fixed (another process must compute the same ones)."""
    L = _lib.load()

    def tags_of(tokens, cap=16):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        out = np.zeros(cap, np.uint64)
        n = C.c_uint32()
        rc = L.brc_radix_prefix_tags(tokens.ctypes.data_as(C.POINTER(C.c_uint32)), tokens.size, 16, out.ctypes.data_as(C.POINTER(C.c_uint64)),
                                     cap, C.byref(n))
        return rc, out[:n.value]

    a = np.arange(100, dtype=np.uint32)
    rc, ta = tags_of(a)
    assert rc == 0 and ta.size == 6 and len(set(ta.tolist())) == 6 and (ta & 1).all()
    b = a.copy()
    b[20] = 999                                   # in the second page
    _, tb = tags_of(b)
    assert tb[0] == ta[0] and all(tb[i] != ta[i] for i in range(1, 6))
    assert np.array_equal(tags_of(a[:47])[1], ta[:2])
    assert tags_of(a[:15])[1].size == 0
    assert tags_of(a, cap=3)[0] == _lib.ERR_CAPACITY
    # pinned values: the hash is part of the file format of a persisted prefix
    assert [hex(int(t)) for t in tags_of(np.zeros(32, np.uint32))[1]] == ['0x94853c2e03ed1ec5', '0x735b619c55021e81']
