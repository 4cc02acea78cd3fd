"""Page gather, page copy and copy-on-write fork: bit-exact byte movers."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200.qsa import KvPool
from helpers import dev_u32, fill_pool_from_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("head_dim,n_kv,n_tokens", [(256, 2, 1025), (256, 2, 16), (128, 4, 7), (256, 2, 0)])
def test_gather_through_a_scattered_table(cuda_device, head_dim, n_kv, n_tokens):
    n_pages = 80
    pool = KvPool(0, 2, n_kv, head_dim, n_pages)
    k, v = fill_pool_from_host(pool, 1, 31)
    table = synth.permutation(9, n_pages)[:70]
    table_dev = dev_u32(table)
    kd, vd = pool.gather(1, table_dev, n_tokens)
    pool.check()
    if n_tokens:
        kb, _ = oracle.gather(k, table, n_tokens, n_kv, head_dim)
        vb, _ = oracle.gather(v, table, n_tokens, n_kv, head_dim)
        assert np.array_equal(kd.view(torch.int16).cpu().numpy().view(np.uint16), kb)
        assert np.array_equal(vd.view(torch.int16).cpu().numpy().view(np.uint16), vb)
    L = _lib.load()
    assert L.brc_page_gather(pool.handle, 1, C.c_void_p(table_dev.data_ptr()), 70, 70 * 16 + 1,
                             C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), None) == _lib.ERR_CAPACITY
    pool.release()


def test_page_copy_all_layers_matches_memcpy_reference(cuda_device):
    n_layers, n_pages = 4, 24
    pool = KvPool(0, n_layers, 2, 256, n_pages)
    host_k, host_v = [], []
    for layer in range(n_layers):
        k, v = fill_pool_from_host(pool, layer, 50 + 2 * layer)
        host_k.append(k)
        host_v.append(v)
    kb = np.concatenate(host_k).view(np.uint8).copy()
    vb = np.concatenate(host_v).view(np.uint8).copy()
    src = np.array([3, 3, 7, 20, 5], np.uint32)
    dst = np.array([0, 1, 8, 21, 5], np.uint32)   # includes a self-copy and a fan-out of page 3
    pool.copy_pages(src, dst)
    pool.check()
    oracle.page_copy(kb, vb, n_layers, n_pages, pool.half_page_bytes, src, dst)
    for layer in range(n_layers):
        n = n_pages * pool.half_page_bytes
        assert np.array_equal(pool.read(0, layer).reshape(-1).view(np.uint8), kb[layer * n:(layer + 1) * n])
        assert np.array_equal(pool.read(1, layer).reshape(-1).view(np.uint8), vb[layer * n:(layer + 1) * n])
    # an out-of-range id is skipped and reported
    pool.copy_pages([1], [n_pages])
    with pytest.raises(_lib.BrcError, match="page id >= n_pages"):
        pool.check()
    pool.release()


@pytest.mark.parametrize("n_tokens", [4088, 4096, 5, 16])
def test_copy_on_write_fork(cuda_device, n_tokens):
    """Full pages are shared (refcount + 1), a partial last page becomes a private copy in every
    layer; writing into the child's copy leaves the parent untouched."""
    n_layers = 3
    n_parent = (n_tokens + 15) // 16
    pool = KvPool(0, n_layers, 2, 256, n_parent + 8)
    parent = pool.alloc(n_parent)
    for layer in range(n_layers):
        fill_pool_from_host(pool, layer, 70 + 2 * layer)
    before = [(pool.read(0, l).copy(), pool.read(1, l).copy()) for l in range(n_layers)]
    child, fresh = pool.fork(parent, n_tokens)
    pool.check()
    full = n_tokens // 16
    assert child[:full].tolist() == parent[:full].tolist()
    for p in parent[:full]:
        assert pool.refcount(int(p)) == 2
    if n_tokens % 16:
        assert fresh is not None and child[full] == fresh and fresh not in parent.tolist()
        assert pool.refcount(int(parent[full])) == 1 and pool.refcount(fresh) == 1
        for l in range(n_layers):
            k, v = pool.read(0, l), pool.read(1, l)
            assert np.array_equal(k[fresh], before[l][0][parent[full]])
            assert np.array_equal(v[fresh], before[l][1][parent[full]])
            mask = np.ones(pool.n_pages, bool)
            mask[fresh] = False
            assert np.array_equal(k[mask], before[l][0][mask]) and np.array_equal(v[mask], before[l][1][mask])
    else:
        assert fresh is None
        assert pool.free_count() == 8
    # releasing the child gives back only what it owns
    pool.release_pages(child)
    for p in parent:
        assert pool.refcount(int(p)) == 1
    assert pool.free_count() == 8
    pool.release()


def test_pool_zero_and_poison(cuda_device):
    pool = KvPool(0, 2, 2, 128, 5)
    pool.poison_nan()
    assert (pool.read(0, 1) == 0xFFFF).all() and (pool.read(1, 0) == 0xFFFF).all()
    pool.zero()
    assert not pool.read(0, 1).any() and not pool.read(1, 0).any()
    assert pool.bytes() == 2 * 2 * 5 * 2 * 16 * 128 * 2
    pool.release()
