"""The C-ABI library without a GPU: it loads, exports exactly what include/breccia_kv.h declares,
its host-side state machine (allocator, refcounts, fork bookkeeping) works, and every compute entry
point refuses loudly instead of falling back to anything."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from breccia_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"BRC_API[^;()]*?\b(brc_\w+)\s*\(", text))
    return names


def exported_symbols():
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True)
    return {line.split()[-1] for line in out.stdout.splitlines() if " T " in line and "brc_" in line}


def test_library_exports_every_declared_symbol_and_nothing_else():
    decl, exp = declared_symbols(), exported_symbols()
    assert decl, "no declarations parsed"
    assert decl - exp == set(), f"declared but not exported: {sorted(decl - exp)}"
    assert exp - decl == set(), f"exported but not declared: {sorted(exp - decl)}"


def test_ctypes_binding_covers_the_header():
    bound = set(_lib.SIGNATURES) | set(_lib._SPECIAL)
    assert bound == declared_symbols()
    assert _lib.load().brc_abi_version() == 1


def test_header_compiles_as_c_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "breccia_kv.h"\nint main(void){return BRC_OK;}\n')
    inc = os.path.join(ROOT, "include")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", inc, "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-x", "c++", "-I", inc, "-c", str(src), "-o", str(tmp_path / "t2.o")], check=True)


@pytest.fixture()
def book():
    L = _lib.load()
    h = C.c_void_p()
    assert L.brc_pool_create_bookkeeping(12, 2, 256, 16, 10, C.byref(h)) == 0
    yield h
    L.brc_pool_destroy(h)


def _ids(a):
    a = np.ascontiguousarray(a, np.uint32)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint32))


def test_allocator_and_refcounts(book):
    L = _lib.load()
    free = C.c_uint32()
    L.brc_pages_free_count(book, C.byref(free))
    assert free.value == 10
    ids, p = _ids(np.zeros(4))
    assert L.brc_pages_alloc(book, 4, p) == 0
    assert sorted(ids.tolist()) == [0, 1, 2, 3]
    rc = C.c_uint32()
    for i in ids:
        L.brc_page_refcount(book, int(i), C.byref(rc))
        assert rc.value == 1
    assert L.brc_pages_retain(book, p, 2) == 0
    L.brc_page_refcount(book, int(ids[0]), C.byref(rc))
    assert rc.value == 2
    assert L.brc_pages_release(book, p, 4) == 0      # 0,1 -> 1 ; 2,3 -> free
    L.brc_pages_free_count(book, C.byref(free))
    assert free.value == 8
    # over-release is refused as a whole and changes nothing
    twice, pt = _ids([ids[0], ids[0]])
    assert L.brc_pages_release(book, pt, 2) == _lib.ERR_INVALID
    assert b"released more often" in L.brc_last_error()
    L.brc_page_refcount(book, int(ids[0]), C.byref(rc))
    assert rc.value == 1
    # exhausting the pool
    big, pb = _ids(np.zeros(9))
    assert L.brc_pages_alloc(book, 9, pb) == _lib.ERR_NO_PAGES
    assert b"9 pages requested, 8 free of 10" in L.brc_last_error()
    # retaining a free page or an out-of-range id is refused
    bad, pbad = _ids([ids[3]])
    assert L.brc_pages_retain(book, pbad, 1) == _lib.ERR_INVALID
    bad, pbad = _ids([77])
    assert L.brc_pages_retain(book, pbad, 1) == _lib.ERR_INVALID
    assert L.brc_page_refcount(book, 10, C.byref(rc)) == _lib.ERR_INVALID


def test_fork_of_page_aligned_sequence_shares_every_page(book):
    L = _lib.load()
    parent, pp = _ids(np.zeros(3))
    assert L.brc_pages_alloc(book, 3, pp) == 0
    child, pc = _ids(np.zeros(3))
    fresh = C.c_uint32()
    assert L.brc_seq_fork(book, pp, 48, pc, C.byref(fresh), None) == 0
    assert child.tolist() == parent.tolist() and fresh.value == 0xFFFFFFFF
    rc = C.c_uint32()
    for i in parent:
        L.brc_page_refcount(book, int(i), C.byref(rc))
        assert rc.value == 2
    # a partial last page needs a device copy: refused on a bookkeeping pool, refcounts untouched
    assert L.brc_seq_fork(book, pp, 40, pc, C.byref(fresh), None) == _lib.ERR_CUDA
    for i in parent:
        L.brc_page_refcount(book, int(i), C.byref(rc))
        assert rc.value == 2


def test_geometry_and_sizes(book):
    L = _lib.load()
    g = _lib.Geometry()
    assert L.brc_pool_geometry(book, C.byref(g)) == 0
    assert (g.n_layers, g.n_kv_head, g.head_dim, g.page_tokens, g.n_pages, g.device) == (12, 2, 256, 16, 10, -1)
    assert g.half_page_bytes == 16384          # K of one page of one layer; K + V = the reference's 32768
    assert g.total_bytes == 12 * 10 * 32768
    b = C.c_uint64()
    assert L.brc_pool_bytes(book, C.byref(b)) == 0 and b.value == g.total_bytes
    assert L.brc_decode_partial_bytes(1, 16, 256, C.byref(b)) == 0 and b.value == 16512


def test_compute_calls_refuse_without_a_gpu(book):
    """No CPU fallback anywhere: a pool without device memory makes every compute entry point fail."""
    L = _lib.load()
    dummy = C.c_void_p(0x1000)
    assert L.brc_kv_append(book, 0, dummy, 4, dummy, 1, 1, None, 1, 1, dummy, dummy, 0, None) == _lib.ERR_CUDA
    assert L.brc_page_gather(book, 0, dummy, 4, 1, dummy, dummy, None) == _lib.ERR_CUDA
    assert L.brc_page_copy(book, dummy, dummy, 1, None) == _lib.ERR_CUDA
    assert L.brc_paged_decode_attn(book, 0, dummy, 1, 16, None, 0, dummy, 4, dummy, 1, 16, 0.0625, dummy, dummy, 1 << 30, None) == _lib.ERR_CUDA
    assert L.brc_decode_partial(book, 0, dummy, 1, 16, dummy, 4, dummy, 1, 16, 0.0625, dummy, dummy, 1 << 30, None) == _lib.ERR_CUDA
    assert b"bookkeeping only" in L.brc_last_error()
    out = C.c_void_p()
    import torch
    if not torch.cuda.is_available():
        assert L.brc_pool_create(0, 1, 2, 256, 16, 8, C.byref(out)) == _lib.ERR_CUDA


def test_argument_validation_messages():
    L = _lib.load()
    out = C.c_void_p()
    assert L.brc_pool_create(0, 1, 2, 96, 16, 8, C.byref(out)) == _lib.ERR_UNSUPPORTED
    assert b"head_dim 96" in L.brc_last_error()
    assert L.brc_pool_create(0, 1, 2, 256, 32, 8, C.byref(out)) == _lib.ERR_UNSUPPORTED
    assert L.brc_pool_create(0, 0, 2, 256, 16, 8, C.byref(out)) == _lib.ERR_INVALID
    assert L.brc_pool_create(0, 1, 2, 256, 16, 8, None) == _lib.ERR_INVALID
    assert L.brc_decode_combine(0, None, 1, 0, 1, 16, 256, None, 0, None, None) == _lib.ERR_INVALID
