"""Page files in the reference's dump format (p<pos>-b<block>-qsa_{k,v}.bin): what brc_state_dump writes
for a sequence whose pages are scattered in the shared pool must be, byte for byte, what the reference
writes for the same cache contents — the first ceil((pos+1)/16) pages of an identity-mapped pool
(crates/breccia-engine/src/graph.rs:2204-2228) — and brc_state_load must bring the pages back."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200.qsa import KvPool, Qsa, QsaState

pytestmark = pytest.mark.gpu
U32P = C.POINTER(C.c_uint32)


def test_dump_matches_identity_pool_bytes_and_load_restores(cuda_device, tmp_path):
    n_head, n_kv, hd, n_tokens, pos = 16, 2, 256, 300, 299
    n_pages = pos // 16 + 1                       # 19
    pool = KvPool(0, 2, n_kv, hd, 64)
    pool.poison_nan()
    table = synth.permutation(21, 64)[:n_pages].astype(np.uint32)
    spare = pool.alloc(64)                        # take every page so that the permutation is valid
    state = QsaState(pool, n_pages * 16, layer=1, block_table=table)
    qsa = Qsa(pool, n_head)
    ws = qsa.workspace(n_tokens)
    k = synth.normal(22, n_tokens * n_kv * hd, 0.5).reshape(n_tokens, n_kv * hd)
    v = synth.normal(23, n_tokens * n_kv * hd, 0.5).reshape(n_tokens, n_kv * hd)
    ws.k_cur.copy_(torch.from_numpy(k))
    ws.v_cur.copy_(torch.from_numpy(v))
    qsa.kv_append(state, ws, 0)
    torch.cuda.synchronize()
    # the reference's bytes: the same append into an identity-mapped pool of n_pages pages; cells past the
    # sequence keep whatever the pool held (here the NaN pattern 0xFFFF of poison_nan)
    words = n_pages * n_kv * 16 * hd // 2
    kp = np.full(words, 0xFFFFFFFF, np.uint32)
    vp = np.full(words, 0xFFFFFFFF, np.uint32)
    assert oracle.kv_append(kp, vp, np.arange(n_pages, dtype=np.uint32), k, v, 0, n_kv, hd) == 0
    d = str(tmp_path).encode()
    _lib.call("brc_state_dump", pool.handle, 1, table.ctypes.data_as(U32P), n_pages, pos, 7, d, None)
    kf = np.fromfile(os.path.join(str(tmp_path), "p000299-b07-qsa_k.bin"), np.uint32)
    vf = np.fromfile(os.path.join(str(tmp_path), "p000299-b07-qsa_v.bin"), np.uint32)
    assert kf.size == words and vf.size == words          # f16_pool_bytes(pages), qsa/mod.rs:316-388
    assert np.array_equal(kf, kp) and np.array_equal(vf, vp)

    # load into other pages of another layer and compare page by page
    table2 = synth.permutation(24, 64)[:n_pages].astype(np.uint32)
    _lib.call("brc_state_load", pool.handle, 0, table2.ctypes.data_as(U32P), n_pages, pos, 7, d, None)
    k0 = pool.read(0, 0).reshape(64, -1)
    v0 = pool.read(1, 0).reshape(64, -1)
    assert np.array_equal(k0[table2].reshape(-1).view(np.uint32), kp)
    assert np.array_equal(v0[table2].reshape(-1).view(np.uint32), vp)

    # refusals: table too short for the position, file of another geometry, missing file
    L = _lib.load()
    assert L.brc_state_dump(pool.handle, 1, table.ctypes.data_as(U32P), n_pages - 1, pos, 7, d, None) == _lib.ERR_CAPACITY
    assert L.brc_state_load(pool.handle, 0, table2.ctypes.data_as(U32P), n_pages, pos - 16, 7, d, None) == _lib.ERR_INVALID  # no such file
    os.rename(os.path.join(str(tmp_path), "p000299-b07-qsa_k.bin"), os.path.join(str(tmp_path), "p000283-b07-qsa_k.bin"))
    os.rename(os.path.join(str(tmp_path), "p000299-b07-qsa_v.bin"), os.path.join(str(tmp_path), "p000283-b07-qsa_v.bin"))
    assert L.brc_state_load(pool.handle, 0, table2.ctypes.data_as(U32P), n_pages, 283, 7, d, None) == _lib.ERR_INVALID
    assert b"does not hold exactly" in L.brc_last_error()
    pool.release_pages(spare)
    pool.release()


def test_q8_0_v_pool_dumps_the_reference_vq8_part_and_loads_it_back(cuda_device, tmp_path):
    """A q8_0 V pool writes p<pos>-b<block>-qsa_vq8.bin (q8v_pool_bytes(pages) raw bytes, graph.rs:2183-2186) beside
    the binary16 K file: the bytes an identity-mapped pool would hold after the same appends."""
    from oracle import q8v

    n_head, n_kv, hd, n_tokens, pos = 24, 2, 256, 100, 99
    n_pages = pos // 16 + 1                       # 7
    pool = KvPool(0, 1, n_kv, hd, 32, v_q8=True)
    table = synth.permutation(31, 32)[:n_pages].astype(np.uint32)
    spare = pool.alloc(32)
    state = QsaState(pool, n_pages * 16, layer=0, block_table=table)
    qsa = Qsa(pool, n_head)
    ws = qsa.workspace(n_tokens)
    k = synth.normal(32, n_tokens * n_kv * hd, 0.5).reshape(n_tokens, n_kv * hd)
    v = synth.normal(33, n_tokens * n_kv * hd, 0.5).reshape(n_tokens, n_kv * hd)
    ws.k_cur.copy_(torch.from_numpy(k))
    ws.v_cur.copy_(torch.from_numpy(v))
    qsa.kv_append(state, ws, 0)
    torch.cuda.synchronize()
    want_v = np.zeros((n_pages * n_kv * 16, q8v.row_bytes(hd)), np.uint8)      # the pool was zeroed at creation
    q8v.v_append(want_v, np.arange(n_pages, dtype=np.uint32), v, 0, n_kv, hd)
    d = str(tmp_path).encode()
    _lib.call("brc_state_dump", pool.handle, 0, table.ctypes.data_as(U32P), n_pages, pos, 3, d, None)
    vf = np.fromfile(os.path.join(str(tmp_path), "p000099-b03-qsa_vq8.bin"), np.uint8)
    kf = np.fromfile(os.path.join(str(tmp_path), "p000099-b03-qsa_k.bin"), np.uint8)
    assert vf.size == n_pages * n_kv * 16 * (hd // 32) * 36 and kf.size == n_pages * n_kv * 16 * hd * 2
    assert np.array_equal(vf, want_v.reshape(-1))
    assert not os.path.exists(os.path.join(str(tmp_path), "p000099-b03-qsa_v.bin"))
    table2 = synth.permutation(34, 32)[:n_pages].astype(np.uint32)
    before_k = pool.read(0, 0).reshape(32, -1)[table].copy()
    _lib.call("brc_state_load", pool.handle, 0, table2.ctypes.data_as(U32P), n_pages, pos, 3, d, None)
    rows = n_kv * 16
    v_now = pool.read(1, 0).reshape(32, rows * q8v.row_bytes(hd))
    assert np.array_equal(v_now[table2].reshape(-1), want_v.reshape(-1))
    assert np.array_equal(pool.read(0, 0).reshape(32, -1)[table2], before_k)
    pool.release_pages(spare)
    pool.release()
