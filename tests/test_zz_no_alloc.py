"""brc_paged_decode_attn_static: decode attention for callers that must not allocate on the device.

Some users of this library cannot call cudaMalloc once they are running: an engine that gave all of
its HBM to its own arena at start-up, or a decode loop for which cudaMalloc's device-wide
synchronisation is a stall it cannot take.  For them the library offers an entry point whose split-KV
scratch is a fixed 4 MiB array inside the library image instead of a caller-provided workspace.

This file is collected last on purpose: if it fails under `-x`, every other test has already run.
It must pass both on its own (fresh process: the first call does the address look-up) and after the
rest of the suite."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16
from breccia_b200.qsa import DecodeBatch, KvPool
from helpers import fill_pool_from_host

pytestmark = pytest.mark.gpu


def _static_call(pool, batch, layer, q, out, n_head):
    _lib.call("brc_paged_decode_attn_static", pool.handle, layer, C.c_void_p(q.data_ptr()), DTYPE_F16, n_head, None, 0,
              C.c_void_p(batch.block_tables.data_ptr()), batch.table_stride, C.c_void_p(batch.seq_lens.data_ptr()),
              batch.n_seqs, int(batch.seq_lens_host.max()), batch.scale, C.c_void_p(out.data_ptr()), None)


def test_static_scratch_entry_point_equals_the_workspace_one_twice_in_a_row(cuda_device):
    n_head, n_kv, hd = 16, 2, 256
    results = []
    for call, (seed, lens) in enumerate([(301, [700, 33, 2049, 16, 1, 512]), (302, [4097, 5, 160, 1023])]):
        lens = np.asarray(lens)
        tables, n_pool = synth.scattered_tables(seed, lens, pool_factor=1.3)
        pool = KvPool(0, 2, n_kv, hd, n_pool)
        k_host, v_host = fill_pool_from_host(pool, 1, seed + 10)
        batch = DecodeBatch(pool, n_head, tables, lens)
        q32 = oracle.to_f16(synth.normal(seed + 20, lens.size * n_head * hd)).reshape(lens.size, n_head, hd)
        q = torch.from_numpy(q32).cuda().half()
        want = torch.full((lens.size, n_head, hd), float("nan"), device="cuda")
        got = torch.full_like(want, float("nan"))
        batch.attend(1, q, want)                      # existing entry point, caller-owned workspace
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _static_call(pool, batch, 1, q, got, n_head)  # new entry point, built-in scratch
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        # the property in the entry point's name: the call (the very first one on this device included, which looks
        # the array's address up) takes no device memory
        assert free_after >= free_before, f"call {call}: {free_before - free_after} bytes of device memory went away"
        pool.check()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        ref, _ = oracle.decode_batch(k_host, v_host, tables, lens, q32, n_head, n_kv, hd)
        assert np.abs(g - ref).max() <= 2e-3          # and against the CPU oracle directly
        assert np.isfinite(g).all()
        # same kernels, same schedule, same arithmetic: the tolerance of the attention tests is the
        # bar, and in fact the two agree to the last bit
        assert np.abs(g - w).max() <= 2e-3
        assert np.array_equal(g, w), f"call {call}: static-scratch result differs from the workspace result"
        results.append(g)
        pool.release()
    assert results[0].shape != results[1].shape  # the second call really was a different batch


def test_static_scratch_refuses_a_batch_beyond_its_array(cuda_device):
    pool = KvPool(0, 1, 2, 256, 8)
    L = _lib.load()
    n = 4096
    q = torch.zeros((1, 16, 256), dtype=torch.half, device="cuda")
    rc = L.brc_paged_decode_attn_static(pool.handle, 0, C.c_void_p(q.data_ptr()), DTYPE_F16, 16, None, 0,
                                        C.c_void_p(q.data_ptr()), 4, C.c_void_p(q.data_ptr()), n, 16, 0.0625,
                                        C.c_void_p(q.data_ptr()), None)
    assert rc == _lib.ERR_CAPACITY
    msg = L.brc_last_error().decode()
    assert "built-in array holds 4194304" in msg and "brc_paged_decode_attn" in msg
    pool.release()
