"""The long-context and the shared-prefix workloads at their full sizes (one layer each): the GPU result
against the oracle where the oracle finishes in seconds, and through size-independent properties otherwise."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16
from breccia_b200.qsa import DecodeBatch, KvPool, decode_combine, decode_partial_bytes
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32, fill_pool_from_host

pytestmark = pytest.mark.gpu


def test_single_stream_of_131072_cells_matches_the_oracle_and_its_split_halves(cuda_device):
    """One sequence of 131 072 cells (8192 pages scattered in the pool), GQA 16q/2kv, head_dim 256: the one-GPU
    decode output against the oracle; the same output from two half-range partials merged (what two ranks of the
    split-KV path compute); two launches bit-identical."""
    n_head, n_kv, hd, n_tokens = 16, 2, 256, 131072
    n_pages = n_tokens // 16
    pool = KvPool(0, 1, n_kv, hd, n_pages + 16)
    k, v = fill_pool_from_host(pool, 0, 500)
    table = synth.permutation(501, n_pages + 16)[:n_pages].astype(np.uint32)
    q = oracle.to_f16(synth.normal(502, n_head * hd)).reshape(1, n_head, hd)
    qd = torch.from_numpy(q).cuda().half()
    batch = DecodeBatch(pool, n_head, table[None, :], [n_tokens])
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    batch.attend(0, qd, out)
    pool.check()
    got = out.cpu().numpy()
    want, _ = oracle.decode_batch(k, v, table[None, :], np.array([n_tokens]), q, n_head, n_kv, hd)
    max_abs, max_rel, ref = attention_errors(got, want)
    print(f"131072 cells: max_abs {max_abs:.2e} max_rel {max_rel:.2e} ref_measure {ref:.2e}")
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5
    again = torch.empty_like(out)
    batch.attend(0, qd, again)
    assert torch.equal(out, again)
    # two halves, as two ranks would hold them
    nbytes = decode_partial_bytes(1, n_head, hd)
    parts = torch.zeros(2 * nbytes, dtype=torch.uint8, device="cuda")
    half = n_tokens // 2
    lo = DecodeBatch(pool, n_head, table[None, : half // 16], [half])
    hi = DecodeBatch(pool, n_head, table[None, half // 16:], [n_tokens - half])
    lo.partial(0, qd, parts[:nbytes])
    hi.partial(0, qd, parts[nbytes:])
    merged = torch.empty_like(out)
    decode_combine(0, parts, 2, nbytes, 1, n_head, hd, merged)
    pool.check()
    assert np.abs(merged.cpu().numpy() - want).max() <= ATTN_MAX_ABS
    assert np.abs(merged.cpu().numpy() - got).max() <= 2e-6
    pool.release()


def test_64_sequences_sharing_a_4096_token_prefix_chunked_prefill(cuda_device):
    """64 sequences, one 4096-token prefix in 256 shared pages, a 256-token chunk each (GQA 16q/2kv, head_dim 256):
    three sequences against the oracle row by row; a sequence given the same suffix pages and queries as another
    must come out bit-identical; every output finite."""
    n_head, n_kv, hd, prefix, chunk, n_seqs = 16, 2, 256, 4096, 256, 64
    n_prefix_pages, per_seq = prefix // 16, chunk // 16
    n_pool = n_prefix_pages + n_seqs * per_seq + 8
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    k, v = fill_pool_from_host(pool, 0, 510)
    perm = synth.permutation(511, n_pool).astype(np.uint32)
    tables = np.zeros((n_seqs, n_prefix_pages + per_seq), np.uint32)
    tables[:, :n_prefix_pages] = perm[:n_prefix_pages]
    for s in range(n_seqs):
        tables[s, n_prefix_pages:] = perm[n_prefix_pages + s * per_seq: n_prefix_pages + (s + 1) * per_seq]
    tables[63, n_prefix_pages:] = tables[5, n_prefix_pages:]          # sequence 63 is sequence 5 again
    q = oracle.to_f16(synth.normal(512, n_seqs * chunk * n_head * hd)).reshape(n_seqs, chunk, n_head, hd)
    q[63] = q[5]
    qd = torch.from_numpy(q).cuda().half()
    out = torch.full((n_seqs, chunk, n_head, hd), float("nan"), device="cuda")
    t_dev, p_dev = dev_u32(tables), dev_u32(np.full(n_seqs, prefix))
    _lib.call("brc_paged_prefill_attn", pool.handle, 0, C.c_void_p(qd.data_ptr()), DTYPE_F16, n_head, None, 0,
              C.c_void_p(t_dev.data_ptr()), tables.shape[1], C.c_void_p(p_dev.data_ptr()), n_seqs, chunk, prefix + chunk,
              1.0 / 16.0, C.c_void_p(out.data_ptr()), None)
    pool.check()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.array_equal(got[63], got[5])
    for s in (0, 5, 40):
        want, _ = oracle.prefill_chunk(k, v, tables[s], prefix, q[s], n_head, n_kv, hd)
        max_abs, max_rel, _ = attention_errors(got[s], want)
        print(f"sequence {s}: max_abs {max_abs:.2e} max_rel {max_rel:.2e}")
        assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
    pool.release()
