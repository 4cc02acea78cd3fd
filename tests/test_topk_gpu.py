"""Top-k block selection on the GPU (brc_topk_blocks) against the oracle, id for id and in order — the reference
tests its shader the same way (exact ids, crates/breccia-kernels/tests/attn_conformance.rs:1457-1513).  Scores are
drawn from a small set of values so that ties are everywhere, some blocks are dead, and row lengths cross the
one-sort limit (8192 blocks) into the chunked path."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle.topk_ref import dense_blocks, topk_blocks
from breccia_b200 import _lib
from breccia_b200.qsa import KvPool
from helpers import dev_u32

pytestmark = pytest.mark.gpu
P = lambda x: C.c_void_p(x.data_ptr())


def run_topk(pool, scores, pos0s, rows_per_seq, k, max_ids, dense=False):
    rows, n_blocks = scores.shape
    sd = torch.from_numpy(scores).cuda()
    before = sd.clone()
    ids = torch.full((rows, max_ids), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
    counts = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    p_dev = dev_u32(np.asarray(pos0s))
    _lib.call("brc_topk_blocks", pool.handle, P(sd), len(pos0s), rows_per_seq, n_blocks, k, max_ids, P(p_dev), 1 if dense else 0,
              P(ids), P(counts), None)
    pool.check()
    assert torch.equal(sd.view(torch.int32), before.view(torch.int32)), "the scores must be left untouched"
    return ids.cpu().numpy(), counts.cpu().numpy()


def make_scores(seed, rows, n_blocks, levels):
    rng = np.random.default_rng(seed)
    s = rng.integers(-levels, levels, size=(rows, n_blocks)).astype(np.float32) * np.float32(0.25)
    s[rng.random((rows, n_blocks)) < 0.1] = np.float32(-1.0e30)       # masked by the score stage
    s[rng.random((rows, n_blocks)) < 0.01] = np.float32(np.nan)
    s[rng.random((rows, n_blocks)) < 0.02] = np.float32(-0.0)
    return s


@pytest.mark.parametrize("n_blocks,k,levels", [(3, 512, 2), (100, 512, 4), (513, 512, 50), (700, 512, 3), (8192, 512, 1000),
                                               (8193, 512, 20), (20000, 512, 5000), (20000, 37, 3), (65536, 512, 100000),
                                               (512, 512, 30), (600, 300, 7), (2048, 512, 2), (5000, 1000, 40), (4096, 1024, 100000),
                                               (9000, 1024, 9), (3000, 512, 1000), (4096, 500, 50), (8192, 512, 10 ** 7), (6000, 512, 1)])
def test_selection_matches_the_oracle_id_for_id(cuda_device, n_blocks, k, levels):
    pool = KvPool(0, 1, 2, 256, 4)
    n_seqs, rows_per_seq = 3, 2
    max_ids = min(n_blocks, k) + 1
    scores = make_scores(n_blocks + k, n_seqs * rows_per_seq, n_blocks, levels)
    scores[1, :] = np.float32(-1.0e30)                               # a row with nothing visible: only its own block
    pos0s = [4 * n_blocks - 9, 5, 4 * (n_blocks // 2)]
    ids, counts = run_topk(pool, scores, pos0s, rows_per_seq, k, max_ids)
    for row in range(n_seqs * rows_per_seq):
        own = (pos0s[row // rows_per_seq] + row % rows_per_seq) // 4
        want = topk_blocks(scores[row], k, own, max_ids)
        assert counts[row] == len(want), f"row {row}: count {counts[row]} != {len(want)}"
        assert ids[row, :len(want)].tolist() == want, f"row {row}"
    pool.release()


def test_dense_selection_and_refusals(cuda_device):
    pool = KvPool(0, 1, 2, 256, 4)
    scores = np.zeros((4, 40), np.float32)
    pos0s = [0, 158]                                                 # rows at positions 0, 1, 158, 159 -> own blocks 0, 0, 39, 39
    ids, counts = run_topk(pool, scores, pos0s, 2, 512, 41, dense=True)
    for row, pos in enumerate([0, 1, 158, 159]):
        want = dense_blocks(40, pos // 4, 41)
        assert counts[row] == len(want) and ids[row, :len(want)].tolist() == want
    ids, counts = run_topk(pool, scores, [400], 4, 512, 41, dense=True)    # own block 100 lies beyond the 40 scored blocks
    assert counts.tolist() == [41] * 4 and ids[0, 40] == 100
    x = torch.zeros(64, device="cuda")
    for args, code in (((P(x), 1, 1, 40, 512, 40), _lib.ERR_INVALID),            # max_ids too small for 40 blocks + own
                       ((P(x), 1, 1, 40, 2000, 41), _lib.ERR_UNSUPPORTED)):      # k beyond the kernel's survivors
        with pytest.raises(_lib.BrcError) as err:
            _lib.call("brc_topk_blocks", pool.handle, *args, P(x), 0, P(x), P(x), None)
        assert err.value.code == code
    pool.release()


def test_selection_feeds_the_selected_block_attention(cuda_device):
    """Scores -> brc_topk_blocks -> brc_paged_sparse_attn on the lists it wrote (descending-score order, own block last)
    against the oracle's attention over the oracle's selection: the two stages fit together without a host round trip."""
    import oracle
    from breccia_b200 import synth
    from breccia_b200.qsa import sparse_attend, topk_blocks as gpu_topk
    from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, fill_pool_from_host

    n_head, n_kv, hd, pos, k_sel = 16, 2, 256, 4101, 64
    n_blocks = pos // 4 + 1
    n_pages = (pos + 16) // 16
    pool = KvPool(0, 1, n_kv, hd, n_pages + 3)
    k, v = fill_pool_from_host(pool, 0, 930)
    table = synth.permutation(931, n_pages + 3)[:n_pages].astype(np.uint32)
    scores = make_scores(932, 1, n_blocks, 6)
    scores[0, n_blocks - 1] = np.float32(-1.0e30)          # the row's own block is not scored: it must still be attended
    q = oracle.normalish(933, n_head * hd).reshape(1, n_head, hd)
    ids, counts = gpu_topk(pool, torch.from_numpy(scores).cuda(), dev_u32(np.array([pos])), 1, topk=k_sel)
    want_ids = topk_blocks(scores[0], k_sel, pos // 4, k_sel + 1)
    assert counts.item() == len(want_ids) == k_sel + 1 and ids[0].tolist() == want_ids
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    sparse_attend(pool, 0, torch.from_numpy(q).cuda(), n_head, dev_u32(table[None, :]), dev_u32(np.array([pos])), 1, ids, counts,
                  pos + 1, out)
    pool.check()
    _, kf = oracle.gather(k, table, n_pages * 16, n_kv, hd)
    _, vf = oracle.gather(v, table, n_pages * 16, n_kv, hd)
    want = oracle.attend(q[0], kf, vf, oracle.cells_of(want_ids, 4), pos, n_head, n_kv, hd)
    max_abs, max_rel, ref = attention_errors(out.cpu().numpy()[0], want)
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5
    pool.release()
