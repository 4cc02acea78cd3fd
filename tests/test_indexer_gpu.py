"""Indexer stages on the GPU (brc_idx_pool / brc_idx_tail / brc_idx_score) against the oracle, in the shapes of the
reference's own tests:

  * pooling across chunk boundaries, 64 tokens in chunks of 5 (the tail-source path), bar 1e-5 on the
    reference's measure (crates/breccia-kernels/tests/attn_conformance.rs:779-835);
  * its 2062-cell fixture END TO END: LCG streams 0xE1 (indexer query) / 0xE2 (pooled keys) / 0xE3-0xE6 (K, V, query,
    gate), score -> top-k -> attention over the selected blocks; the id list must equal the CPU selection exactly
    and in order, the output must meet the 1e-5 bar (attn_conformance.rs:897-1037);
  * a batch of sequences with multi-row chunks, where blocks that complete inside the chunk are dead for the
    rows that cannot see all of their cells (shaders/qsa_idx_score.comp:74-81)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from oracle import indexer_ref, prepare_ref
from oracle.topk_ref import topk_blocks
from breccia_b200 import _lib
from breccia_b200._lib import DTYPE_F32
from breccia_b200.qsa import IDX_BLOCK, IDX_DIM, IDX_N_HEAD, IndexerState, KvPool, Qsa, QsaState, sparse_attend
from breccia_b200.qsa import topk_blocks as gpu_topk_blocks
from helpers import attention_errors, dev_u32

pytestmark = pytest.mark.gpu
N_ROT, ROPE_BASE, EPS = 64, 1e7, 1e-6      # ops::MODEL_N_ROT, MODEL_ROPE_BASE, MODEL_RMS_EPS


def ref_measure(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float((np.abs(got - want) / np.maximum(np.abs(want), 1.0)).max())


def test_pooling_across_chunk_boundaries_matches_the_oracle(cuda_device):
    tokens, chunk, max_pos = 64, 5, 4096
    pool = KvPool(0, 1, 2, 256, 4)
    gamma = np.abs(oracle.normalish(0xBA, IDX_DIM)) + 0.5
    table = prepare_ref.rope_table(ROPE_BASE, N_ROT, max_pos)
    # two sequences in one batch: the reference's stream, and a second one shifted by two cells so that its
    # chunks straddle the block boundaries differently
    raws = [oracle.normalish(0xD1, tokens * IDX_DIM).reshape(tokens, IDX_DIM), oracle.normalish(0xD2, (tokens + 2) * IDX_DIM).reshape(tokens + 2, IDX_DIM)]
    state = IndexerState(pool, 2, tokens + 8)
    g_dev, t_dev = torch.from_numpy(gamma).cuda(), torch.from_numpy(table).cuda()
    # the second sequence already holds two cells: their raw keys sit in its tail, as a previous call would have left them
    state.tail[1, 0].copy_(torch.from_numpy(raws[1][0]))
    state.tail[1, 1].copy_(torch.from_numpy(raws[1][1]))
    for start in range(0, tokens, chunk):
        n = min(chunk, tokens - start)
        raw = np.stack([raws[0][start:start + n], raws[1][2 + start:2 + start + n]])
        state.append(torch.from_numpy(raw).cuda(), dev_u32([start, start + 2]), tokens + 2, g_dev, t_dev, N_ROT, EPS)
    pool.check()
    got = state.pooled.cpu().numpy()
    for s, cells in ((0, tokens), (1, tokens + 2)):
        want = indexer_ref.pool_keys(raws[s], cells, gamma, table, n_rot=N_ROT, eps=EPS)
        rel = ref_measure(got[s, :cells // IDX_BLOCK], want)
        print(f"indexer pooling, sequence {s}: {rel:.2e} (bar 1e-5, {cells // IDX_BLOCK} blocks, chunk {chunk})")
        assert rel <= 1e-5
    # the tail holds the raw keys of the block being filled: sequence 1 is at 66 cells = 16 blocks + 2
    assert np.array_equal(state.tail[1, :2].cpu().numpy(), raws[1][64:66])
    # refusals: the reference's wording when the completed blocks would not fit the state
    small = torch.zeros((2, 4, IDX_DIM), device="cuda")
    L = _lib.load()
    raw = torch.zeros((2, 4, IDX_DIM), device="cuda")
    rc = L.brc_idx_pool(pool.handle, C.c_void_p(raw.data_ptr()), C.c_void_p(state.tail.data_ptr()), C.c_void_p(g_dev.data_ptr()),
                        C.c_void_p(t_dev.data_ptr()), N_ROT, max_pos, EPS, C.c_void_p(dev_u32([16, 16]).data_ptr()), 2, 4, 20, IDX_DIM,
                        IDX_BLOCK, C.c_void_p(small.data_ptr()), 4, None)
    assert rc == _lib.ERR_CAPACITY and b"idx_pool would write pooled rows" in L.brc_last_error()
    pool.release()


def test_reference_fixture_2062_cells_score_topk_attention_end_to_end(cuda_device):
    n_head, n_kv, hd, cells = 24, 2, 256, 2062
    n_blocks = cells // IDX_BLOCK                       # 515 whole blocks + 2 tail cells
    pos0 = cells - 1
    idx_q = oracle.normalish(0xE1, IDX_N_HEAD * IDX_DIM).reshape(1, IDX_N_HEAD, IDX_DIM)
    pooled = oracle.normalish(0xE2, (n_blocks + 1) * IDX_DIM).reshape(n_blocks + 1, IDX_DIM)
    k_all = oracle.normalish(0xE3, cells * n_kv * hd).reshape(cells, n_kv * hd)
    v_all = oracle.normalish(0xE4, cells * n_kv * hd).reshape(cells, n_kv * hd)
    q = oracle.normalish(0xE5, n_head * hd).reshape(1, n_head, hd)
    q_full = oracle.normalish(0xE6, n_head * 2 * hd).reshape(1, n_head, 2, hd)
    pool = KvPool(0, 1, n_kv, hd, 4096 // 16)
    qsa = Qsa(pool, n_head)
    state = QsaState(pool, cells)
    for start in range(0, cells, 256):                  # the cache filled in 256-cell chunks, as the reference's test does
        n = min(256, cells - start)
        ws = qsa.workspace(n)
        ws.k_cur.copy_(torch.from_numpy(k_all[start:start + n]))
        ws.v_cur.copy_(torch.from_numpy(v_all[start:start + n]))
        qsa.kv_append(state, ws, start)
    idx = IndexerState(pool, 1, 4096)
    idx.pooled[0, :n_blocks + 1].copy_(torch.from_numpy(pooled))
    p_dev = dev_u32([pos0])
    scores = idx.score(torch.from_numpy(idx_q).cuda(), p_dev, 1, n_blocks)
    ids, counts = gpu_topk_blocks(pool, scores, p_dev, 1, topk=512)
    pool.check()
    # reference: score the same pooled keys, select, then attend
    want_scores = indexer_ref.indexer_score(idx_q[0], pooled, n_blocks, pos0)
    assert ref_measure(scores.cpu().numpy()[0], want_scores) <= 1e-5
    want_ids = topk_blocks(want_scores.astype(np.float32), 512, own_block=pos0 // IDX_BLOCK)
    count = int(counts.cpu().numpy()[0])
    assert count == len(want_ids) == 513, "selection length"
    assert ids.cpu().numpy()[0, :count].tolist() == want_ids, "selection order/set differs (descending score, ties to the lower block, tail last)"
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    gate = torch.from_numpy(q_full).cuda()
    tables = state.page_table_dev.unsqueeze(0).contiguous()
    sparse_attend(pool, 0, torch.from_numpy(q).cuda(), n_head, tables, p_dev, 1, ids, counts, cells, out,
                  gate=gate.view(-1)[hd:], gate_head_stride=2 * hd)
    pool.check()
    want = oracle.attend(q[0], oracle.to_f16(k_all), oracle.to_f16(v_all), oracle.cells_of(want_ids, IDX_BLOCK), pos0, n_head, n_kv, hd,
                         gate=q_full[0, :, 1, :])
    max_abs, max_rel, ref = attention_errors(out.cpu().numpy()[0], want)
    print(f"reference fixture end to end: selected {count} blocks, attention max_abs {max_abs:.2e} ref_measure {ref:.2e} (bar 1e-5)")
    assert ref <= 1e-5 and max_abs <= 2e-3
    state.release()
    pool.release()


def test_scores_of_a_batch_with_multi_row_chunks(cuda_device):
    """Three sequences, five rows each: a block that completes inside the chunk is dead for the rows before its
    last cell, live after; n_blocks is not a multiple of anything the kernel steps by."""
    n_seqs, rows_per_seq, n_blocks = 3, 5, 1037
    pos0s = np.array([4140, 4141, 7])                      # the last sequence sees only blocks 0 and 1 at its last rows
    pool = KvPool(0, 1, 2, 256, 4)
    idx = IndexerState(pool, n_seqs, n_blocks * IDX_BLOCK)
    pooled = oracle.normalish(0x71, n_seqs * idx.max_blocks * IDX_DIM).reshape(n_seqs, idx.max_blocks, IDX_DIM)
    idx.pooled.copy_(torch.from_numpy(pooled))
    q = oracle.normalish(0x72, n_seqs * rows_per_seq * IDX_N_HEAD * IDX_DIM).reshape(n_seqs * rows_per_seq, IDX_N_HEAD, IDX_DIM)
    scores = idx.score(torch.from_numpy(q).cuda(), dev_u32(pos0s), rows_per_seq, n_blocks).cpu().numpy()
    pool.check()
    for s in range(n_seqs):
        for t in range(rows_per_seq):
            row = s * rows_per_seq + t
            want = indexer_ref.indexer_score(q[row], pooled[s], n_blocks, int(pos0s[s]) + t, mask="last")
            dead = np.isneginf(want)
            assert np.array_equal(scores[row] <= -1e29, dead), f"sequence {s} row {t}: dead blocks differ"
            assert ref_measure(scores[row][~dead], want[~dead]) <= 1e-5
    assert (scores[2 * rows_per_seq + 0] > -1e29).sum() == 2 and (scores[2 * rows_per_seq + 4] > -1e29).sum() == 3
    pool.release()


@pytest.mark.parametrize("rows_per_seq,n_blocks,pos0s", [(17, 777, [3100, 40]), (8, 512, [2047, 2040]), (2, 65, [300, 3])])
def test_scores_of_row_tiles_that_share_the_keys(cuda_device, rows_per_seq, n_blocks, pos0s):
    """More than one row per sequence takes the kernel that holds a key in registers for eight rows: tiles that are
    not full (17 = 8 + 8 + 1), blocks past the last row's reach, block counts that are no multiple of the 512
    a CTA covers."""
    n_seqs = len(pos0s)
    pool = KvPool(0, 1, 2, 256, 4)
    idx = IndexerState(pool, n_seqs, n_blocks * IDX_BLOCK)
    pooled = oracle.normalish(0x81, n_seqs * idx.max_blocks * IDX_DIM).reshape(n_seqs, idx.max_blocks, IDX_DIM)
    idx.pooled.copy_(torch.from_numpy(pooled))
    q = oracle.normalish(0x82, n_seqs * rows_per_seq * IDX_N_HEAD * IDX_DIM).reshape(n_seqs * rows_per_seq, IDX_N_HEAD, IDX_DIM)
    scores = idx.score(torch.from_numpy(q).cuda(), dev_u32(pos0s), rows_per_seq, n_blocks).cpu().numpy()
    pool.check()
    for s in range(n_seqs):
        for t in range(rows_per_seq):
            row = s * rows_per_seq + t
            want = indexer_ref.indexer_score(q[row], pooled[s], n_blocks, int(pos0s[s]) + t, mask="last")
            dead = np.isneginf(want)
            assert np.array_equal(scores[row] <= -1e29, dead), f"sequence {s} row {t}: dead blocks differ"
            if (~dead).any():
                assert ref_measure(scores[row][~dead], want[~dead]) <= 1e-5
    pool.release()
