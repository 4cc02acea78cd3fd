"""The oracle's indexer functions against the reference's own unit tests and contracts (no GPU)."""
import numpy as np

import oracle
from oracle import indexer_ref, prepare_ref


def test_completed_blocks_follow_the_trigger_cell():
    """crates/breccia-kernels/src/qsa/mod.rs:2110-2127, value for value."""
    bc = indexer_ref.blocks_completed
    assert bc(0, 1) == (0, 0) and bc(3, 1) == (0, 1) and bc(4, 1) == (1, 0) and bc(7, 1) == (1, 1)
    assert bc(0, 4) == (0, 1) and bc(2, 4) == (0, 1) and bc(0, 16) == (0, 4) and bc(0, 5) == (0, 1) and bc(5, 5) == (1, 1)


def test_pooling_takes_the_mean_of_raw_keys_then_norm_then_rotation_at_the_first_cell():
    """The three properties qsa_idx_pool.comp:10-14 pins: mean over RAW keys before the norm; rotation at the
    block's first cell 4b; dims beyond n_rot pass through."""
    cells, dim, n_rot = 16, 128, 64
    raw = oracle.normalish(0xD1, cells * dim).reshape(cells, dim)
    gamma = np.abs(oracle.normalish(0xBA, dim)) + 0.5
    table = prepare_ref.rope_table(10000.0, n_rot, 64)
    pooled = indexer_ref.pool_keys(raw, cells, gamma, table, n_rot=n_rot)
    assert pooled.shape == (4, dim)
    b = 2
    mean = raw[4 * b:4 * b + 4].astype(np.float64).mean(axis=0)
    normed = mean / np.sqrt((mean * mean).mean() + 1e-6) * gamma
    assert np.allclose(pooled[b, n_rot:], normed[n_rot:], rtol=1e-6, atol=1e-6)
    c, s = table[4 * b, :, 0].astype(np.float64), table[4 * b, :, 1].astype(np.float64)
    assert np.allclose(pooled[b, :32], normed[:32] * c - normed[32:64] * s, rtol=1e-5, atol=1e-6)
    assert np.allclose(pooled[b, 32:64], normed[:32] * s + normed[32:64] * c, rtol=1e-5, atol=1e-6)
    # rotating at the block's LAST cell keeps every magnitude but is a different vector
    wrong = prepare_ref.rope_apply(normed.astype(np.float32)[None, :], dim, n_rot, table, [4 * b + 3])[0]
    assert not np.allclose(pooled[b, :64], wrong[:64], atol=1e-3)


def test_scores_are_scaled_relu_sums_and_future_blocks_are_dead():
    q = oracle.normalish(0xE1, 4 * 128).reshape(4, 128)
    pooled = oracle.normalish(0xE2, 10 * 128).reshape(10, 128)
    sc = indexer_ref.indexer_score(q, pooled, 10, pos=21)          # blocks 0..5 start at or before 21
    assert np.isneginf(sc[6:]).all() and np.isfinite(sc[:6]).all()
    want = sum(max(float(q[h].astype(np.float64) @ pooled[3].astype(np.float64)), 0.0) for h in range(4)) / np.sqrt(128.0)
    assert abs(sc[3] - want) < 1e-12 and (sc[:6] >= 0).all()
    # the shipped shader masks on the block's LAST cell: block 5 (cells 20..23) is dead for a row at 21
    last = indexer_ref.indexer_score(q, pooled, 10, pos=21, mask="last")
    assert np.isneginf(last[5]) and np.array_equal(last[:5], sc[:5])
