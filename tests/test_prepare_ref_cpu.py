"""Known answers and invariants of the float64 restatement of the reference's RMSNorm / rotary code
(oracle/prepare_ref.py; the reference holds no golden vectors for these steps, so the restatement is checked
against what the formulas of crates/breccia-kernels/src/ops/cpu.rs:52-153 imply)."""
import numpy as np

from oracle import prepare_ref


def test_rmsnorm_known_answers():
    # a constant row normalises to gamma (up to eps); scaling the input does not change the result
    x = np.full((1, 256), 3.0, np.float32)
    g = np.linspace(0.5, 1.5, 256).astype(np.float32)
    y = prepare_ref.rmsnorm(x, 256, g, 1e-6)
    assert np.allclose(y[0], g, rtol=0, atol=1e-6)
    z = np.random.default_rng(1).standard_normal((5, 256)).astype(np.float32)
    a, b = prepare_ref.rmsnorm(z, 256, g, 0.0), prepare_ref.rmsnorm(7.0 * z, 256, g, 0.0)
    assert np.abs(a - b).max() <= 2e-6
    # definition, one row, by hand
    r = z[2].astype(np.float64)
    want = r / np.sqrt((r * r).mean() + 1e-6) * g
    assert np.abs(prepare_ref.rmsnorm(z[2:3], 256, g, 1e-6)[0] - want).max() <= 1e-6


def test_rope_table_and_pairing():
    t = prepare_ref.rope_table(1.0e6, 64, 128)
    assert t.shape == (128, 32, 2) and t.dtype == np.float32
    assert np.all(t[0, :, 0] == 1.0) and np.all(t[0, :, 1] == 0.0)          # position 0: no rotation
    assert np.isclose(t[5, 0, 0], np.cos(5.0)) and np.isclose(t[5, 0, 1], np.sin(5.0))   # pair 0 turns by pos radians
    assert np.isclose(t[7, 16, 0], np.cos(7.0 * 1.0e6 ** (-0.5)), atol=1e-7)
    x = np.random.default_rng(2).standard_normal((3, 256)).astype(np.float32)
    pos = np.array([0, 9, 500])                                                 # 500 is clamped to 127
    y = prepare_ref.rope_apply(x, 256, 64, t, pos)
    assert np.array_equal(y[0], x[0])                                           # identity at position 0
    assert np.array_equal(y[:, 64:], x[:, 64:])                                 # dims [n_rot, head_dim) pass through
    # NEOX pairing (j, j + 32): each pair keeps its length; the adjacent pairing would not
    for r in range(3):
        assert np.allclose(y[r, :32] ** 2 + y[r, 32:64] ** 2, x[r, :32] ** 2 + x[r, 32:64] ** 2, rtol=1e-5)
    assert np.array_equal(y[2], prepare_ref.rope_apply(x[2:3], 256, 64, t, np.array([127]))[0])
    # one pair by hand
    c, s = np.float64(t[9, 3, 0]), np.float64(t[9, 3, 1])
    assert np.isclose(y[1, 3], np.float32(x[1, 3] * c - x[1, 35] * s)) and np.isclose(y[1, 35], np.float32(x[1, 3] * s + x[1, 35] * c))


def test_prepare_order_and_shapes():
    rng = np.random.default_rng(3)
    T, n_head, n_kv, hd, stride = 4, 6, 2, 128, 256
    q_full = rng.standard_normal((T, n_head, stride)).astype(np.float32)
    k = rng.standard_normal((T, n_kv * hd)).astype(np.float32)
    v = rng.standard_normal((T, n_kv * hd)).astype(np.float32)
    g1, g2 = np.ones(hd, np.float32), np.full(hd, 2.0, np.float32)
    t = prepare_ref.rope_table(1.0e4, 32, 64)
    pos = np.array([3, 4, 5, 6])
    q, k2, v2 = prepare_ref.prepare(q_full, k, v, g1, g2, 1e-6, t, 32, pos, n_head, n_kv, hd, stride)
    assert q.shape == (T, n_head, hd) and k2.shape == (T, n_kv * hd) and np.array_equal(v2, v)
    # norm first, rotation second: the rotation keeps the normalised row's length (sqrt(hd) for gamma 1, twice for 2)
    assert np.allclose(np.linalg.norm(q, axis=-1), np.sqrt(hd), rtol=1e-4)
    assert np.allclose(np.linalg.norm(k2.reshape(T, n_kv, hd), axis=-1), 2 * np.sqrt(hd), rtol=1e-4)
    # the gate half of q_full is never read
    q_full[:, :, hd:] = np.nan
    q_again, _, _ = prepare_ref.prepare(q_full, k, v, g1, g2, 1e-6, t, 32, pos, n_head, n_kv, hd, stride)
    assert np.array_equal(q, q_again)
