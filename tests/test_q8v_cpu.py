"""The q8_0 V store / load rule of the oracle against the reference's own tests of cpu::to_q8_0
(crates/breccia-kernels/src/qsa/mod.rs:2072-2107) and its size pins (qsa/mod.rs:1983, 2046, 339-349)."""
import numpy as np

from oracle import q8v


def lcg_values(n: int) -> np.ndarray:
    """The input of the reference's test: a 64-bit LCG, top 24 bits, mapped to [-4, 4)."""
    s, out = 12345, np.empty(n, np.float32)
    for i in range(n):
        s = (s * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
        out[i] = (np.float32(s >> 40) / np.float32(1 << 24) - np.float32(0.5)) * np.float32(8.0)
    return out


def test_zeros_round_trip_exactly():
    zeros = np.zeros(64, np.float32)
    assert np.array_equal(q8v.to_q8_0(zeros), zeros)
    scale, q = q8v.quantize(zeros)
    assert np.array_equal(scale, np.ones(2, np.float32)) and not q.any()


def test_error_within_half_a_step_and_block_maximum_on_the_grid():
    x = lcg_values(256)
    q = q8v.to_q8_0(x)
    assert q.shape == x.shape
    for b in range(x.size // 32):
        xb, qb = x[32 * b: 32 * b + 32], q[32 * b: 32 * b + 32]
        amax = np.abs(xb).max()
        half_lsb = amax / np.float32(127.0) / np.float32(2.0)
        assert (np.abs(qb - xb) <= half_lsb * 1.001).all()
        assert abs(np.abs(qb).max() - amax) <= half_lsb * 1.001


def test_sizes():
    assert q8v.BLOCK_BYTES == 36 and q8v.BLOCK_ELEMS == 32
    assert q8v.row_bytes(256) == 288 and q8v.row_bytes(256) / (256 * 2) == 0.5625


def test_rounding_is_half_away_from_zero_and_clamped():
    # scale = 127 / 127 = 1: the values are their own quanta before rounding
    x = np.zeros(32, np.float32)
    x[:8] = [127.0, 0.5, -0.5, 1.5, -1.5, 2.5, 0.49999997, -126.5]
    scale, q = q8v.quantize(x)
    assert scale[0] == 1.0
    assert q[0, :8].tolist() == [127, 1, -1, 2, -2, 3, 0, -127]


def test_pool_bytes_layout_scale_word_first_then_quanta_lowest_byte_first():
    x = np.arange(-16, 16, dtype=np.float32)[None, :] * np.float32(0.25)
    raw = q8v.pack_rows(x)
    assert raw.shape == (1, 36)
    scale, q = q8v.quantize(x)
    assert raw[0, :4].tobytes() == np.float32(scale[0, 0]).tobytes()
    assert raw[0, 4:].view(np.int8).tolist() == q[0, 0].tolist()
    assert np.array_equal(q8v.unpack_rows(raw), q8v.to_q8_0(x))


def test_append_and_gather_through_a_page_table():
    n_kv, hd = 2, 64
    rng = np.random.default_rng(3)
    pool = np.zeros((5 * n_kv * 16, q8v.row_bytes(hd)), np.uint8)
    table = np.array([3, 0, 4], np.uint32)
    v = rng.standard_normal((40, n_kv * hd)).astype(np.float32)
    q8v.v_append(pool, table, v[:30], 0, n_kv, hd)
    q8v.v_append(pool, table, v[30:], 30, n_kv, hd)
    got = q8v.gather_v(pool, table, 40, n_kv, hd)
    assert np.array_equal(got, q8v.to_q8_0(v.reshape(40 * n_kv, hd)).reshape(40, n_kv * hd))
    assert not pool.reshape(5, -1)[[1, 2]].any()          # pages the table does not name stay untouched
