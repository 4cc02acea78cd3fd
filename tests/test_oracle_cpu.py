"""The CPU oracle against the reference's own known-answer tests, and against an independent
NumPy float64 restatement.  No GPU."""
import json
import os
import struct

import numpy as np
import pytest

import oracle
from oracle import numpy_ref

KATS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


def _f32(bits: int) -> float:
    return struct.unpack("<f", struct.pack("<I", bits))[0]


def test_to_f16_known_answers():
    L = oracle.lib()
    for x, want in KATS["to_f16"]["cases"]:
        assert L.brc_ref_to_f16(x) == np.float32(want), x
        assert L.brc_ref_f16_bits_to_f32(L.brc_ref_f32_to_f16_bits(x)) == np.float32(want), x
    for x, bits in KATS["to_f16"]["bits"]:
        assert L.brc_ref_f32_to_f16_bits(x) == int(bits, 16)
    for x in KATS["to_f16"]["infinite"]:
        assert np.isinf(L.brc_ref_to_f16(x))


def test_store_rule_is_round_to_nearest_even_not_truncation():
    L = oracle.lib()
    for src, want in KATS["store_bits"]["cases"]:
        assert L.brc_ref_f32_to_f16_bits(_f32(int(src, 16))) == int(want, 16)


def test_f16_edges():
    L = oracle.lib()
    enc = L.brc_ref_f32_to_f16_bits
    assert enc(65519.99) == 0x7BFF and enc(65520.0) == 0x7C00 and enc(-65520.0) == 0xFC00
    assert enc(float("nan")) & 0x7FFF == 0x7C00           # NaN stores as inf
    assert enc(2.0 ** -14) == 0x0400                       # smallest normal survives
    assert enc(_f32(0x387FFFFF)) == 0                      # just below: flushed BEFORE rounding
    assert enc(-(2.0 ** -15)) == 0x8000                    # signed zero
    assert L.brc_ref_f16_bits_to_f32(0x0001) == 0.0        # subnormal bits read as zero
    assert L.brc_ref_f16_bits_to_f32(0x8200) == 0.0
    assert np.isnan(L.brc_ref_f16_bits_to_f32(0x7E00))


def test_rust_and_glsl_statements_of_the_rule_agree():
    L = oracle.lib()
    # every 4093rd bit pattern over the whole f32 range, plus dense windows on the edges
    assert L.brc_ref_f16_rule_mismatches(0, 4093, (1 << 32) // 4093) == 0
    for first in (0x38000000, 0x387FF000, 0x477F0000, 0x7F7F0000, 0xB87FF000, 0xC77F0000):
        assert L.brc_ref_f16_rule_mismatches(first, 1, 1 << 17) == 0


def test_numpy_codec_equals_c_codec():
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 1 << 32, size=200000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    got = oracle.f32_to_f16_bits_np(x)
    want = oracle.f32_to_f16_bits(x[:20000])
    assert np.array_equal(got[:20000], want)
    back = oracle.f16_bits_to_f32(got[:20000])
    L = oracle.lib()
    for i in range(0, 20000, 97):
        w = L.brc_ref_f16_bits_to_f32(int(got[i]))
        assert (np.isnan(w) and np.isnan(back[i])) or w == back[i]


def test_pool_size_kats():
    L = oracle.lib()
    s = KATS["sizes"]
    assert L.brc_ref_page_bytes(2, 16, 256) == s["page_bytes"]
    assert L.brc_ref_f16_row_words(256) == s["f16_row_words"]
    assert L.brc_ref_q8v_row_words(256) == s["q8v_row_words"]
    for pages in s["pages"]:
        rows = L.brc_ref_pool_rows(pages, 2, 16)
        assert rows == pages * 2 * 16
        assert L.brc_ref_f16_pool_bytes(pages, 2, 16, 256) == rows * s["f16_row_words"] * 4
        assert L.brc_ref_q8v_pool_bytes(pages, 2, 16, 256) == rows * s["q8v_row_words"] * 4


def layout_kat_inputs(cell: int, dim: int):
    i = np.arange(dim, dtype=np.float32)
    k = np.sin((np.float32(cell * 97) + i * np.float32(13)) * np.float32(0.017)).astype(np.float32) * np.float32(3.0)
    v = np.cos((np.float32(cell * 61) + i * np.float32(7)) * np.float32(0.031)).astype(np.float32) * np.float32(2.0)
    return k, v


def test_layout_kat_cells_5_to_37():
    """The reference's `qsa_kv_cache_layout_and_f16_precision`: 33 single-token appends crossing a page
    boundary; every element's address and binary16 bits."""
    lay = KATS["layout"]
    nkv, hd = lay["n_kv_head"], lay["head_dim"]
    pages = (lay["cells"] + 15) // 16
    words = pages * nkv * 16 * hd // 2
    kp = np.zeros(words, np.uint32)
    vp = np.zeros(words, np.uint32)
    table = np.arange(pages, dtype=np.uint32)
    expect = {}
    for t in range(lay["n_tok"]):
        cell = lay["start"] + t
        k, v = layout_kat_inputs(cell, nkv * hd)
        expect[cell] = (k, v)
        assert oracle.kv_append(kp, vp, table, k, v, cell, nkv, hd) == 0
    k16, v16 = kp.view(np.uint16), vp.view(np.uint16)
    L = oracle.lib()
    checked = 0
    for cell, (k, v) in expect.items():
        for kvh in range(nkv):
            base = ((cell // 16 * nkv + kvh) * 16 + cell % 16) * hd
            assert base == L.brc_ref_elem_index(cell // 16, kvh, cell % 16, 0, nkv, 16, hd)
            want_k = oracle.f32_to_f16_bits_np(k[kvh * hd:(kvh + 1) * hd])
            want_v = oracle.f32_to_f16_bits_np(v[kvh * hd:(kvh + 1) * hd])
            assert np.array_equal(k16[base:base + hd], want_k)
            assert np.array_equal(v16[base:base + hd], want_v)
            checked += hd
    assert checked == lay["checked_elements"]
    # untouched cells stay zero
    assert not k16[:5 * 0 + 0].any()
    touched = np.zeros(k16.size, bool)
    for cell in expect:
        for kvh in range(nkv):
            base = ((cell // 16 * nkv + kvh) * 16 + cell % 16) * hd
            touched[base:base + hd] = True
    assert not k16[~touched].any() and not v16[~touched].any()


def test_append_refuses_past_capacity():
    kp = np.zeros(2 * 16 * 256 // 2, np.uint32)
    vp = np.zeros_like(kp)
    k = np.zeros(2 * 512, np.float32)
    before = kp.copy()
    assert oracle.kv_append(kp, vp, [0], k, k, 15, 2, 256, capacity_cells=16) == -1
    assert np.array_equal(kp, before)


def test_append_through_a_permuted_table_and_gather_back():
    rng = np.random.default_rng(7)
    nkv, hd, pages = 2, 256, 9
    table = rng.permutation(pages).astype(np.uint32)
    kp = np.zeros(pages * nkv * 16 * hd // 2, np.uint32)
    vp = np.zeros_like(kp)
    n = 130
    k = rng.standard_normal((n, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((n, nkv * hd)).astype(np.float32)
    assert oracle.kv_append(kp, vp, table, k[:100], v[:100], 0, nkv, hd) == 0
    assert oracle.kv_append(kp, vp, table, k[100:], v[100:], 100, nkv, hd) == 0
    kb, kf = oracle.gather(kp.view(np.uint16), table, n, nkv, hd)
    assert np.array_equal(kb.reshape(n, -1), oracle.f32_to_f16_bits_np(k))
    assert np.array_equal(kf.reshape(n, -1), oracle.to_f16(k))
    view = numpy_ref.paged_view(vp.view(np.uint16), table, n, nkv, hd)
    assert np.array_equal(view.reshape(n, -1), oracle.f32_to_f16_bits_np(v))


@pytest.mark.parametrize("n_head,n_kv,hd,cells", [(16, 2, 256, 300), (24, 2, 256, 77), (8, 8, 128, 33), (4, 1, 64, 5)])
def test_attend_equals_numpy_float64(n_head, n_kv, hd, cells):
    rng = np.random.default_rng(cells)
    q = rng.standard_normal((n_head, hd)).astype(np.float32)
    k = oracle.to_f16(rng.standard_normal((cells, n_kv, hd)).astype(np.float32) * 0.5)
    v = oracle.to_f16(rng.standard_normal((cells, n_kv, hd)).astype(np.float32) * 0.5)
    gate = rng.standard_normal((n_head, hd)).astype(np.float32)
    sel = np.arange(cells, dtype=np.uint32)
    pos = cells - 3  # the last two listed cells are in the future and must be skipped
    for g in (None, gate):
        a = oracle.attend(q, k, v, sel, pos, n_head, n_kv, hd, g)
        b = numpy_ref.attend(q, k, v, sel, pos, n_head, n_kv, hd, g)
        assert oracle.max_rel(a, b.astype(np.float64)) < 2e-7
    # no gate == gate of +1e4 (sigmoid is exactly 1 in f64)
    a = oracle.attend(q, k, v, sel, pos, n_head, n_kv, hd, None)
    b = oracle.attend(q, k, v, sel, pos, n_head, n_kv, hd, np.full((n_head, hd), 1e4, np.float32))
    assert np.array_equal(a, b)


def test_attend_sparse_cell_list_like_the_reference_q8_case():
    """ids [0, 5, 9, 15] of 4-cell blocks over 64 cells, LCG inputs 0xF1..0xF4
    (crates/breccia-kernels/tests/attn_conformance.rs:1354-1439), f16 V path."""
    n_head, n_kv, hd, cells = 24, 2, 256, 64
    k = oracle.to_f16(oracle.normalish(0xF1, cells * n_kv * hd))
    v = oracle.to_f16(oracle.normalish(0xF2, cells * n_kv * hd))
    q = oracle.normalish(0xF3, n_head * hd)
    q_full = oracle.normalish(0xF4, n_head * 2 * hd).reshape(n_head, 2, hd)
    gate = q_full[:, 1, :]
    sel = oracle.cells_of([0, 5, 9, 15], 4)
    assert sel.tolist() == [0, 1, 2, 3, 20, 21, 22, 23, 36, 37, 38, 39, 60, 61, 62, 63]
    a = oracle.attend(q, k, v, sel, cells - 1, n_head, n_kv, hd, gate)
    b = numpy_ref.attend(q, k, v, sel, cells - 1, n_head, n_kv, hd, gate)
    assert oracle.max_rel(a, b.astype(np.float64)) <= KATS["attention_bars"]["output_max_rel"]


def test_split_kv_partials_combine_to_the_unsplit_result():
    """CPU 'ranks' each hold a KV range; their (m, l, acc) partials merged by the LSE rule must equal
    attention over the whole range."""
    rng = np.random.default_rng(11)
    n_head, n_kv, hd, cells = 16, 2, 256, 1000
    q = rng.standard_normal((n_head, hd)).astype(np.float32)
    k = oracle.to_f16(rng.standard_normal((cells, n_kv, hd)).astype(np.float32) * 0.5)
    v = oracle.to_f16(rng.standard_normal((cells, n_kv, hd)).astype(np.float32) * 0.5)
    whole = oracle.attend(q, k, v, np.arange(cells, dtype=np.uint32), cells - 1, n_head, n_kv, hd)
    for cuts in ([0, 1000], [0, 250, 500, 750, 1000], [0, 16, 16, 999, 1000], [0, 0, 1000]):
        for h in (0, 7, 8, 15):
            kvh = h * n_kv // n_head
            parts = [oracle.partial_head(q[h], k, v, cuts[i], cuts[i + 1], kvh, n_kv, hd, 1 / 16.0)
                     for i in range(len(cuts) - 1)]
            out = oracle.lse_combine([p[0] for p in parts], [p[1] for p in parts], np.stack([p[2] for p in parts]))
            assert np.abs(out - whole[h]).max() < 1e-6


def test_decode_batch_equals_attend_per_sequence():
    rng = np.random.default_rng(5)
    n_head, n_kv, hd = 16, 2, 256
    lens = np.array([1, 16, 17, 100, 0], np.uint32)
    pages = 16
    table = rng.permutation(pages).astype(np.uint32)
    tables = np.zeros((lens.size, 7), np.uint32)
    at = 0
    for s, n in enumerate(lens):
        need = (int(n) + 15) // 16
        tables[s, :need] = table[at:at + need]
        at += need
    kp = oracle.f32_to_f16_bits_np(rng.standard_normal(pages * n_kv * 16 * hd).astype(np.float32) * 0.5)
    vp = oracle.f32_to_f16_bits_np(rng.standard_normal(pages * n_kv * 16 * hd).astype(np.float32) * 0.5)
    q = rng.standard_normal((lens.size, n_head, hd)).astype(np.float32)
    out, used = oracle.decode_batch(kp, vp, tables, lens, q, n_head, n_kv, hd)
    assert used >= 1
    for s, n in enumerate(lens):
        if n == 0:
            assert not out[s].any()
            continue
        _, kf = oracle.gather(kp, tables[s], int(n), n_kv, hd)
        _, vf = oracle.gather(vp, tables[s], int(n), n_kv, hd)
        want = oracle.attend(q[s], kf, vf, np.arange(n, dtype=np.uint32), int(n) - 1, n_head, n_kv, hd)
        assert np.array_equal(out[s], want)


def test_prefill_chunk_rows_are_causal():
    rng = np.random.default_rng(9)
    n_head, n_kv, hd = 16, 2, 128
    pos0, chunk, pages = 37, 5, 4
    table = rng.permutation(pages).astype(np.uint32)
    kp = oracle.f32_to_f16_bits_np(rng.standard_normal(pages * n_kv * 16 * hd).astype(np.float32))
    vp = oracle.f32_to_f16_bits_np(rng.standard_normal(pages * n_kv * 16 * hd).astype(np.float32))
    q = rng.standard_normal((chunk, n_head, hd)).astype(np.float32)
    out, _ = oracle.prefill_chunk(kp, vp, table, pos0, q, n_head, n_kv, hd)
    _, kf = oracle.gather(kp, table, pos0 + chunk, n_kv, hd)
    _, vf = oracle.gather(vp, table, pos0 + chunk, n_kv, hd)
    for t in range(chunk):
        want = oracle.attend(q[t], kf, vf, np.arange(pos0 + chunk, dtype=np.uint32), pos0 + t, n_head, n_kv, hd)
        assert np.array_equal(out[t], want)


def test_q8_0_round_trip_rule():
    L = oracle.lib()
    import ctypes as C
    x = np.concatenate([np.linspace(-3, 3, 32), np.zeros(32)]).astype(np.float32)
    out = np.empty_like(x)
    assert L.brc_ref_to_q8_0(x.ctypes.data_as(C.POINTER(C.c_float)), x.size, out.ctypes.data_as(C.POINTER(C.c_float))) == 0
    scale = np.float32(3.0) / np.float32(127.0)
    assert np.allclose(out[:32], np.round(x[:32] / scale) * scale, atol=1e-7)
    assert not out[32:].any()
    assert L.brc_ref_to_q8_0(x.ctypes.data_as(C.POINTER(C.c_float)), 33, out.ctypes.data_as(C.POINTER(C.c_float))) == -1


def test_page_copy_reference_is_a_byte_copy():
    rng = np.random.default_rng(2)
    layers, pages, half = 3, 6, 64
    k = rng.integers(0, 256, layers * pages * half, dtype=np.uint8)
    v = rng.integers(0, 256, layers * pages * half, dtype=np.uint8)
    k0, v0 = k.copy(), v.copy()
    oracle.page_copy(k, v, layers, pages, half, [1, 4], [0, 5])
    K, K0 = k.reshape(layers, pages, half), k0.reshape(layers, pages, half)
    assert np.array_equal(K[:, 0], K0[:, 1]) and np.array_equal(K[:, 5], K0[:, 4])
    assert np.array_equal(K[:, [1, 2, 3, 4]], K0[:, [1, 2, 3, 4]])
    V, V0 = v.reshape(layers, pages, half), v0.reshape(layers, pages, half)
    assert np.array_equal(V[:, 0], V0[:, 1]) and np.array_equal(V[:, 5], V0[:, 4])
