"""Paged decode attention on the GPU through the C ABI against the oracle.

Tolerance (target, fp32 accumulate over f16 KV): max-abs <= 2e-3, max-rel <= 1e-2.
The reference's own measure max|g-w|/max(|w|,1) (bar 1e-5 for its kernels) is asserted too."""
import ctypes as C
import hashlib
import os
import sys

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import DecodeBatch, KvPool, Qsa, QsaState, decode_combine, decode_partial_bytes
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32, fill_pool_from_host

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_cfg1_golden import CONTEXT, HD, N_HEAD, N_KV, POOL_PAGES, cfg1_inputs  # noqa: E402

pytestmark = pytest.mark.gpu

REF_MEASURE_BAR = 1e-5  # crates/breccia-kernels/tests/attn_conformance.rs:1148-1158


def assert_attention_close(got, want, what=""):
    max_abs, max_rel, ref = attention_errors(got, want)
    assert np.isfinite(np.asarray(got)).all(), f"{what}: non-finite output"
    assert max_abs <= ATTN_MAX_ABS, f"{what}: max-abs {max_abs:.3e} > {ATTN_MAX_ABS}"
    assert max_rel <= ATTN_MAX_REL, f"{what}: max-rel {max_rel:.3e} > {ATTN_MAX_REL}"
    assert ref <= REF_MEASURE_BAR, f"{what}: reference measure {ref:.3e} > {REF_MEASURE_BAR}"
    return max_abs, max_rel, ref


def test_cfg1_conformance_against_committed_golden(cuda_device):
    """The conformance configuration end to end through the mirror API: fill 1024 cells through kv_append in
    256-cell chunks, append one token, one decode step; cache pages bit-exact, output in tolerance."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "cfg1_golden.npz"))
    table, k_ctx, v_ctx, k_new, v_new, q = cfg1_inputs()
    pool = KvPool(0, 1, N_KV, HD, POOL_PAGES)
    qsa = Qsa(pool, N_HEAD)
    state = QsaState(pool, CONTEXT + 1, block_table=table)
    ws = qsa.workspace(256)
    for start in range(0, CONTEXT, 256):
        ws.k_cur.copy_(torch.from_numpy(k_ctx[start:start + 256]))
        ws.v_cur.copy_(torch.from_numpy(v_ctx[start:start + 256]))
        qsa.kv_append(state, ws, start)
    ws1 = qsa.workspace(1, q_dtype=DTYPE_F16)
    ws1.k_cur.copy_(torch.from_numpy(k_new))
    ws1.v_cur.copy_(torch.from_numpy(v_new))
    ws1.q.copy_(torch.from_numpy(q).view(1, N_HEAD, HD))
    qsa.kv_append(state, ws1, CONTEXT)
    qsa.topk_dense(ws1, CONTEXT)
    qsa.attend(state, ws1, CONTEXT)
    qsa.apply(state, ws1, CONTEXT)
    pool.check()
    kp, vp = pool.read(0, 0), pool.read(1, 0)
    assert hashlib.sha256(kp.tobytes()).digest() == bytes(g["k_pool_sha256"])
    assert hashlib.sha256(vp.tobytes()).digest() == bytes(g["v_pool_sha256"])
    assert np.array_equal(kp[table[64]], g["last_page_k"])
    out = ws1.attn_out.cpu().numpy()[0]
    errs = assert_attention_close(out, g["out"], "cfg1")
    print("cfg1 max_abs %.2e max_rel %.2e ref_measure %.2e" % errs)
    # f32 query path gives the same answer
    ws2 = qsa.workspace(1, q_dtype=DTYPE_F32)
    ws2.q.copy_(torch.from_numpy(q).view(1, N_HEAD, HD))
    qsa.topk_dense(ws2, CONTEXT)
    qsa.attend(state, ws2, CONTEXT)
    assert_attention_close(ws2.attn_out.cpu().numpy()[0], g["out"], "cfg1 f32 q")
    pool.release()


def _batch_case(n_head, n_kv, hd, lens, seed, n_layers=1, layer=0, gate=False, q_dtype=DTYPE_F16, poison=False):
    lens = np.asarray(lens, np.int64)
    tables, n_pool = synth.scattered_tables(seed, np.maximum(lens, 1), pool_factor=1.3)
    pool = KvPool(0, n_layers, n_kv, hd, n_pool)
    if poison:
        pool.poison_nan()
    k, v = fill_pool_from_host(pool, layer, seed + 10)
    if poison:
        # everything the sequences do not own, and the tail of every last page, is NaN
        k = k.reshape(n_pool, n_kv, 16, hd).copy()
        v = v.reshape(n_pool, n_kv, 16, hd).copy()
        live = np.zeros((n_pool, 16), bool)
        for s, n in enumerate(lens):
            for c in range(int(n)):
                live[tables[s, c // 16], c % 16] = True
        dead = np.broadcast_to(~live[:, None, :, None], k.shape)
        k[dead] = 0xFFFF
        v[dead] = 0xFFFF
        pool.write(0, layer, k)
        pool.write(1, layer, v)
        k, v = k.reshape(-1), v.reshape(-1)
    q32 = synth.normal(seed + 20, lens.size * n_head * hd, 1.0).reshape(lens.size, n_head, hd)
    if q_dtype == DTYPE_F16:
        q32 = oracle.to_f16(q32)
    g = synth.normal(seed + 30, lens.size * n_head * 2 * hd, 1.0).reshape(lens.size, n_head, 2, hd) if gate else None
    batch = DecodeBatch(pool, n_head, tables, lens, q_dtype=q_dtype)
    qd = torch.from_numpy(q32).cuda()
    if q_dtype == DTYPE_F16:
        qd = qd.half()
    out = torch.full((lens.size, n_head, hd), float("nan"), device="cuda")
    gd = torch.from_numpy(g).cuda() if gate else None
    batch.attend(layer, qd, out, gate=gd.view(-1)[hd:] if gate else None, gate_head_stride=2 * hd if gate else 0)
    pool.check()
    want, _ = oracle.decode_batch(k, v, tables, lens, q32, n_head, n_kv, hd, gate=g[:, :, 1, :] if gate else None)
    return pool, batch, qd, out.cpu().numpy(), want


@pytest.mark.parametrize("lens", [[1], [15], [16], [17], [1025], [4097, 3, 160, 16, 1, 2049, 31, 700]])
def test_ragged_lengths_and_page_edges(cuda_device, lens):
    pool, _, _, got, want = _batch_case(16, 2, 256, lens, seed=40 + len(lens))
    assert_attention_close(got, want, f"lens {lens}")
    pool.release()


def test_reference_fixture_2062_cells_24_heads_lcg_streams_with_gate(cuda_device):
    """The reference's own attention fixture (crates/breccia-kernels/tests/attn_conformance.rs:897-1037): its
    LCG `normalish` streams 0xE3 (K) / 0xE4 (V) for 2062 cells x 2 kv heads x 256, appended in 256-cell chunks
    as the test does, one f32 query 0xE5 of 24 heads at the last cell, the gate read in place from the second
    half of each head's 512-wide block of stream 0xE6.  Here over ALL cells (the dense selection); expected
    values = the oracle's f64 attend over the binary16-rounded K/V, bars as the reference's (1e-5 on its
    measure).  The cache must hold the reference store rule's bits."""
    n_head, n_kv, hd, cells = 24, 2, 256, 2062
    k_all = oracle.normalish(0xE3, cells * n_kv * hd).reshape(cells, n_kv * hd)
    v_all = oracle.normalish(0xE4, cells * n_kv * hd).reshape(cells, n_kv * hd)
    q = oracle.normalish(0xE5, n_head * hd).reshape(1, n_head, hd)
    q_full = oracle.normalish(0xE6, n_head * 2 * hd).reshape(1, n_head, 2, hd)
    pool = KvPool(0, 1, n_kv, hd, 4096 // 16)
    qsa = Qsa(pool, n_head)
    state = QsaState(pool, cells)                      # identity-like table from the allocator
    for start in range(0, cells, 256):
        n = min(256, cells - start)
        ws = qsa.workspace(n)
        ws.k_cur.copy_(torch.from_numpy(k_all[start:start + n]))
        ws.v_cur.copy_(torch.from_numpy(v_all[start:start + n]))
        qsa.kv_append(state, ws, start)
    ws1 = qsa.workspace(1, q_dtype=DTYPE_F32)
    ws1.q.copy_(torch.from_numpy(q))
    ws1.q_full = torch.from_numpy(q_full).cuda().reshape(1, n_head * 2 * hd)
    qsa.topk_dense(ws1, cells - 1)
    qsa.attend(state, ws1, cells - 1)
    qsa.apply(state, ws1, cells - 1)
    pool.check()
    kg, vg = pool.gather(0, state.page_table_dev, cells)
    assert np.array_equal(kg.view(torch.int16).cpu().numpy().view(np.uint16).reshape(cells, -1), oracle.f32_to_f16_bits_np(k_all))
    assert np.array_equal(vg.view(torch.int16).cpu().numpy().view(np.uint16).reshape(cells, -1), oracle.f32_to_f16_bits_np(v_all))
    want = oracle.attend(q[0], oracle.to_f16(k_all), oracle.to_f16(v_all), np.arange(cells, dtype=np.uint32), cells - 1,
                         n_head, n_kv, hd, gate=q_full[0, :, 1, :])
    errs = assert_attention_close(ws1.attn_out.cpu().numpy()[0], want, "reference fixture, 2062 cells")
    print("reference fixture 2062 cells / 24 heads: max_abs %.2e max_rel %.2e ref_measure %.2e" % errs)
    state.release()
    pool.release()


@pytest.mark.parametrize("n_head,n_kv,hd", [(16, 2, 256), (8, 2, 256), (4, 4, 256), (32, 4, 128), (6, 2, 128), (8, 1, 256), (12, 3, 128),
                                            (24, 2, 256),    # the reference model's heads: 12 per kv head, two passes of 8 + 4
                                            (20, 1, 128)])   # 20 per kv head: three passes, one kv head per unit
def test_geometries(cuda_device, n_head, n_kv, hd):
    pool, _, _, got, want = _batch_case(n_head, n_kv, hd, [333, 48, 1000], seed=60 + n_head, n_layers=2, layer=1)
    assert_attention_close(got, want, f"{n_head}q/{n_kv}kv hd{hd}")
    pool.release()


def test_cfg2_layer_at_full_size_matches_oracle_and_repeats_bit_identically(cuda_device):
    """One layer of the batched-decode workload at full size (32 sequences, lengths uniform in [512, 8192],
    pages scattered in a pool of 1.25x need: every CTA streams dozens of pages through its ring and
    crosses several sequence boundaries).  Output in tolerance against the oracle, and ten
    back-to-back launches give bit-identical results."""
    n_head, n_kv, hd = 16, 2, 256
    lens = synth.uniform_ints(20261125, 32, 512, 8192)
    tables, n_pool = synth.scattered_tables(20261125 + 7, lens, pool_factor=1.25)
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    rng = np.random.default_rng(5)
    n = n_pool * n_kv * 16 * hd
    k = np.empty(n, np.uint16)
    v = np.empty(n, np.uint16)
    for at in range(0, n, 1 << 22):
        m = min(1 << 22, n - at)
        k[at:at + m] = oracle.f32_to_f16_bits_np(rng.standard_normal(m, dtype=np.float32) * np.float32(0.5))
        v[at:at + m] = oracle.f32_to_f16_bits_np(rng.standard_normal(m, dtype=np.float32) * np.float32(0.5))
    pool.write(0, 0, k)
    pool.write(1, 0, v)
    q32 = oracle.to_f16(synth.normal(77, lens.size * n_head * hd, 1.0)).reshape(lens.size, n_head, hd)
    qd = torch.from_numpy(q32).cuda().half()
    batch = DecodeBatch(pool, n_head, tables, lens)
    outs = [torch.full((lens.size, n_head, hd), float("nan"), device="cuda") for _ in range(10)]
    for o in outs:
        batch.attend(0, qd, o)
    pool.check()
    want, _ = oracle.decode_batch(k, v, tables, lens, q32, n_head, n_kv, hd)
    got = outs[0].cpu().numpy()
    errs = assert_attention_close(got, want, "cfg2 layer")
    print("cfg2 layer max_abs %.2e max_rel %.2e ref_measure %.2e" % errs)
    for o in outs[1:]:
        assert np.array_equal(o.cpu().numpy(), got)
    pool.release()


@pytest.mark.parametrize("kv_f16", [False, True])
def test_decode_step_appends_bit_exactly_and_attends(cuda_device, kv_f16):
    """brc_decode_step over three layers, three steps in a row: positions advance on the device, the
    new cell of every sequence is written by the attention kernel itself (fused append) — the pool
    must equal the oracle's append bit for bit — and the outputs must match the oracle's attention.
    Lengths include a sequence whose new cell opens a fresh page and a sequence of length 0."""
    n_head, n_kv, hd, n_layers = 16, 2, 256, 3
    lens = np.array([16, 5, 1023, 0, 300, 31])
    tables, n_pool = synth.scattered_tables(55, lens, pool_factor=1.4, extra_tokens=4)
    pool = KvPool(0, n_layers, n_kv, hd, n_pool)
    host = []
    for layer in range(n_layers):
        k, v = fill_pool_from_host(pool, layer, 500 + 2 * layer)
        host.append([k.view(np.uint32).copy(), v.view(np.uint32).copy()])
    batch = DecodeBatch(pool, n_head, tables, lens)
    cur = lens.copy()
    for step in range(3):
        q32 = oracle.to_f16(synth.normal(600 + step, n_layers * lens.size * n_head * hd)).reshape(n_layers, lens.size, n_head, hd)
        kn = synth.normal(700 + step, n_layers * lens.size * n_kv * hd, 0.5).reshape(n_layers, lens.size, n_kv * hd)
        vn = synth.normal(800 + step, n_layers * lens.size * n_kv * hd, 0.5).reshape(n_layers, lens.size, n_kv * hd)
        if kv_f16:
            kn, vn = oracle.to_f16(kn), oracle.to_f16(vn)
            kd, vd = torch.from_numpy(kn).cuda().half(), torch.from_numpy(vn).cuda().half()
        else:
            kd, vd = torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda()
        out = torch.full((n_layers, lens.size, n_head, hd), float("nan"), device="cuda")
        batch.step(torch.from_numpy(q32).cuda().half(), kd, vd, out, kv_dtype=_lib.DTYPE_F16 if kv_f16 else DTYPE_F32)
        pool.check()
        got = out.cpu().numpy()
        for layer in range(n_layers):
            kw, vw = host[layer]
            for s in range(lens.size):
                assert oracle.kv_append(kw, vw, tables[s], kn[layer, s], vn[layer, s], int(cur[s]), n_kv, hd) == 0
            assert np.array_equal(pool.read(0, layer).reshape(-1), kw.view(np.uint16)), f"K pool, layer {layer}, step {step}"
            assert np.array_equal(pool.read(1, layer).reshape(-1), vw.view(np.uint16)), f"V pool, layer {layer}, step {step}"
            want, _ = oracle.decode_batch(kw.view(np.uint16), vw.view(np.uint16), tables, cur + 1, q32[layer], n_head, n_kv, hd)
            assert_attention_close(got[layer], want, f"step {step} layer {layer}")
        cur += 1
    assert batch.seq_lens.cpu().numpy().tolist() == cur.tolist()
    pool.release()


@pytest.mark.parametrize("parts,pinned_out,download,upload", [(1, True, False, True), (2, True, False, True), (5, True, False, True),
                                                              (1, False, False, True), (3, False, False, True), (1, True, True, True),
                                                              (3, True, True, True), (1, True, False, False), (3, True, False, False),
                                                              (1, False, False, False), (1, True, True, False)])
def test_step_from_host_buffers_in_parts_equals_the_device_step(cuda_device, parts, pinned_out, download, upload):
    """brc_decode_step_host (pinned host q / k / v either read in place by the kernels or uploaded, output
    back to the host, layers in `parts` groups with uploads and downloads on streams of their own; with
    everything in place no staging buffer is given at all) against brc_decode_step on a twin pool: outputs,
    both pools and the advanced lengths must be bit-identical, two steps in a row (the outputs bit-identical
    for one group, within 2e-6 when the layers go in several launches, whose shares are cut differently).  A pinned output buffer
    is written by the kernels directly unless the caller asks for the download; a pageable one is downloaded
    group by group."""
    n_head, n_kv, hd, n_layers = 16, 2, 256, 5
    lens = np.array([16, 5, 700, 0, 31, 255])
    tables, n_pool = synth.scattered_tables(56, lens, pool_factor=1.4, extra_tokens=4)
    pools = [KvPool(0, n_layers, n_kv, hd, n_pool) for _ in range(2)]
    for pool in pools:
        for layer in range(n_layers):
            fill_pool_from_host(pool, layer, 520 + 2 * layer)
    dev_batch, host_batch = DecodeBatch(pools[0], n_head, tables, lens), DecodeBatch(pools[1], n_head, tables, lens)
    shape_q, shape_kv = (n_layers, lens.size, n_head, hd), (n_layers, lens.size, n_kv * hd)
    staging = host_batch.host_staging(n_layers)
    out_h = torch.empty(shape_q).pin_memory() if pinned_out else torch.empty(shape_q)
    for step in range(2):
        q_h = torch.from_numpy(oracle.to_f16(synth.normal(610 + step, int(np.prod(shape_q)))).reshape(shape_q)).half().pin_memory()
        k_h = torch.from_numpy(synth.normal(710 + step, int(np.prod(shape_kv)), 0.5).reshape(shape_kv)).pin_memory()
        v_h = torch.from_numpy(synth.normal(810 + step, int(np.prod(shape_kv)), 0.5).reshape(shape_kv)).pin_memory()
        want = torch.full(shape_q, float("nan"), device="cuda")
        dev_batch.step(q_h.cuda(), k_h.cuda(), v_h.cuda(), want)
        out_h.fill_(float("nan"))
        in_place = pinned_out and not download and not upload
        host_batch.step_host(q_h, k_h, v_h, out_h, None if in_place else staging, parts=parts, download=download, upload=upload)
        for pool in pools:
            pool.check()
        if parts == 1 or not upload:   # inputs in place: one launch whatever `parts` says
            assert torch.equal(out_h, want.cpu()), f"step {step}"
        else:   # groups of layers are cut into shares of their own: same sums, another order
            assert float((out_h - want.cpu()).abs().max()) <= 2e-6, f"step {step}"
        for layer in range(n_layers):
            for which in (0, 1):
                assert np.array_equal(pools[0].read(which, layer), pools[1].read(which, layer)), f"pool {which} layer {layer}"
    assert torch.equal(dev_batch.seq_lens, host_batch.seq_lens)
    assert host_batch.seq_lens_host.tolist() == (lens + 2).tolist()
    for pool in pools:
        pool.release()


def test_step_in_two_parts_on_one_stream_equals_the_whole_step(cuda_device):
    """brc_decode_step_part twice (layers 0-1, then 2-4) against brc_decode_step on a twin pool; a part
    that reaches past the step's layers is refused."""
    n_head, n_kv, hd, n_layers = 16, 2, 256, 5
    lens = np.array([40, 3, 333, 0])
    tables, n_pool = synth.scattered_tables(57, lens, pool_factor=1.4, extra_tokens=4)
    pools = [KvPool(0, n_layers, n_kv, hd, n_pool) for _ in range(2)]
    for pool in pools:
        for layer in range(n_layers):
            fill_pool_from_host(pool, layer, 540 + 2 * layer)
    whole, split = DecodeBatch(pools[0], n_head, tables, lens), DecodeBatch(pools[1], n_head, tables, lens)
    q = torch.from_numpy(oracle.to_f16(synth.normal(620, n_layers * lens.size * n_head * hd))).cuda().half().reshape(n_layers, lens.size, n_head, hd)
    kn = torch.from_numpy(synth.normal(720, n_layers * lens.size * n_kv * hd, 0.5)).cuda().reshape(n_layers, lens.size, n_kv * hd)
    vn = torch.from_numpy(synth.normal(820, n_layers * lens.size * n_kv * hd, 0.5)).cuda().reshape(n_layers, lens.size, n_kv * hd)
    want, got = torch.full(q.shape, float("nan"), device="cuda"), torch.full(q.shape, float("nan"), device="cuda")
    whole.step(q, kn, vn, want)
    split.step_part(0, 2, q, kn, vn, got)
    split.step_part(2, 3, q, kn, vn, got)
    for pool in pools:
        pool.check()
    assert float((got - want).abs().max()) <= 2e-6   # two launches cut their shares differently: same sums, another order
    assert torch.equal(whole.seq_lens, split.seq_lens)
    for layer in range(n_layers):
        assert np.array_equal(pools[0].read(0, layer), pools[1].read(0, layer))
    with pytest.raises(_lib.BrcError) as err:
        split.step_part(3, 3, q, kn, vn, got)
    assert err.value.code == _lib.ERR_INVALID
    for pool in pools:
        pool.release()


def test_twelve_layers_in_one_launch_short_and_skewed_sequences_four_steps(cuda_device):
    """One launch per step over twelve layers (the flat list runs over layer, unit, page): sequences of 1, 2
    and 0 cells beside one of 5000, so most CTAs hold a stretch of one layer and many units lie whole inside
    a share while others span several.  Four steps back to back without a host wait in between, then every
    layer of every step against the oracle and the pool bit for bit."""
    n_head, n_kv, hd, n_layers, n_steps = 16, 2, 256, 12, 4
    lens = np.array([1, 2, 700, 0, 17, 16, 3, 5000])
    tables, n_pool = synth.scattered_tables(58, lens, pool_factor=1.3, extra_tokens=n_steps + 1)
    pool = KvPool(0, n_layers, n_kv, hd, n_pool)
    host = []
    for layer in range(n_layers):
        k, v = fill_pool_from_host(pool, layer, 900 + 2 * layer)
        host.append([k.view(np.uint32).copy(), v.view(np.uint32).copy()])
    batch = DecodeBatch(pool, n_head, tables, lens)
    qs, kns, vns, outs = [], [], [], []
    for step in range(n_steps):
        qs.append(oracle.to_f16(synth.normal(930 + step, n_layers * lens.size * n_head * hd)).reshape(n_layers, lens.size, n_head, hd))
        kns.append(synth.normal(940 + step, n_layers * lens.size * n_kv * hd, 0.5).reshape(n_layers, lens.size, n_kv * hd))
        vns.append(synth.normal(950 + step, n_layers * lens.size * n_kv * hd, 0.5).reshape(n_layers, lens.size, n_kv * hd))
        outs.append(torch.full((n_layers, lens.size, n_head, hd), float("nan"), device="cuda"))
    dev = [(torch.from_numpy(q).cuda().half(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()) for q, k, v in zip(qs, kns, vns)]
    for step in range(n_steps):
        batch.step(dev[step][0], dev[step][1], dev[step][2], outs[step])
    pool.check()
    cur = lens.copy()
    for step in range(n_steps):
        got = outs[step].cpu().numpy()
        for layer in range(n_layers):
            kw, vw = host[layer]
            for s in range(lens.size):
                assert oracle.kv_append(kw, vw, tables[s], kns[step][layer, s], vns[step][layer, s], int(cur[s]), n_kv, hd) == 0
            want, _ = oracle.decode_batch(kw.view(np.uint16), vw.view(np.uint16), tables, cur + 1, qs[step][layer], n_head, n_kv, hd)
            assert_attention_close(got[layer], want, f"step {step} layer {layer}")
        cur += 1
    for layer in range(n_layers):
        assert np.array_equal(pool.read(0, layer).reshape(-1), host[layer][0].view(np.uint16)), f"K pool, layer {layer}"
        assert np.array_equal(pool.read(1, layer).reshape(-1), host[layer][1].view(np.uint16)), f"V pool, layer {layer}"
    pool.release()


def test_fused_append_skips_a_sequence_beyond_the_callers_bound(cuda_device):
    """A step whose bound is below one sequence's new length: that sequence is reported (brc_pool_check),
    attended up to the bound, and NOTHING is appended for it - the last cell under the bound keeps its
    bytes - while the other sequence's cell is appended as usual."""
    n_head, n_kv, hd = 16, 2, 256
    lens = np.array([40, 20])
    tables, n_pool = synth.scattered_tables(59, lens, pool_factor=1.5, extra_tokens=8)
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    k, v = fill_pool_from_host(pool, 0, 960)
    kw, vw = k.view(np.uint32).copy(), v.view(np.uint32).copy()
    batch = DecodeBatch(pool, n_head, tables, lens)
    q = torch.from_numpy(oracle.to_f16(synth.normal(961, lens.size * n_head * hd))).cuda().half().reshape(1, lens.size, n_head, hd)
    kn = synth.normal(962, lens.size * n_kv * hd, 0.5).reshape(1, lens.size, n_kv * hd)
    vn = synth.normal(963, lens.size * n_kv * hd, 0.5).reshape(1, lens.size, n_kv * hd)
    kd, vd = torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda()
    out = torch.zeros((1, lens.size, n_head, hd), device="cuda")
    bound = 30   # sequence 0 would reach 41 cells
    _lib.call("brc_decode_step", pool.handle, 0, 1, C.c_void_p(batch.block_tables.data_ptr()), batch.table_stride,
              C.c_void_p(batch.seq_lens.data_ptr()), C.c_void_p(batch.pos0.data_ptr()), lens.size, bound,
              C.c_void_p(q.data_ptr()), DTYPE_F16, 0, n_head, C.c_void_p(kd.data_ptr()), C.c_void_p(vd.data_ptr()), DTYPE_F32, 0,
              None, 0, 0, 0.0625, C.c_void_p(out.data_ptr()), 0, C.c_void_p(batch.scratch.data_ptr()), batch.scratch.numel(), None)
    with pytest.raises(_lib.BrcError):
        pool.check()
    assert oracle.kv_append(kw, vw, tables[1], kn[0, 1], vn[0, 1], 20, n_kv, hd) == 0   # only sequence 1 appends
    assert np.array_equal(pool.read(0, 0).reshape(-1), kw.view(np.uint16))
    assert np.array_equal(pool.read(1, 0).reshape(-1), vw.view(np.uint16))
    pool.release()


def test_nan_poison_outside_live_cells_never_reaches_the_output(cuda_device):
    """Unowned pages and the cells past each sequence end hold NaN (the reference's poison flag,
    qsa/mod.rs:509-523): the output must equal the oracle's, which never looks there."""
    pool, _, _, got, want = _batch_case(16, 2, 256, [5, 100, 1, 511, 16], seed=77, poison=True)
    assert_attention_close(got, want, "poisoned pool")
    pool.release()


def test_empty_sequence_yields_zeros_and_empty_batch_is_a_no_op(cuda_device):
    pool, batch, qd, got, want = _batch_case(16, 2, 256, [0, 40, 0], seed=81)
    assert not got[0].any() and not got[2].any()
    assert_attention_close(got, want, "with empty sequences")
    L = _lib.load()
    assert L.brc_paged_decode_attn(pool.handle, 0, C.c_void_p(qd.data_ptr()), DTYPE_F16, 16, None, 0,
                                   C.c_void_p(batch.block_tables.data_ptr()), batch.table_stride,
                                   C.c_void_p(batch.seq_lens.data_ptr()), 0, 0, 0.0625, C.c_void_p(qd.data_ptr()),
                                   None, 0, None) == 0
    pool.release()


def test_block_table_permutation_invariance(cuda_device):
    """The same logical cache under two different physical placements gives bit-identical output."""
    n_head, n_kv, hd, n = 16, 2, 256, 777
    n_pages = (n + 15) // 16
    k = synth.normal(5, n_pages * 16 * n_kv * hd, 0.5).reshape(n_pages, 16, n_kv, hd)
    v = synth.normal(6, n_pages * 16 * n_kv * hd, 0.5).reshape(n_pages, 16, n_kv, hd)
    q = torch.from_numpy(oracle.to_f16(synth.normal(7, n_head * hd))).cuda().half().view(1, n_head, hd)
    outs = []
    for seed in (1, 2):
        pool = KvPool(0, 1, n_kv, hd, 3 * n_pages)
        table = synth.permutation(seed, 3 * n_pages)[:n_pages]
        kp = np.zeros((3 * n_pages, n_kv, 16, hd), np.uint16)
        vp = np.zeros_like(kp)
        kp[table] = oracle.f32_to_f16_bits_np(k).transpose(0, 2, 1, 3)
        vp[table] = oracle.f32_to_f16_bits_np(v).transpose(0, 2, 1, 3)
        pool.write(0, 0, kp)
        pool.write(1, 0, vp)
        batch = DecodeBatch(pool, n_head, table[None, :], [n])
        out = torch.empty((1, n_head, hd), device="cuda")
        batch.attend(0, q, out)
        pool.check()
        outs.append(out.cpu().numpy())
        pool.release()
    assert np.array_equal(outs[0], outs[1])


def test_chunking_does_not_change_the_answer(cuda_device):
    """Rows of a multi-row call are causal (row t sees cells <= pos0 + t) and equal the same rows
    computed one at a time — the reference's T = 1 / 8 / 32 agreement test
    (crates/breccia-kernels/tests/attn_conformance.rs:769-776)."""
    n_head, n_kv, hd, pos0, T = 16, 2, 256, 100, 8
    pool = KvPool(0, 1, n_kv, hd, 16)
    qsa = Qsa(pool, n_head)
    state = QsaState(pool, pos0 + T)
    k = synth.normal(1, (pos0 + T) * n_kv * hd, 0.5).reshape(pos0 + T, -1)
    v = synth.normal(2, (pos0 + T) * n_kv * hd, 0.5).reshape(pos0 + T, -1)
    wsf = qsa.workspace(pos0 + T)
    wsf.k_cur.copy_(torch.from_numpy(k))
    wsf.v_cur.copy_(torch.from_numpy(v))
    qsa.kv_append(state, wsf, 0)
    q = synth.normal(3, T * n_head * hd).reshape(T, n_head, hd)
    ws = qsa.workspace(T)
    ws.q.copy_(torch.from_numpy(q))
    qsa.topk_dense(ws, pos0)
    qsa.attend(state, ws, pos0)
    many = ws.attn_out.cpu().numpy()
    kf, vf = oracle.to_f16(k).reshape(pos0 + T, n_kv, hd), oracle.to_f16(v).reshape(pos0 + T, n_kv, hd)
    ws1 = qsa.workspace(1)
    for t in range(T):
        ws1.q.copy_(torch.from_numpy(q[t:t + 1]))
        qsa.topk_dense(ws1, pos0 + t)
        qsa.attend(state, ws1, pos0 + t)
        one = ws1.attn_out.cpu().numpy()[0]
        want = oracle.attend(q[t], kf, vf, np.arange(pos0 + T, dtype=np.uint32), pos0 + t, n_head, n_kv, hd)
        assert_attention_close(many[t], want, f"row {t}")
        assert np.abs(one - many[t]).max() <= 2e-6
    pool.check()
    pool.release()


def test_partials_then_combine_equals_fused_call(cuda_device):
    """brc_decode_partial over two halves of the KV range + brc_decode_combine == one fused call
    (the split-KV-across-GPUs path, exercised on one device)."""
    n_head, n_kv, hd = 16, 2, 256
    lens = np.array([2048, 640])
    pool, batch, qd, fused, want = _batch_case(n_head, n_kv, hd, lens, seed=91)
    nbytes = decode_partial_bytes(lens.size, n_head, hd)
    assert nbytes == lens.size * 16512
    parts = torch.zeros(2 * nbytes, dtype=torch.uint8, device="cuda")
    half = lens // 2 // 16 * 16
    tables = batch.block_tables.cpu().numpy().astype(np.uint32)
    lo = DecodeBatch(pool, n_head, tables, half)
    hi_tables = np.zeros_like(tables)
    for s in range(lens.size):
        n = (lens[s] - half[s] + 15) // 16
        hi_tables[s, :n] = tables[s, half[s] // 16: half[s] // 16 + n]
    hi = DecodeBatch(pool, n_head, hi_tables, lens - half)
    lo.partial(0, qd, parts[:nbytes])
    hi.partial(0, qd, parts[nbytes:])
    out = torch.empty((lens.size, n_head, hd), device="cuda")
    decode_combine(0, parts, 2, nbytes, lens.size, n_head, hd, out)
    pool.check()
    assert_attention_close(out.cpu().numpy(), want, "partials + combine")
    assert np.abs(out.cpu().numpy() - fused).max() <= 2e-6
    # (m, l, acc) of one head against the oracle's partial
    acc = parts[:nbytes].view(torch.float32)[: lens.size * n_head * hd].view(lens.size, n_head, hd).cpu().numpy()
    ml = parts[:nbytes].view(torch.float32)[lens.size * n_head * hd:].view(lens.size, n_head, 2).cpu().numpy()
    kpool, vpool = pool.read(0, 0).reshape(-1), pool.read(1, 0).reshape(-1)
    _, kf = oracle.gather(kpool, tables[1], int(half[1]), n_kv, hd)
    _, vf = oracle.gather(vpool, tables[1], int(half[1]), n_kv, hd)
    q1 = qd[1].float().cpu().numpy()
    m, l, a = oracle.partial_head(q1[9], kf, vf, 0, int(half[1]), 1, n_kv, hd, 1 / 16.0)
    assert abs(ml[1, 9, 0] - m) < 1e-4 and abs(ml[1, 9, 1] - l) / l < 1e-5
    assert np.abs(acc[1, 9] - a).max() < 1e-4 * max(1.0, np.abs(a).max())
    pool.release()


@pytest.mark.parametrize("n_head,n_kv,lens", [
    (16, 2, [24000]),            # one unit over every CTA: 148 pieces, a handful of (row, column) items per CTA
    (16, 2, [9000, 12000]),      # two units of ~60 and ~85 shares; they meet inside one CTA
    (8, 1, [13000, 40, 9000]),   # one kv head per unit (a 16-row box), a short unit in between
    (32, 4, [30000]),            # two units per sequence (4 kv heads), head_dim 128
])
def test_units_spanning_many_ctas(cuda_device, n_head, n_kv, lens):
    """Long sequences alone on the GPU: every unit spans dozens of CTA shares, each of which takes a few of the
    unit's (row, column) items in the merge, several threads per item.  Final output and the partial (acc, m, l)
    form, twice over, so that the ticket words (never cleared, 2^16 more per launch) are seen to work again."""
    hd = 128 if n_head == 32 else 256
    pool, batch, qd, got, want = _batch_case(n_head, n_kv, hd, lens, seed=120 + len(lens) + n_kv)
    assert_attention_close(got, want, f"units over many CTAs {lens}")
    again = torch.full_like(torch.from_numpy(got), float("nan")).cuda()
    batch.attend(0, qd, again)
    assert np.array_equal(again.cpu().numpy(), got), "second launch differs"
    n = len(lens)
    nbytes = decode_partial_bytes(n, n_head, hd)
    part = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    batch.partial(0, qd, part)
    out = torch.empty((n, n_head, hd), device="cuda")
    decode_combine(0, part, 1, nbytes, n, n_head, hd, out)
    pool.check()
    assert_attention_close(out.cpu().numpy(), want, f"units over many CTAs, partial form {lens}")
    pool.release()


@pytest.mark.parametrize("name,lens,n_kv", [
    # the per-unit surcharge of the cut dominates the pages: most thresholds fall into a surcharge and snap to a unit's start
    ("400 one-page sequences", [1 + i % 16 for i in range(400)], 2),
    # runs of sequences without cells between the others, at the start and at the end of the batch
    ("empty runs", [0, 0, 0, 700, 0, 33, 0, 0, 0, 0, 5000, 0, 17, 0, 0], 2),
    # fewer page-units than CTAs: shares in between are empty, the unit's pieces are counted from the table
    ("nine pages", [40, 0, 64, 33], 2),
    ("one unit of three pages among four kv heads", [0, 48], 4),
    # one long unit beside many short ones: the long one spans most CTAs, the short ones share a CTA
    ("one long, sixty short", [40000] + [20 + i for i in range(60)], 2),
])
def test_cost_weighted_cut_of_the_page_list(cuda_device, name, lens, n_kv):
    pool, _, _, got, want = _batch_case(16 if n_kv == 2 else 8, n_kv, 256, lens, seed=131 + len(lens))
    assert_attention_close(got, want, name)
    for s, n in enumerate(lens):
        if n == 0:
            assert not got[s].any(), f"{name}: sequence {s} has no cells, its rows must be zero"
    pool.release()


def test_shares_in_proportion_to_measured_rates_when_asked(cuda_device):
    """BRC_DECODE_CALIBRATE=1: a pool of more than 1 GiB measures the SMs' streaming rates once per device, launches
    cut their work in proportion (brc_decode_share_rates reports the shares), and the output still matches the
    oracle.  Without the variable (every other test of this suite) the shares are equal and the report is empty."""
    import os
    import subprocess
    import sys

    pool = KvPool(0, 1, 2, 256, 8)
    rates, n = (C.c_float * 256)(), C.c_uint32(7)
    _lib.call("brc_decode_share_rates", pool.handle, rates, 256, C.byref(n))
    assert n.value == 0
    pool.release()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_calibrated_worker.py")
    r = subprocess.run([sys.executable, worker], env=dict(os.environ, BRC_DECODE_CALIBRATE="1"), capture_output=True, text=True, timeout=600)
    print(r.stdout[-400:], r.stderr[-2000:])
    assert r.returncode == 0


def test_more_units_than_one_launch_holds(cuda_device):
    """1100 short sequences x 2 kv heads exceed the 2048 units one launch schedules: the host loops."""
    lens = (np.arange(1100) % 37 + 1).astype(np.int64)
    pool, _, _, got, want = _batch_case(16, 2, 256, lens, seed=97)
    assert_attention_close(got, want, "1100 sequences")
    pool.release()


def test_decode_refusals(cuda_device):
    pool = KvPool(0, 1, 2, 256, 8)
    L = _lib.load()
    q = torch.zeros((1, 16, 256), dtype=torch.half, device="cuda")
    out = torch.zeros((1, 16, 256), device="cuda")
    table, lens = dev_u32([[0, 1, 2, 3]]), dev_u32([10])
    ws = torch.zeros(1 << 22, dtype=torch.uint8, device="cuda")
    args = lambda **kw: [pool.handle, kw.get("layer", 0), C.c_void_p(q.data_ptr()), kw.get("dt", 1), kw.get("nh", 16), None, 0,
                         C.c_void_p(table.data_ptr()), 4, C.c_void_p(lens.data_ptr()), 1, kw.get("maxlen", 10), 0.0625,
                         C.c_void_p(out.data_ptr()), C.c_void_p(ws.data_ptr()), kw.get("wsb", ws.numel()), None]
    assert L.brc_paged_decode_attn(*args(maxlen=65)) == _lib.ERR_CAPACITY
    assert b"cells up to 65" in L.brc_last_error()
    assert L.brc_paged_decode_attn(*args(layer=3)) == _lib.ERR_INVALID
    assert L.brc_paged_decode_attn(*args(nh=15)) == _lib.ERR_INVALID
    assert L.brc_paged_decode_attn(*args(nh=80)) == _lib.ERR_UNSUPPORTED   # 40 per kv head: more than four passes of 8
    assert L.brc_paged_decode_attn(*args(dt=9)) == _lib.ERR_INVALID
    assert L.brc_paged_decode_attn(*args(wsb=16)) == _lib.ERR_INVALID
    # a length beyond the caller's bound and a table entry beyond the pool are caught on the device
    lens.fill_(40)
    assert L.brc_paged_decode_attn(*args(maxlen=10)) == 0
    with pytest.raises(_lib.BrcError, match="position past bound"):
        pool.check()
    lens.fill_(10)
    table.fill_(1000)
    assert L.brc_paged_decode_attn(*args()) == 0
    with pytest.raises(_lib.BrcError, match="page id >= n_pages"):
        pool.check()
    pool.release()


def test_twelve_heads_per_kv_head_in_two_passes(cuda_device):
    """The reference model's 24q / 2kv: the kernels take 8 query heads per kv head at a time, so the launch runs
    two passes (heads 0-7 and 8-11 of each kv head).  f32 query with gate, the partial form, and a decode step
    whose fused append must happen once."""
    n_head, n_kv, hd = 24, 2, 256
    lens = np.array([700, 33, 2062])
    pool, batch, qd, got, want = _batch_case(n_head, n_kv, hd, lens, seed=140, gate=True, q_dtype=DTYPE_F32)
    assert_attention_close(got, want, "24q/2kv with gate")
    nbytes = decode_partial_bytes(lens.size, n_head, hd)
    part = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    batch.partial(0, qd, part)
    out = torch.empty((lens.size, n_head, hd), device="cuda")
    decode_combine(0, part, 1, nbytes, lens.size, n_head, hd, out)
    pool.check()
    k, v = pool.read(0, 0).reshape(-1), pool.read(1, 0).reshape(-1)
    tables = batch.block_tables.cpu().numpy().astype(np.uint32)
    want_plain, _ = oracle.decode_batch(k, v, tables, lens, qd.cpu().numpy(), n_head, n_kv, hd)
    assert_attention_close(out.cpu().numpy(), want_plain, "24q/2kv partial form")
    # one decode step: the new cell is appended by the first pass only and seen by both
    k_new = torch.from_numpy(synth.normal(141, lens.size * n_kv * hd, 0.5).reshape(1, lens.size, n_kv * hd)).cuda()
    v_new = torch.from_numpy(synth.normal(142, lens.size * n_kv * hd, 0.5).reshape(1, lens.size, n_kv * hd)).cuda()
    step_out = torch.empty((1, lens.size, n_head, hd), device="cuda")
    batch.step(qd.unsqueeze(0).contiguous(), k_new, v_new, step_out)
    pool.check()
    k2, v2 = pool.read(0, 0).reshape(-1), pool.read(1, 0).reshape(-1)
    want_step, _ = oracle.decode_batch(k2, v2, tables, lens + 1, qd.cpu().numpy(), n_head, n_kv, hd)
    assert_attention_close(step_out[0].cpu().numpy(), want_step, "24q/2kv decode step")
    kb = oracle.f32_to_f16_bits_np(k_new.cpu().numpy()).reshape(lens.size, n_kv, hd)
    kp = k2.reshape(-1, n_kv, 16, hd)
    for s, n in enumerate(lens):
        assert np.array_equal(kp[tables[s, n // 16], :, n % 16, :], kb[s])
    pool.release()
