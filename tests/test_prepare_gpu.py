"""The steps in front of the cache fused into one launch (brc_qk_prepare_append): per-head RMSNorm of q and k,
partial NEOX rotary, f16 append — against the float64 restatement of the reference's CPU code
(oracle/prepare_ref.py).

Bars: the prepared query within 2e-6 relative to max(|want|, 1) (fp32 arithmetic against f64); the stored K bits
equal to the integer-rule rounding of the oracle's fp32 K except where that value sits within fp32 noise of a
rounding boundary (then one f16 step apart at most), V bit-exact (it is only converted)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from oracle import prepare_ref
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import KvPool
from helpers import dev_u32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_head,n_kv,hd,q_stride,n_rot,pos0s,T", [
    (16, 2, 256, 512, 64, [1024, 0, 37], 1),       # decode shapes: one token per sequence, gate half present
    (24, 2, 256, 512, 64, [5], 33),                # the reference's own head count; a chunk across page edges
    (8, 4, 128, 128, 128, [100, 7], 4),            # full rotary, no gate half
])
def test_prepare_matches_reference_arithmetic(cuda_device, n_head, n_kv, hd, q_stride, n_rot, pos0s, T):
    pos0s = np.asarray(pos0s)
    n_seqs, max_pos = pos0s.size, 2048
    tables, n_pool = synth.scattered_tables(70 + T, pos0s + T, pool_factor=1.5)
    pool = KvPool(0, 2, n_kv, hd, n_pool)
    pool.zero()
    tok = n_seqs * T
    q_full = synth.normal(71, tok * n_head * q_stride, 1.3).reshape(tok, n_head, q_stride)
    k_cur = synth.normal(72, tok * n_kv * hd, 0.7).reshape(tok, n_kv * hd)
    v_cur = synth.normal(73, tok * n_kv * hd, 0.5).reshape(tok, n_kv * hd)
    q_gamma = (1.0 + 0.1 * synth.normal(74, hd)).astype(np.float32)
    k_gamma = (1.0 + 0.1 * synth.normal(75, hd)).astype(np.float32)
    table = prepare_ref.rope_table(1.0e6, n_rot, max_pos)
    eps = 1e-6
    positions = np.concatenate([p0 + np.arange(T) for p0 in pos0s])
    want_q, want_k, _ = prepare_ref.prepare(q_full, k_cur, v_cur, q_gamma, k_gamma, eps, table, n_rot, positions, n_head, n_kv, hd, q_stride)

    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    qf, kc, vc, qg, kg, tb = d(q_full), d(k_cur), d(v_cur), d(q_gamma), d(k_gamma), d(table)
    t_dev, p_dev = dev_u32(tables), dev_u32(pos0s)
    for q_dtype in (DTYPE_F32, DTYPE_F16):
        q_out = torch.full((tok, n_head, hd), float("nan"), device="cuda", dtype=torch.float32 if q_dtype == DTYPE_F32 else torch.float16)
        _lib.call("brc_qk_prepare_append", pool.handle, 1, C.c_void_p(qf.data_ptr()), q_stride, n_head, C.c_void_p(kc.data_ptr()),
                  C.c_void_p(vc.data_ptr()), C.c_void_p(qg.data_ptr()), C.c_void_p(kg.data_ptr()), eps, C.c_void_p(tb.data_ptr()),
                  n_rot, max_pos, C.c_void_p(t_dev.data_ptr()), tables.shape[1], C.c_void_p(p_dev.data_ptr()), n_seqs, T,
                  int(pos0s.max() + T), C.c_void_p(q_out.data_ptr()), q_dtype, None)
        pool.check()
        got_q = q_out.float().cpu().numpy()
        tol = 2e-6 if q_dtype == DTYPE_F32 else 1e-3
        assert np.abs(got_q - want_q).max() <= tol * max(1.0, np.abs(want_q).max())

    # the cache: gather every sequence's new cells and compare bit patterns
    kp, vp = pool.read(0, 1).reshape(n_pool, n_kv, 16, hd), pool.read(1, 1).reshape(n_pool, n_kv, 16, hd)
    want_k_bits = oracle.f32_to_f16_bits_np(want_k).reshape(tok, n_kv, hd)
    want_v_bits = oracle.f32_to_f16_bits_np(v_cur).reshape(tok, n_kv, hd)
    off = 0
    for s, p0 in enumerate(pos0s):
        for t in range(T):
            c = int(p0) + t
            pg = tables[s, c // 16]
            assert np.array_equal(vp[pg, :, c % 16, :], want_v_bits[off]), f"V sequence {s} cell {c}"
            diff = kp[pg, :, c % 16, :].astype(np.int32) - want_k_bits[off].astype(np.int32)
            assert np.abs(diff).max() <= 1, f"K sequence {s} cell {c}: more than one f16 step"
            assert (diff != 0).mean() <= 0.01, f"K sequence {s} cell {c}: {(diff != 0).mean():.3%} of elements differ"
            off += 1
    # nothing else in the pool was touched
    live = np.zeros((n_pool, 16), bool)
    for s, p0 in enumerate(pos0s):
        for t in range(T):
            live[tables[s, (int(p0) + t) // 16], (int(p0) + t) % 16] = True
    assert not kp[~np.broadcast_to(live[:, None, :, None], kp.shape)].any()
    assert not pool.read(0, 0).any()          # the other layer
    pool.release()


def test_prepare_refusals(cuda_device):
    L = _lib.load()
    pool = KvPool(0, 1, 2, 256, 8)
    z = torch.zeros(16 * 512 * 4, device="cuda")
    t, p0 = dev_u32([[0, 1]]), dev_u32([30])
    P = lambda x: C.c_void_p(x.data_ptr())
    args = lambda **kw: [pool.handle, 0, P(z), kw.get("qs", 512), 16, P(z), P(z), P(z), P(z), 1e-6, P(z), kw.get("n_rot", 64), 64, P(t), 2,
                         P(p0), 1, kw.get("T", 1), kw.get("end", 31), P(z), kw.get("dt", 0), None]
    assert L.brc_qk_prepare_append(*args(end=33)) == _lib.ERR_CAPACITY and b"kv_append would write" in L.brc_last_error()
    assert L.brc_qk_prepare_append(*args(qs=128)) == _lib.ERR_INVALID
    assert L.brc_qk_prepare_append(*args(n_rot=63)) == _lib.ERR_INVALID
    assert L.brc_qk_prepare_append(*args(dt=5)) == _lib.ERR_INVALID
    # a position past the caller's bound is caught on the device and the rows are skipped
    assert L.brc_qk_prepare_append(*args(end=20)) == 0
    with pytest.raises(_lib.BrcError, match="position past bound"):
        pool.check()
    pool.release()


def test_prepare_on_a_q8_0_v_pool_quantises_v_by_the_append_rule(cuda_device):
    """On a q8_0 V pool the fused launch stores V as q8_0 blocks, byte for byte what brc_kv_append stores from the
    same f32 rows (store rule of shaders/qsa_kv_append.comp:117-133); K and the prepared query as on any pool."""
    from oracle import q8v

    n_head, n_kv, hd, q_stride, n_rot, T = 24, 2, 256, 512, 64, 21
    pos0s = np.array([5, 40])
    n_seqs, max_pos = pos0s.size, 512
    tables, n_pool = synth.scattered_tables(91, pos0s + T, pool_factor=1.5)
    pool = KvPool(0, 1, n_kv, hd, n_pool, v_q8=True)
    tok = n_seqs * T
    q_full = synth.normal(92, tok * n_head * q_stride, 1.3).reshape(tok, n_head, q_stride)
    k_cur = synth.normal(93, tok * n_kv * hd, 0.7).reshape(tok, n_kv * hd)
    v_cur = synth.normal(94, tok * n_kv * hd, 0.5).reshape(tok, n_kv * hd)
    v_cur[3, :32] = 0.0                                   # an all-zero block: scale 1, quanta 0
    gam = np.ones(hd, np.float32)
    table = prepare_ref.rope_table(1.0e6, n_rot, max_pos)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    qf, kc, vc, qg, tb = d(q_full), d(k_cur), d(v_cur), d(gam), d(table)
    t_dev, p_dev = dev_u32(tables), dev_u32(pos0s)
    q_out = torch.empty((tok, n_head, hd), device="cuda")
    _lib.call("brc_qk_prepare_append", pool.handle, 0, C.c_void_p(qf.data_ptr()), q_stride, n_head, C.c_void_p(kc.data_ptr()),
              C.c_void_p(vc.data_ptr()), C.c_void_p(qg.data_ptr()), C.c_void_p(qg.data_ptr()), 1e-6, C.c_void_p(tb.data_ptr()),
              n_rot, max_pos, C.c_void_p(t_dev.data_ptr()), tables.shape[1], C.c_void_p(p_dev.data_ptr()), n_seqs, T,
              int(pos0s.max() + T), C.c_void_p(q_out.data_ptr()), DTYPE_F32, None)
    pool.check()
    got_v = pool.read(1, 0)                                # [rows][288] bytes
    want_v = np.zeros_like(got_v)
    for s in range(n_seqs):
        q8v.v_append(want_v, tables[s], v_cur[s * T:(s + 1) * T], int(pos0s[s]), n_kv, hd)
    assert np.array_equal(got_v, want_v)
    pool.release()
