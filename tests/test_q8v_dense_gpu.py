"""Dense paged decode attention over q8_0 V page bodies (the reference dequantises V in registers in its apply shaders,
shaders/qsa_attn_apply.comp:60-77; sizes crates/breccia-kernels/src/qsa/mod.rs:339-349).  The oracle is the reference's own
statement: cpu::attend over K rounded to binary16 and V passed through cpu::to_q8_0 (attn_conformance.rs:1354-1452), and the
bar is the reference's, 1e-5 on its measure, on top of the target's max-abs 2e-3 / max-rel 1e-2: the quanta enter the tensor
cores as exact integers and the block scales ride on the probabilities, so nothing is lost against the binary16-V kernel."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from oracle import q8v
from breccia_b200 import _lib, synth
from breccia_b200._lib import DTYPE_F16, DTYPE_F32
from breccia_b200.qsa import DecodeBatch, KvPool
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors, dev_u32

pytestmark = pytest.mark.gpu
P = lambda x: C.c_void_p(x.data_ptr())


def fill(pool, layer, tables, lens, seed):
    """Appends lens[s] cells of LCG data to every sequence through the append kernel; returns the logical K (as stored,
    binary16 values) and V (through q8_0) of every sequence."""
    dim = pool.n_kv_head * pool.head_dim
    ks, vs = [], []
    for s, n in enumerate(lens):
        n = int(n)
        k = oracle.normalish(seed + 2 * s, max(n, 1) * dim).reshape(-1, dim)[:n]
        v = oracle.normalish(seed + 2 * s + 1, max(n, 1) * dim).reshape(-1, dim)[:n]
        if n:
            t_dev, p_dev = dev_u32(tables[s][None, :]), dev_u32(np.array([0]))
            kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
            _lib.call("brc_kv_append", pool.handle, layer, P(t_dev), tables.shape[1], P(p_dev), 1, n, None, n, n, P(kd), P(vd), DTYPE_F32, None)
            torch.cuda.synchronize()
        ks.append(oracle.to_f16(k))
        vs.append(q8v.to_q8_0(v.reshape(n * pool.n_kv_head, pool.head_dim)).reshape(n, dim) if n else v)
    pool.check()
    return ks, vs


def check(got, want, what):
    max_abs, max_rel, ref = attention_errors(got, want)
    print(f"{what}: max_abs {max_abs:.2e} max_rel {max_rel:.2e} ref_measure {ref:.2e}")
    assert np.isfinite(np.asarray(got)).all(), f"{what}: non-finite output"
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL and ref <= 1e-5, f"{what}: {max_abs:.2e} {max_rel:.2e} {ref:.2e}"


def test_reference_q8_case_64_cells_dense(cuda_device):
    """The reference's q8 fixture (LCG streams 0xF1..0xF4, 24 query heads over 2 kv heads, gate on) over all 64 cells."""
    n_head, n_kv, hd, cells = 24, 2, 256, 64
    dim = n_kv * hd
    pool = KvPool(0, 1, n_kv, hd, 8, v_q8=True)
    table = synth.permutation(92, 8)[:4].astype(np.uint32)
    k_all = oracle.normalish(0xF1, cells * dim).reshape(cells, dim)
    v_all = oracle.normalish(0xF2, cells * dim).reshape(cells, dim)
    q = oracle.normalish(0xF3, n_head * hd).reshape(1, n_head, hd)
    q_full = oracle.normalish(0xF4, n_head * 2 * hd).reshape(1, n_head, 2, hd)
    t_dev, p_dev = dev_u32(table[None, :]), dev_u32(np.array([0]))
    kd, vd = torch.from_numpy(k_all).cuda(), torch.from_numpy(v_all).cuda()     # named: they must outlive the call
    _lib.call("brc_kv_append", pool.handle, 0, P(t_dev), 4, P(p_dev), 1, cells, None, cells, cells, P(kd), P(vd), DTYPE_F32, None)
    torch.cuda.synchronize()
    batch = DecodeBatch(pool, n_head, table[None, :], [cells], q_dtype=DTYPE_F32)
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    gate = torch.from_numpy(q_full).cuda()
    batch.attend(0, torch.from_numpy(q).cuda(), out, gate=gate.view(-1)[hd:], gate_head_stride=2 * hd)
    pool.check()
    vq = q8v.to_q8_0(v_all.reshape(cells * n_kv, hd)).reshape(cells, dim)
    want = oracle.attend(q[0], oracle.to_f16(k_all), vq, np.arange(cells, dtype=np.uint32), cells - 1, n_head, n_kv, hd, gate=q_full[0, :, 1, :])
    check(out.cpu().numpy()[0], want, "reference q8 case, dense")
    pool.release()


@pytest.mark.parametrize("n_head,n_kv,hd,lens", [
    (16, 2, 256, [1, 15, 16, 17, 1025, 0, 300, 4097]),     # page edges, an empty sequence, units spanning several CTAs
    (8, 1, 256, [333, 48]),                                # one kv head per unit
    (12, 3, 128, [1000, 31, 257]),                         # head_dim 128, odd number of kv heads
    (32, 4, 128, [700, 5]),
    (24, 2, 256, [2062, 100]),                             # 12 query heads per kv head: two passes
])
def test_ragged_batches_and_geometries(cuda_device, n_head, n_kv, hd, lens):
    lens = np.asarray(lens)
    tables, n_pool = synth.scattered_tables(70 + n_head, np.maximum(lens, 1), pool_factor=1.3)
    pool = KvPool(0, 2, n_kv, hd, n_pool, v_q8=True)
    ks, vs = fill(pool, 1, tables, lens, 0x300)
    q = oracle.to_f16(oracle.normalish(0x3F0, lens.size * n_head * hd)).reshape(lens.size, n_head, hd)
    batch = DecodeBatch(pool, n_head, tables, lens, q_dtype=DTYPE_F16)
    out = torch.full((lens.size, n_head, hd), float("nan"), device="cuda")
    batch.attend(1, torch.from_numpy(q).cuda().half(), out)
    pool.check()
    got = out.cpu().numpy()
    for s, n in enumerate(lens):
        if n == 0:
            assert not got[s].any()
            continue
        want = oracle.attend(q[s], ks[s], vs[s], np.arange(n, dtype=np.uint32), int(n) - 1, n_head, n_kv, hd)
        check(got[s], want, f"{n_head}q/{n_kv}kv hd{hd}, sequence of {n}")
    pool.release()


def test_decode_steps_quantise_the_new_cell_in_the_attention_kernel(cuda_device):
    """brc_decode_step on a q8_0 pool, three layers, three steps: the kernel that is about to stream a sequence's newest
    page quantises and writes that cell itself (the reference's store rule, from the f32 value): the V pool must equal
    the oracle's bytes, K the binary16 append, and the outputs the oracle's attention."""
    n_head, n_kv, hd, n_layers = 16, 2, 256, 3
    dim = n_kv * hd
    lens = np.array([16, 5, 1023, 0, 300, 31])
    tables, n_pool = synth.scattered_tables(71, lens, pool_factor=1.4, extra_tokens=4)
    pool = KvPool(0, n_layers, n_kv, hd, n_pool, v_q8=True)
    logical = []
    for layer in range(n_layers):
        logical.append(fill(pool, layer, tables, lens, 0x400 + 64 * layer))
    want_v = [pool.read(1, layer).copy() for layer in range(n_layers)]
    want_k = [pool.read(0, layer).reshape(-1).view(np.uint32).copy() for layer in range(n_layers)]
    batch = DecodeBatch(pool, n_head, tables, lens)
    cur = lens.copy()
    for step in range(3):
        q = oracle.to_f16(synth.normal(1600 + step, n_layers * lens.size * n_head * hd)).reshape(n_layers, lens.size, n_head, hd)
        kn = synth.normal(1700 + step, n_layers * lens.size * dim, 0.5).reshape(n_layers, lens.size, dim)
        vn = synth.normal(1800 + step, n_layers * lens.size * dim, 0.5).reshape(n_layers, lens.size, dim)
        out = torch.full((n_layers, lens.size, n_head, hd), float("nan"), device="cuda")
        batch.step(torch.from_numpy(q).cuda().half(), torch.from_numpy(kn).cuda(), torch.from_numpy(vn).cuda(), out)
        pool.check()
        got = out.cpu().numpy()
        for layer in range(n_layers):
            ks, vs = logical[layer]
            for s in range(lens.size):
                q8v.v_append(want_v[layer], tables[s], vn[layer, s][None, :], int(cur[s]), n_kv, hd)
                assert oracle.kv_append(want_k[layer], want_k[layer].copy(), tables[s], kn[layer, s], vn[layer, s], int(cur[s]), n_kv, hd) == 0
                ks[s] = np.concatenate([ks[s].reshape(-1, dim), oracle.to_f16(kn[layer, s])[None, :]])
                vs[s] = np.concatenate([vs[s].reshape(-1, dim), q8v.to_q8_0(vn[layer, s].reshape(n_kv, hd)).reshape(1, dim)])
                n = int(cur[s]) + 1
                want = oracle.attend(q[layer, s], ks[s], vs[s], np.arange(n, dtype=np.uint32), n - 1, n_head, n_kv, hd)
                check(got[layer, s], want, f"step {step} layer {layer} sequence {s}")
            assert np.array_equal(pool.read(1, layer), want_v[layer]), f"V pool, layer {layer}, step {step}"
            assert np.array_equal(pool.read(0, layer).reshape(-1), want_k[layer].view(np.uint16)), f"K pool, layer {layer}, step {step}"
        cur += 1
    # binary16 sources cannot feed the fused q8_0 append
    with pytest.raises(_lib.BrcError) as err:
        batch.step(torch.zeros((1, lens.size, n_head, hd), device="cuda").half(), torch.zeros((1, lens.size, dim), device="cuda").half(),
                   torch.zeros((1, lens.size, dim), device="cuda").half(), out, kv_dtype=DTYPE_F16)
    assert err.value.code == _lib.ERR_UNSUPPORTED
    pool.release()


def test_a_layer_of_the_batched_workload_size(cuda_device):
    """16 sequences of 2048..8192 cells (70 k cells, every CTA busy): q8_0 output against the oracle on two sequences,
    finite everywhere, two launches bit-identical, and within the storage loss of the binary16 answer."""
    n_head, n_kv, hd = 16, 2, 256
    lens = synth.uniform_ints(77, 16, 2048, 8192)
    tables, n_pool = synth.scattered_tables(78, lens, pool_factor=1.25)
    pool = KvPool(0, 1, n_kv, hd, n_pool, v_q8=True)
    ks, vs = fill(pool, 0, tables, lens, 0x500)
    q = oracle.to_f16(oracle.normalish(0x5F0, lens.size * n_head * hd)).reshape(lens.size, n_head, hd)
    batch = DecodeBatch(pool, n_head, tables, lens)
    qd = torch.from_numpy(q).cuda().half()
    out, again = torch.full((lens.size, n_head, hd), float("nan"), device="cuda"), torch.zeros((lens.size, n_head, hd), device="cuda")
    batch.attend(0, qd, out)
    batch.attend(0, qd, again)
    pool.check()
    got = out.cpu().numpy()
    assert np.isfinite(got).all() and torch.equal(out, again)
    for s in (0, 9):
        n = int(lens[s])
        want = oracle.attend(q[s], ks[s], vs[s], np.arange(n, dtype=np.uint32), n - 1, n_head, n_kv, hd)
        check(got[s], want, f"sequence {s} of {n} cells")
    pool.release()
