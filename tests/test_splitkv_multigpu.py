"""Split-KV decode across GPUs (partials pushed to the peers by the attention kernel itself; NCCL all-gather +
merge as the baseline).  The cross-GPU cases need at least two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("n_tokens", [5000, 33])
def test_split_kv_across_gpus_equals_the_whole(cuda_device, n_tokens):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + n_tokens % 97), os.path.join(HERE, "_splitkv_worker.py"), str(n_tokens)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0


def test_split_kv_machinery_with_one_rank(cuda_device):
    """World of one: the exchange kernel has no peer to store to or wait for and reduces to the merge."""
    import numpy as np

    import oracle
    from breccia_b200 import synth
    from breccia_b200.qsa import KvPool
    from breccia_b200.splitkv import SplitKvDecode
    from helpers import fill_pool_from_host

    n_head, n_kv, hd, n_tokens = 16, 2, 256, 3000
    n_pages = (n_tokens + 15) // 16
    pool = KvPool(0, 1, n_kv, hd, n_pages + 4)
    k, v = fill_pool_from_host(pool, 0, 31)
    table = synth.permutation(5, n_pages + 4)[:n_pages]
    q = oracle.to_f16(synth.normal(6, n_head * hd)).reshape(1, n_head, hd)
    gate = synth.normal(7, n_head * hd).reshape(1, n_head, hd).astype(np.float32)
    split = SplitKvDecode(pool, n_head, table, n_tokens)
    out = torch.full((1, n_head, hd), float("nan"), device="cuda")
    g = torch.from_numpy(gate).cuda()
    for _ in range(6):
        split.attend(0, torch.from_numpy(q).cuda().half(), out, gate=g, gate_head_stride=hd)
    pool.check()
    want, _ = oracle.decode_batch(k, v, table[None, :], np.array([n_tokens]), q, n_head, n_kv, hd, gate=gate)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-3
    # brc_comm_reset (what every rank calls after an exchange timed out) empties the receive buffers and restarts
    # the call count: the next calls give the same bits
    import ctypes as C

    from breccia_b200 import _lib
    first = out.clone()
    _lib.call("brc_comm_reset", split.comm, None)
    out.fill_(float("nan"))
    for _ in range(5):
        split.attend(0, torch.from_numpy(q).cuda().half(), out, gate=g, gate_head_stride=hd)
    pool.check()
    assert torch.equal(out, first)
    split.close()
    pool.release()


def test_split_kv_step_over_layers_with_one_rank(cuda_device):
    """brc_splitkv_step: the layers of one token launched together (overlapping kernels, one bank of
    partials per layer), then one exchange + merge kernel for all of them; every layer against the oracle."""
    import numpy as np

    import oracle
    from breccia_b200 import synth
    from breccia_b200.qsa import KvPool
    from breccia_b200.splitkv import SplitKvDecode
    from helpers import fill_pool_from_host

    n_head, n_kv, hd, n_tokens, n_layers = 16, 2, 256, 9000, 4
    n_pages = (n_tokens + 15) // 16
    pool = KvPool(0, n_layers, n_kv, hd, n_pages + 4)
    kv = [fill_pool_from_host(pool, layer, 41 + layer) for layer in range(n_layers)]
    table = synth.permutation(8, n_pages + 4)[:n_pages]
    q = oracle.to_f16(synth.normal(9, n_layers * n_head * hd)).reshape(n_layers, 1, n_head, hd)
    split = SplitKvDecode(pool, n_head, table, n_tokens, max_layers=n_layers)
    out = torch.full((n_layers, 1, n_head, hd), float("nan"), device="cuda")
    qd = torch.from_numpy(q).cuda().half()
    for _ in range(3):
        split.step(qd, out)
    pool.check()
    got = out.cpu().numpy()
    for layer in range(n_layers):
        want, _ = oracle.decode_batch(kv[layer][0], kv[layer][1], table[None, :], np.array([n_tokens]), q[layer], n_head, n_kv, hd)
        assert np.abs(got[layer] - want).max() <= 2e-3, f"layer {layer}"
    split.close()
    pool.release()


def test_a_peer_that_never_arrives_times_out_and_leaves_the_context_usable(cuda_device):
    """Rank 0 of a world of two exchanges alone (rank 1's end exists but never calls): the wait for its
    flag runs out after 20 ms, the output stays as it was, the pool reports BRC_ERR_TIMEOUT, and the next
    call on the same context works."""
    import ctypes as C

    from breccia_b200 import _lib
    from breccia_b200.qsa import KvPool, decode_partial_bytes

    n_head, hd = 16, 256
    pool = KvPool(0, 1, 2, hd, 8)
    comms = [C.c_void_p(), C.c_void_p()]
    for r in range(2):
        _lib.call("brc_comm_create", pool.handle, 2, r, 1, n_head, C.byref(comms[r]))
    arr = (C.c_void_p * 2)(comms[0], comms[1])
    for r in range(2):
        _lib.call("brc_comm_connect_local", comms[r], arr, 2)
    _lib.call("brc_comm_set_wait_ms", comms[0], 20)
    part = torch.zeros(decode_partial_bytes(1, n_head, hd), dtype=torch.uint8, device="cuda")
    out = torch.full((1, n_head, hd), 7.0, device="cuda")
    _lib.call("brc_splitkv_exchange_combine", comms[0], C.c_void_p(part.data_ptr()), 1, None, 0, C.c_void_p(out.data_ptr()), None)
    torch.cuda.synchronize()
    with pytest.raises(_lib.BrcError, match="wait"):
        pool.check()
    assert bool((out == 7.0).all())
    pool.check()                      # the check word was cleared; the context still works
    assert float((out + 1).sum()) == 8.0 * n_head * hd
    for c in comms:
        _lib.call("brc_comm_destroy", c)
    pool.release()


def test_fused_exchange_whose_peer_never_arrives_times_out_and_leaves_the_context_usable(cuda_device):
    """The same for the exchange that rides in the attention kernel (brc_splitkv_attend): rank 0 of a world
    of two attends alone; its own partial lands and is flagged, rank 1's flag is never set, so the unit's
    cross-rank merge gives up after 20 ms, leaves the output rows as they were and reports the expiry."""
    import ctypes as C

    import numpy as np

    from breccia_b200 import _lib, synth
    from breccia_b200.qsa import DecodeBatch, KvPool
    from helpers import fill_pool_from_host

    n_head, hd, lens = 16, 256, np.array([100])
    tables, n_pool = synth.scattered_tables(3, lens, extra_tokens=1)
    pool = KvPool(0, 1, 2, hd, n_pool)
    fill_pool_from_host(pool, 0, 77)
    batch = DecodeBatch(pool, n_head, tables, lens)
    comms = [C.c_void_p(), C.c_void_p()]
    for r in range(2):
        _lib.call("brc_comm_create", pool.handle, 2, r, 1, n_head, C.byref(comms[r]))
    arr = (C.c_void_p * 2)(comms[0], comms[1])
    for r in range(2):
        _lib.call("brc_comm_connect_local", comms[r], arr, 2)
    _lib.call("brc_comm_set_wait_ms", comms[0], 20)
    q = torch.randn((1, n_head, hd), device="cuda").half()
    out = torch.full((1, n_head, hd), 7.0, device="cuda")
    _lib.call("brc_splitkv_attend", comms[0], 0, C.c_void_p(q.data_ptr()), _lib.DTYPE_F16, None, 0,
              C.c_void_p(batch.block_tables.data_ptr()), batch.table_stride, C.c_void_p(batch.seq_lens.data_ptr()), 1,
              batch.capacity, 0.0625, C.c_void_p(out.data_ptr()), C.c_void_p(batch.scratch.data_ptr()), batch.scratch.numel(), None)
    torch.cuda.synchronize()
    with pytest.raises(_lib.BrcError, match="wait"):
        pool.check()
    assert bool((out == 7.0).all())
    pool.check()
    batch.attend(0, q, out)           # the plain call on the same pool still works
    pool.check()
    assert bool(torch.isfinite(out).all()) and not bool((out == 7.0).all())
    for c in comms:
        _lib.call("brc_comm_destroy", c)
    pool.release()
