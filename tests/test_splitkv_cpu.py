"""Split-KV across ranks on the CPU (gloo, world size 2 and 3): the partition of the cell range, the
layout of the exchanged partial buffers and the log-sum-exp merge, with the oracle standing in for the
device kernels.  The merged result must equal attention over the whole range."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from breccia_b200.splitkv import kv_range

N_HEAD, N_KV, HD = 16, 2, 256


def test_kv_range_is_a_page_aligned_partition():
    for n_tokens in (1, 15, 16, 17, 1000, 131072, 131073):
        for world in (1, 2, 3, 4, 8):
            cuts = [kv_range(r, world, n_tokens) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n_tokens
            for r in range(world):
                b, e = cuts[r]
                assert b <= e and (b % 16 == 0 or b == n_tokens)
                if r + 1 < world:
                    assert e == cuts[r + 1][0] and (e % 16 == 0 or e == n_tokens)
            sizes = [e - b for b, e in cuts]
            assert max(sizes) - min(sizes) < 32 or n_tokens < 16 * world  # one page, plus a partial last page


def _worker(rank, world, port, n_tokens, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(123)          # same data on every rank
    q = rng.standard_normal((N_HEAD, HD)).astype(np.float32)
    k = oracle.to_f16(rng.standard_normal((n_tokens, N_KV, HD)).astype(np.float32) * 0.5)
    v = oracle.to_f16(rng.standard_normal((n_tokens, N_KV, HD)).astype(np.float32) * 0.5)
    b, e = kv_range(rank, world, n_tokens)
    # this rank's partial in the layout brc_decode_partial writes: acc [n_head][hd] f32, then (m, l) [n_head][2]
    part = np.zeros(N_HEAD * (HD + 2), np.float32)
    for h in range(N_HEAD):
        m, l, acc = oracle.partial_head(q[h], k, v, b, e, h * N_KV // N_HEAD, N_KV, HD, 1.0 / 16.0)
        part[h * HD:(h + 1) * HD] = acc
        part[N_HEAD * HD + 2 * h] = m
        part[N_HEAD * HD + 2 * h + 1] = l
    mine = torch.from_numpy(part)
    gathered = torch.zeros(world * part.size, dtype=torch.float32)
    dist.all_gather_into_tensor(gathered, mine)
    g = gathered.numpy().reshape(world, -1)
    out = np.zeros((N_HEAD, HD))
    for h in range(N_HEAD):
        ms = g[:, N_HEAD * HD + 2 * h].astype(np.float64)
        ls = g[:, N_HEAD * HD + 2 * h + 1].astype(np.float64)
        accs = g[:, h * HD:(h + 1) * HD].astype(np.float64)
        out[h] = oracle.lse_combine(ms, ls, accs)
    whole = oracle.attend(q, k, v, np.arange(n_tokens, dtype=np.uint32), n_tokens - 1, N_HEAD, N_KV, HD)
    err = float(np.abs(out - whole).max())
    np.save(os.path.join(out_dir, f"err{rank}.npy"), np.array([err]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_tokens", [(2, 1000), (3, 37)])
def test_split_kv_over_gloo_ranks_equals_unsplit(tmp_path, world, n_tokens):
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_worker, args=(world, port, n_tokens, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert np.load(tmp_path / f"err{r}.npy")[0] < 1e-5   # partials travel as f32
