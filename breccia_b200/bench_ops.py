"""Per-operator benchmark of the paged-KV path (the counterpart of the reference's `breccia bench ops
--op qsa`, crates/breccia-kernels/src/qsa/bench.rs; one JSON line per cell with the fields of its
`OpCell`: op, case, units, bytes or flops, us, GB/s or TFLOP/s, iters).

    python -m breccia_b200.bench_ops [--op prefill|prepare|sparse|topk|indexer|chain|movers|all] [--iters N]

Timing: CUDA events on the launching stream, 3 warm-up runs, the mean of `iters` runs (`us`).  Calls of a few
tens of microseconds are also replayed from a CUDA graph (`us_graph`): back to back from Python such a call
measures the host's cost of issuing it, the replay the device's time; GB/s and TFLOP/s of those lines are
computed from `us_graph`.  `chain` = block scores -> top-k -> selected-block attention in a row.  Shapes are the
benchmark configurations: prefill = 64 sequences sharing a 4096-token prefix, 256-token chunk each
(GQA 16q/2kv, head_dim 256); the byte movers run on the same pool.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np
import torch

from . import _lib, synth
from ._lib import DTYPE_F16, DTYPE_F32
from .qsa import KvPool, _ptr, _stream_ptr

N_HEAD, N_KV, HD = 16, 2, 256


def timed(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters  # us


def timed_graph(fn, iters: int) -> float:
    """The same calls captured once in a CUDA graph and replayed: the device's time per call without the
    host's cost of issuing it (for calls of a few tens of microseconds `timed` measures the host)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters  # us


def emit(**kw):
    print(json.dumps(kw), flush=True)


def dev_u32(a):
    return torch.as_tensor(np.ascontiguousarray(a, np.uint32).astype(np.int32), device="cuda")


def cfg4_tables(pool: KvPool, n_seqs: int, prefix: int, chunk: int):
    """Shared prefix pages + private suffix pages; a partial last prefix page is forked copy-on-write."""
    n_prefix_pages = (prefix + 15) // 16
    owner = pool.alloc(n_prefix_pages)
    total_pages = (prefix + chunk + 15) // 16
    tables = np.zeros((n_seqs, total_pages), np.uint32)
    fork_us = 0.0
    for s in range(n_seqs):
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        child, fresh = pool.fork(owner, prefix)
        t1.record()
        torch.cuda.synchronize()
        fork_us += t0.elapsed_time(t1) * 1e3
        tables[s, :n_prefix_pages] = child
        tables[s, n_prefix_pages:] = pool.alloc(total_pages - n_prefix_pages)
    return owner, tables, fork_us / n_seqs


def bench_prefill(iters: int, prefix: int):
    n_seqs, chunk = 64, 256
    n_pages = (prefix + 15) // 16 + n_seqs * 18 + 8
    pool = KvPool(0, 1, N_KV, HD, n_pages)
    owner, tables, fork_us = cfg4_tables(pool, n_seqs, prefix, chunk)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    # fill the prefix once (through the owner's table) and every suffix (chunk append of 64 x 256 tokens)
    t_dev = dev_u32(tables)
    zero = dev_u32([0])
    kp = torch.randn((prefix, N_KV * HD), generator=gen, device="cuda") * 0.5
    vp = torch.randn((prefix, N_KV * HD), generator=gen, device="cuda") * 0.5
    # each sequence's copy-on-write page holds the same prefix cells, so write the prefix through every table
    for s in range(n_seqs if prefix % 16 else 1):
        _lib.call("brc_kv_append", pool.handle, 0, C.c_void_p(t_dev[s].data_ptr()), tables.shape[1], _ptr(zero), 1, prefix, None,
                  prefix, prefix, _ptr(kp), _ptr(vp), DTYPE_F32, _stream_ptr())
    pos0 = dev_u32(np.full(n_seqs, prefix))
    ks = torch.randn((n_seqs * chunk, N_KV * HD), generator=gen, device="cuda") * 0.5
    vs = torch.randn((n_seqs * chunk, N_KV * HD), generator=gen, device="cuda") * 0.5

    def append():
        _lib.call("brc_kv_append", pool.handle, 0, _ptr(t_dev), tables.shape[1], _ptr(pos0), n_seqs, chunk, None,
                  n_seqs * chunk, prefix + chunk, _ptr(ks), _ptr(vs), DTYPE_F32, _stream_ptr())

    us = timed(append, iters)
    us_graph = timed_graph(append, iters)
    nbytes = n_seqs * chunk * (N_KV * HD * 2 * 2 + N_KV * HD * 4 * 2)
    emit(op="kv_append", case=f"chunk append, {n_seqs} sequences x {chunk} tokens, f32 sources, 1 layer", units=n_seqs * chunk,
         bytes=nbytes, us=us, us_graph=us_graph, gbps=nbytes / us_graph / 1e3, iters=iters)
    q = (torch.randn((n_seqs, chunk, N_HEAD, HD), generator=gen, device="cuda")).half()
    out = torch.empty((n_seqs, chunk, N_HEAD, HD), dtype=torch.float32, device="cuda")

    def prefill():
        _lib.call("brc_paged_prefill_attn", pool.handle, 0, _ptr(q), DTYPE_F16, N_HEAD, None, 0, _ptr(t_dev), tables.shape[1],
                  _ptr(pos0), n_seqs, chunk, prefix + chunk, 1.0 / 16.0, _ptr(out), _stream_ptr())

    us = timed(prefill, iters)
    pool.check()
    visible = chunk * prefix + chunk * (chunk + 1) // 2
    flops = 4.0 * N_HEAD * HD * visible * n_seqs
    emit(op="paged_prefill_attn", case=f"{n_seqs} sequences, shared {prefix}-token prefix, {chunk}-token chunk, 16q/2kv hd256, 1 layer",
         units=n_seqs * chunk, flops=flops, us=us, tflops=flops / us / 1e6, iters=iters,
         cow_fork_us_per_sequence=fork_us, partial_prefix_page=bool(prefix % 16))
    pool.release()


def bench_prepare(iters: int):
    """RMSNorm + rotary + append in one launch: a decode step's rows (32 sequences x 1 token) and a prefill
    chunk's (64 x 256 tokens); the reference's head layout (q | gate blocks of 512)."""
    import math

    for n_seqs, T in ((32, 1), (64, 256)):
        tokens = n_seqs * T
        pages_per_seq = (4096 + T + 15) // 16
        pool = KvPool(0, 1, N_KV, HD, n_seqs * pages_per_seq)
        tables = np.arange(n_seqs * pages_per_seq, dtype=np.uint32).reshape(n_seqs, pages_per_seq)
        t_dev, p_dev = dev_u32(tables), dev_u32(np.full(n_seqs, 4096))
        gen = torch.Generator(device="cuda")
        gen.manual_seed(5)
        q_full = torch.randn((tokens, N_HEAD, 2 * HD), generator=gen, device="cuda")
        k_cur = torch.randn((tokens, N_KV * HD), generator=gen, device="cuda")
        v_cur = torch.randn((tokens, N_KV * HD), generator=gen, device="cuda")
        gamma = torch.ones(HD, device="cuda")
        n_rot, max_pos = 64, 8192
        inv = torch.pow(torch.tensor(1.0e6, dtype=torch.float64), -2.0 * torch.arange(n_rot // 2, dtype=torch.float64) / n_rot)
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
        table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().cuda().contiguous()
        q_out = torch.empty((tokens, N_HEAD, HD), dtype=torch.float16, device="cuda")

        def prepare():
            _lib.call("brc_qk_prepare_append", pool.handle, 0, _ptr(q_full), 2 * HD, N_HEAD, _ptr(k_cur), _ptr(v_cur), _ptr(gamma),
                      _ptr(gamma), 1e-6, _ptr(table), n_rot, max_pos, _ptr(t_dev), pages_per_seq, _ptr(p_dev), n_seqs, T,
                      4096 + T, _ptr(q_out), DTYPE_F16, _stream_ptr())

        us = timed(prepare, iters)
        us_graph = timed_graph(prepare, iters)
        pool.check()
        nbytes = tokens * (N_HEAD * HD * 4 + 2 * N_KV * HD * 4 + N_HEAD * HD * 2 + 2 * N_KV * HD * 2)
        emit(op="qk_prepare_append", case=f"{n_seqs} sequences x {T} tokens: RMSNorm + rotary of 16 q / 2 k heads, f16 append of k and v, 1 layer",
             units=tokens, bytes=nbytes, us=us, us_graph=us_graph, gbps=nbytes / us_graph / 1e3, iters=iters)
        pool.release()


def bench_sparse(iters: int):
    """The reference's decode shape: one row per sequence at position ~32 k, 513 selected 4-cell blocks (2052 cells),
    24 query heads over 2 kv heads; one sequence and a batch of 32."""
    from .qsa import sparse_attend

    n_head, ctx, n_sel = 24, 32768, 513
    for n_seqs, v_q8 in ((1, False), (32, False), (1, True), (32, True)):
        pages = ctx // 16
        pool = KvPool(0, 1, N_KV, HD, n_seqs * pages, v_q8=v_q8)
        tables = synth.permutation(3, n_seqs * pages).reshape(n_seqs, pages)
        ids = np.stack([np.sort(synth.permutation(10 + s, ctx // 4)[:n_sel]) for s in range(n_seqs)]).astype(np.uint32)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(6)
        q = torch.randn((n_seqs, n_head, HD), generator=gen, device="cuda")
        out = torch.empty((n_seqs, n_head, HD), device="cuda")
        t_dev, p_dev, i_dev = dev_u32(tables), dev_u32(np.full(n_seqs, ctx - 1)), dev_u32(ids)
        c_dev = dev_u32(np.full(n_seqs, n_sel))

        def run():
            sparse_attend(pool, 0, q, n_head, t_dev, p_dev, 1, i_dev, c_dev, ctx, out)

        us = timed(run, iters)
        us_graph = timed_graph(run, iters)
        pool.check()
        # every selected cell's K and V once per kv head; a q8_0 V row is 9/16 of a binary16 one
        nbytes = int(n_seqs * n_sel * 4 * N_KV * HD * 2 * (1 + (0.5625 if v_q8 else 1)))
        emit(op="paged_sparse_attn", case=f"{n_seqs} sequence(s), 1 row each, {n_sel} selected blocks = {n_sel * 4} cells of {ctx}, "
             f"{n_head}q/{N_KV}kv hd{HD}, 1 layer, V {'q8_0' if v_q8 else 'f16'}", units=n_seqs, bytes=nbytes, us=us,
             us_graph=us_graph, gbps=nbytes / us_graph / 1e3, iters=iters)
        pool.release()


def bench_topk(iters: int):
    """Top-k block selection at the reference's shapes: 512 of 8192 blocks (32 768 cells) for one decode row, for 32
    rows and for a 256-row prefill chunk of 8 sequences; 512 of 65 536 blocks (its longest cache) for one row."""
    from .qsa import topk_blocks

    pool = KvPool(0, 1, N_KV, HD, 4)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    for n_seqs, rows_per_seq, n_blocks in ((1, 1, 8192), (32, 1, 8192), (8, 256, 8192), (1, 1, 65536)):
        rows = n_seqs * rows_per_seq
        scores = torch.randn((rows, n_blocks), generator=gen, device="cuda")
        pos0 = dev_u32(np.full(n_seqs, 4 * n_blocks - rows_per_seq))
        us = timed(lambda: topk_blocks(pool, scores, pos0, rows_per_seq), iters)
        us_graph = timed_graph(lambda: topk_blocks(pool, scores, pos0, rows_per_seq), iters)
        pool.check()
        emit(op="topk_blocks", case=f"{rows} row(s) x {n_blocks} blocks, top 512 + own block", units=rows,
             bytes=rows * n_blocks * 4, us=us, us_graph=us_graph, gbps=rows * n_blocks * 4 / us_graph / 1e3, iters=iters)
    pool.release()


def bench_indexer(iters: int):
    """Indexer stages at the reference's shapes: scores of one decode row, of 32 rows and of a 256-row chunk of 8
    sequences over 8192 pooled keys (32 768 cells); pooling + tail of a 256-token chunk of 8 sequences."""
    from .qsa import IDX_BLOCK, IDX_DIM, IDX_N_HEAD, IndexerState

    pool = KvPool(0, 1, N_KV, HD, 4)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(8)
    n_blocks = 8192
    for n_seqs, rows_per_seq in ((1, 1), (32, 1), (8, 256)):
        rows = n_seqs * rows_per_seq
        idx = IndexerState(pool, n_seqs, n_blocks * IDX_BLOCK)
        idx.pooled.copy_(torch.randn(idx.pooled.shape, generator=gen, device="cuda"))
        q = torch.randn((rows, IDX_N_HEAD, IDX_DIM), generator=gen, device="cuda")
        pos0 = dev_u32(np.full(n_seqs, IDX_BLOCK * n_blocks - rows_per_seq))
        us = timed(lambda: idx.score(q, pos0, rows_per_seq, n_blocks), iters)
        us_graph = timed_graph(lambda: idx.score(q, pos0, rows_per_seq, n_blocks), iters)
        pool.check()
        # every pooled key once per sequence (the rows of a sequence share them), the queries, the scores
        nbytes = n_seqs * n_blocks * IDX_DIM * 4 + rows * IDX_N_HEAD * IDX_DIM * 4 + rows * n_blocks * 4
        flops = 2 * rows * IDX_N_HEAD * n_blocks * IDX_DIM
        emit(op="idx_score", case=f"{rows} row(s) x {n_blocks} pooled keys, {IDX_N_HEAD} index heads of {IDX_DIM}", units=rows,
             bytes=nbytes, flops=flops, us=us, us_graph=us_graph, gbps=nbytes / us_graph / 1e3, tflops=flops / us_graph / 1e6, iters=iters)
    n_seqs, tokens, max_pos = 8, 256, 32768
    idx = IndexerState(pool, n_seqs, max_pos)
    raw = torch.randn((n_seqs, tokens, IDX_DIM), generator=gen, device="cuda")
    gamma = torch.ones(IDX_DIM, device="cuda")
    half = 32
    ang = torch.arange(max_pos, device="cuda", dtype=torch.float64)[:, None] * (1e7 ** (-torch.arange(half, device="cuda", dtype=torch.float64) / half))[None, :]
    table = torch.stack([ang.cos(), ang.sin()], dim=-1).reshape(max_pos, 2 * half).float().contiguous()
    pos0 = dev_u32(np.full(n_seqs, 16384))
    us = timed(lambda: idx.append(raw, pos0, 16384 + tokens, gamma, table, 2 * half), iters)
    us_graph = timed_graph(lambda: idx.append(raw, pos0, 16384 + tokens, gamma, table, 2 * half), iters)
    pool.check()
    nbytes = n_seqs * tokens * IDX_DIM * 4 + n_seqs * (tokens // IDX_BLOCK) * IDX_DIM * 4
    emit(op="idx_pool+idx_tail", case=f"{n_seqs} sequences x {tokens}-token chunk: RMSNorm + rotary + mean of every completed 4-cell block, tail stored",
         units=n_seqs * tokens, bytes=nbytes, us=us, us_graph=us_graph, gbps=nbytes / us_graph / 1e3, iters=iters)
    pool.release()


def bench_qsa_chain(iters: int):
    """What a selected-block (QSA) layer does per decode token behind the query: indexer scores over the pooled keys,
    top-k selection, attention over the selected blocks (Qsa::forward, qsa/mod.rs:1618-1641) - the three calls in
    a row, one query row per sequence at position ~32 k (8192 pooled keys, 512 blocks selected + the row's own),
    24 query heads over 2 kv heads; one sequence and a batch of 32."""
    from .qsa import IDX_BLOCK, IDX_DIM, IDX_N_HEAD, IndexerState, sparse_attend, topk_blocks

    n_head, ctx = 24, 32768
    n_blocks = ctx // IDX_BLOCK
    for n_seqs in (1, 32):
        pages = ctx // 16
        pool = KvPool(0, 1, N_KV, HD, n_seqs * pages)
        tables = dev_u32(synth.permutation(13, n_seqs * pages).reshape(n_seqs, pages))
        gen = torch.Generator(device="cuda")
        gen.manual_seed(12)
        idx = IndexerState(pool, n_seqs, ctx)
        idx.pooled.copy_(torch.randn(idx.pooled.shape, generator=gen, device="cuda"))
        qi = torch.randn((n_seqs, IDX_N_HEAD, IDX_DIM), generator=gen, device="cuda")
        q = torch.randn((n_seqs, n_head, HD), generator=gen, device="cuda")
        out = torch.empty((n_seqs, n_head, HD), device="cuda")
        pos0 = dev_u32(np.full(n_seqs, ctx - 1))

        def chain():
            scores = idx.score(qi, pos0, 1, n_blocks)
            ids, counts = topk_blocks(pool, scores, pos0, 1)
            sparse_attend(pool, 0, q, n_head, tables, pos0, 1, ids, counts, ctx, out)

        us = timed(chain, iters)
        us_graph = timed_graph(chain, iters)
        pool.check()
        emit(op="qsa_decode_chain", case=f"{n_seqs} sequence(s): idx_score over {n_blocks} pooled keys -> top 512 + own block -> attention over "
             f"the selected cells, {n_head}q/{N_KV}kv hd{HD}, 1 layer", units=n_seqs, us=us, us_graph=us_graph, iters=iters)
        pool.release()


def bench_movers(iters: int):
    n_layers, n_pages = 12, 4096
    pool = KvPool(0, n_layers, N_KV, HD, n_pages)
    ids = pool.alloc(n_pages)
    perm = synth.permutation(9, n_pages)
    # gather: 8192 cells of one sequence through a scattered table
    table = dev_u32(perm[:512])
    k_out, v_out = pool.gather(0, table, 8192)

    def gather():
        _lib.call("brc_page_gather", pool.handle, 0, _ptr(table), 512, 8192, _ptr(k_out), _ptr(v_out), _stream_ptr())

    us = timed(gather, iters)
    us_graph = timed_graph(gather, iters)
    nbytes = 2 * 8192 * N_KV * HD * 2 * 2
    emit(op="page_gather", case="8192 cells of one sequence, 1 layer, K and V", units=512, bytes=nbytes, us=us, us_graph=us_graph,
         gbps=nbytes / us_graph / 1e3, iters=iters)
    # copy: 1024 pages, all 12 layers, K and V
    src, dst = dev_u32(perm[:1024]), dev_u32(perm[1024:2048])

    def copy():
        _lib.call("brc_page_copy", pool.handle, _ptr(src), _ptr(dst), 1024, _stream_ptr())

    us = timed(copy, iters)
    nbytes = 2 * 1024 * n_layers * 2 * pool.half_page_bytes
    emit(op="page_copy", case="1024 pages x 12 layers, K and V (read + write)", units=1024, bytes=nbytes, us=us,
         gbps=nbytes / us / 1e3, iters=iters)
    # tiering: demote / promote 512 pages (all layers) on the tier's side stream
    L = _lib.load()
    tier = C.c_void_p()
    _lib.call("brc_tier_create", pool.handle, 600, C.byref(tier))
    n = 512
    pages = np.ascontiguousarray(ids[:n], np.uint32)
    slots = np.zeros(n, np.uint32)
    back = np.zeros(n, np.uint32)
    U32P = C.POINTER(C.c_uint32)
    d_us, p_us = [], []
    for _ in range(max(2, iters // 4)):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        torch.cuda.synchronize()
        import time
        t0 = time.perf_counter()
        _lib.call("brc_tier_demote", tier, pages.ctypes.data_as(U32P), n, slots.ctypes.data_as(U32P), None)
        _lib.call("brc_tier_sync", tier)
        t1 = time.perf_counter()
        _lib.call("brc_tier_promote", tier, slots.ctypes.data_as(U32P), n, back.ctypes.data_as(U32P))
        _lib.call("brc_tier_sync", tier)
        t2 = time.perf_counter()
        pages = back.copy()
        d_us.append((t1 - t0) * 1e6)
        p_us.append((t2 - t1) * 1e6)
    nbytes = n * 2 * n_layers * pool.half_page_bytes
    emit(op="tier_demote", case=f"{n} pages x 12 layers HBM -> pinned host (wall clock incl. issue)", units=n, bytes=nbytes,
         us=min(d_us), gbps=nbytes / min(d_us) / 1e3, iters=len(d_us))
    emit(op="tier_promote", case=f"{n} pages x 12 layers pinned host -> HBM (wall clock incl. issue)", units=n, bytes=nbytes,
         us=min(p_us), gbps=nbytes / min(p_us) / 1e3, iters=len(p_us))
    _lib.call("brc_tier_destroy", tier)
    pool.release()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "prefill", "prepare", "sparse", "topk", "indexer", "chain", "movers"])
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_ops needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(0)
    if a.op in ("all", "prefill"):
        bench_prefill(a.iters, 4096)
        bench_prefill(a.iters, 4088)   # last prefix page partial: forked copy-on-write per sequence
    if a.op in ("all", "prepare"):
        bench_prepare(a.iters)
    if a.op in ("all", "sparse"):
        bench_sparse(a.iters)
    if a.op in ("all", "topk"):
        bench_topk(a.iters)
    if a.op in ("all", "indexer"):
        bench_indexer(a.iters)
    if a.op in ("all", "chain"):
        bench_qsa_chain(a.iters)
    if a.op in ("all", "movers"):
        bench_movers(a.iters)


if __name__ == "__main__":
    main()
