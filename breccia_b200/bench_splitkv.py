"""Benchmark of the long-context single-stream workload: one sequence of 131 072 cells, 12 layers, decode attention split along
the KV length over the GPUs of one box, partials merged over NVLink.

    python -m breccia_b200.bench_splitkv                                   # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m breccia_b200.bench_splitkv --steps 50                          # N GPUs, one rank each

A step = one decode token: in each layer, local split-KV attention over this rank's cells, exchange of
the (acc, m, l) partials (all-gather, 16 512 B per rank per layer), merge.  Strong scaling: the total
work is fixed.  Time = CUDA events around the timed steps, max over ranks.  One JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from . import _lib, synth
from ._lib import DTYPE_F32
from .qsa import KvPool, _ptr, _stream_ptr
from .splitkv import SplitKvDecode, kv_range

N_LAYERS, N_HEAD, N_KV, HD = 12, 16, 2, 256


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--graph", action="store_true", help="replay the step from a CUDA graph instead of launching every call from Python")
    ap.add_argument("--per-layer", action="store_true",
                    help="one attention call per layer, each waiting for the one before (a model's dependency chain); the "
                         "default launches the layers of a step together, as the batched decode benchmark does")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="p2p: one kernel stores the partials to the peers and merges; nccl: all-gather + merge kernel")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench_splitkv needs CUDA devices: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    b, e = kv_range(rank, world, a.tokens)
    n_local = e - b
    n_pages = (n_local + 15) // 16
    pool = KvPool(local, N_LAYERS, N_KV, HD, n_pages + 8)
    table = synth.permutation(100 + rank, n_pages + 8)[:n_pages]
    split = SplitKvDecode(pool, N_HEAD, table, n_local, exchange=a.exchange, max_layers=N_LAYERS)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    for layer in range(N_LAYERS):   # fill through the append kernel
        ks = torch.randn((n_local, N_KV * HD), generator=gen, device=dev) * 0.5
        vs = torch.randn((n_local, N_KV * HD), generator=gen, device=dev) * 0.5
        _lib.call("brc_kv_append", pool.handle, layer, _ptr(split.batch.block_tables), split.batch.table_stride, _ptr(zero), 1,
                  n_local, None, n_local, n_local, _ptr(ks), _ptr(vs), DTYPE_F32, _stream_ptr())
        torch.cuda.synchronize()
    gq = torch.Generator(device=dev)
    gq.manual_seed(99)   # the query is the same on every rank
    q = torch.randn((N_LAYERS, 1, N_HEAD, HD), generator=gq, device=dev).half()
    out = torch.empty((N_LAYERS, 1, N_HEAD, HD), dtype=torch.float32, device=dev)

    def step():
        if a.per_layer or a.exchange == "nccl":
            for layer in range(N_LAYERS):
                split.attend(layer, q[layer], out[layer])
        else:
            split.step(q, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(a.warmup, 3)):
        step()
    barrier()
    # The step is launch-bound from Python (36 small calls); capture it once in a CUDA graph (the
    # library allocates nothing in a launch and NCCL collectives are capturable) and replay it.
    graph = None
    if a.graph:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        run = graph.replay
    else:
        run = step
    for _ in range(3):
        run()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    pool.check()
    ms_step = ms / a.steps
    kv_bytes = a.tokens * N_KV * HD * 2 * 2 * N_LAYERS
    if rank == 0:
        print(json.dumps({"metric": "splitkv_decode_tok_per_s", "value": 1e3 / ms_step, "unit": "tok/s", "n_gpus": world,
                          "steps": a.steps, "ms_per_step": ms_step, "scaling": "strong", "higher_is_better": True, "cuda_graph": bool(a.graph),
                          "layers": "one call each, in order" if (a.per_layer or a.exchange == "nccl") else "launched together (brc_splitkv_step)",
                          "kv_gb_per_s": kv_bytes / (ms_step * 1e-3) / 1e9, "us_per_layer": ms_step * 1e3 / N_LAYERS,
                          "exchange": ("stores of 16512 B per peer per layer into peer memory + flags + merge, one kernel (brc_splitkv_attend)"
                                       if a.exchange == "p2p" else "ncclAllGather of 16512 B per rank per layer + brc_decode_combine"),
                          "config": {"workload": f"1 sequence x {a.tokens} cells, 12 layers, GQA 16q/2kv, head_dim 256, "
                                                 f"f16 KV, KV range split over {world} GPU(s)"}}), flush=True)
    split.close()
    del run, graph   # a captured graph that holds NCCL nodes must go before the communicator does
    torch.cuda.synchronize()
    pool.release()
    if world > 1:
        if a.graph and a.exchange == "nccl":
            # tearing the communicator down after a capture has been seen to block: leave at once instead
            import sys
            sys.stdout.flush()
            os._exit(0)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
