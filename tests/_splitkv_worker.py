"""Worker of tests/test_splitkv_multigpu.py (launched with torch.distributed.run, one rank per GPU):
one long sequence split along its KV length over the ranks; every rank must obtain the attention
output of the whole sequence.  Rank 0 checks it against the oracle.  Prints one line and exits 0 / 1."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from breccia_b200 import synth  # noqa: E402
from breccia_b200.qsa import DecodeBatch, KvPool  # noqa: E402
from breccia_b200.splitkv import SplitKvDecode, kv_range  # noqa: E402


def _step_same_layer(split, q3, out3):
    """brc_splitkv_step over the three layers of the worker's pool (which hold the same pages), so the
    three outputs must equal the single-layer result (within 2e-6: one launch over three layers cuts its
    shares differently from a launch over one, so the same sums are taken in another order)."""
    split.step(q3, out3)


def main():
    n_tokens = int(sys.argv[1]) if len(sys.argv) > 1 else 5000
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n_head, n_kv, hd = 16, 2, 256
    # the whole sequence's K/V (logical order), the same on every rank
    k = oracle.f32_to_f16_bits_np(synth.normal(1, n_tokens * n_kv * hd, 0.5)).reshape(n_tokens, n_kv, hd)
    v = oracle.f32_to_f16_bits_np(synth.normal(2, n_tokens * n_kv * hd, 0.5)).reshape(n_tokens, n_kv, hd)
    q = oracle.to_f16(synth.normal(3, n_head * hd)).reshape(1, n_head, hd)
    b, e = kv_range(rank, world, n_tokens)
    n_local = e - b
    n_pages = max((n_local + 15) // 16, 1)
    pool = KvPool(local, 3, n_kv, hd, n_pages + 3)
    table = synth.permutation(10 + rank, n_pages + 3)[:n_pages]
    kp = np.zeros((n_pages + 3, n_kv, 16, hd), np.uint16)
    vp = np.zeros_like(kp)
    for c in range(n_local):
        kp[table[c // 16], :, c % 16, :] = k[b + c]
        vp[table[c // 16], :, c % 16, :] = v[b + c]
    for layer in range(3):
        pool.write(0, layer, kp)
        pool.write(1, layer, vp)
    qd = torch.from_numpy(q).cuda().half()
    ok = True
    want = None
    if rank == 0:
        kf = oracle.f16_bits_to_f32(k)
        vf = oracle.f16_bits_to_f32(v)
        want = oracle.attend(q[0], kf, vf, np.arange(n_tokens, dtype=np.uint32), n_tokens - 1, n_head, n_kv, hd)
    for exchange in ("p2p", "nccl"):
        split = SplitKvDecode(pool, n_head, table, n_local, exchange=exchange)
        out = torch.full((1, n_head, hd), float("nan"), device="cuda")
        for _ in range(11):   # more calls than the receive buffer has banks
            split.attend(0, qd, out)
        torch.cuda.synchronize()
        pool.check()
        got = out.cpu().numpy()[0]
        ref = out.clone()
        dist.broadcast(ref, 0)   # every rank must hold the same answer
        same = bool(torch.equal(ref, out))
        ok = ok and same
        if rank == 0:
            err = float(np.abs(got - want).max())
            ok = ok and bool(np.isfinite(got).all()) and err <= 2e-3
            print(f"splitkv {exchange} world {world} tokens {n_tokens}: max_abs {err:.2e} identical_on_all_ranks {same}", flush=True)
        if exchange == "p2p":
            # the step form over 3 "layers" (the pool has one: the same layer three times) gives three copies
            step = SplitKvDecode(pool, n_head, table, n_local, max_layers=3)
            q3 = qd.unsqueeze(0).repeat(3, 1, 1, 1).contiguous()
            out3 = torch.full((3, 1, n_head, hd), float("nan"), device="cuda")
            _step_same_layer(step, q3, out3)
            torch.cuda.synchronize()
            pool.check()
            step_err = max(float((out3[i] - out).abs().max()) for i in range(3))
            ref3 = out3.clone()
            dist.broadcast(ref3, 0)
            ok = ok and step_err <= 2e-6 and bool(torch.equal(ref3, out3))
            if rank == 0:
                print(f"splitkv step over 3 layers, world {world}: max_abs vs single-layer call {step_err:.2e}", flush=True)
            step.close()
            # two calls recorded in a CUDA graph and replayed more often than the receive buffer has banks: the call
            # count lives on the device, so every replay uses the next bank on every rank
            out_g = torch.full((2, 1, n_head, hd), float("nan"), device="cuda")
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                split.attend(0, qd, out_g[0])
                split.attend(0, qd, out_g[1])
            for _ in range(7):
                graph.replay()
            torch.cuda.synchronize()
            pool.check()
            graph_same = bool(torch.equal(out_g[0], out)) and bool(torch.equal(out_g[1], out))
            ok = ok and graph_same
            if rank == 0:
                print(f"splitkv two calls in a CUDA graph, 7 replays, world {world}: equal to the plain call {graph_same}", flush=True)
        split.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    pool.release()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
