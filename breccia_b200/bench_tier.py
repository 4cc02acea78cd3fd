"""Benchmark of the tiered-paging churn workload: 128 decoding sequences, context lengths uniform
in [1024, 16384] (seeded), 12 layers, GQA 16q/2kv, head_dim 256, f16 KV, the HBM page pool capped at
60 % of the total need, the rest of the pages in pinned host memory.

    python -m breccia_b200.bench_tier [--steps 20] [--warmup 3] [--seqs 128]

The access pattern (seeded, stated here because the configuration leaves it open): a window of
`--window` sequences slides by `--slide` sequences per step over a seeded permutation of the
sequences; the window at step t is what step t wants to decode.  In every step
  * the sequences of the window whose pages are all in HBM decode one token (brc_decode_step: append +
    attention in all 12 layers) on the main stream, after a fence on the tier's copies issued so far;
  * meanwhile, on the tier's two side streams (one per direction), 10 % of the not-resident pages that the NEXT step's window
    needs are promoted (in window order, so sequences complete one after another), and as many pages
    are demoted first to make room: least-recently-decoded sequences outside both windows give up
    pages from their tail.
Reported: decode tok/s over the decoded sequences, host<->device GB/s of the paging traffic over the
timed steps, and the box's pinned cudaMemcpyAsync rate in each direction measured in the same run (the
roofline of the copies).  Time = CUDA events on the main stream (which fences on the side stream's
copies every step and once more at the end).  One JSON line.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math

import numpy as np
import torch

from . import _lib, synth
from ._lib import DTYPE_F16, DTYPE_F32
from .qsa import KvPool, _ptr, _stream_ptr

N_LAYERS, N_HEAD, N_KV, HD, PAGE = 12, 16, 2, 256, 16
U32P = C.POINTER(C.c_uint32)


def u32p(a: np.ndarray):
    return a.ctypes.data_as(U32P)


def pcie_peak(nbytes: int = 512 << 20) -> dict:
    """Pinned cudaMemcpyAsync rates in GB/s (best of 4): each direction alone, and both at once on two
    streams (what a link that carries promotions and demotions together can give per direction)."""
    host_in, host_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev_in, dev_out = torch.empty(nbytes, dtype=torch.uint8, device="cuda"), torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def run(do_in: bool, do_out: bool) -> tuple[float, float]:
        best_in = best_out = 0.0
        for _ in range(4):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            torch.cuda.synchronize()
            if do_in:
                with torch.cuda.stream(s_in):
                    ev[0].record()
                    dev_in.copy_(host_in, non_blocking=True)
                    ev[1].record()
            if do_out:
                with torch.cuda.stream(s_out):
                    ev[2].record()
                    host_out.copy_(dev_out, non_blocking=True)
                    ev[3].record()
            torch.cuda.synchronize()
            if do_in:
                best_in = max(best_in, nbytes / (ev[0].elapsed_time(ev[1]) * 1e-3) / 1e9)
            if do_out:
                best_out = max(best_out, nbytes / (ev[2].elapsed_time(ev[3]) * 1e-3) / 1e9)
        return best_in, best_out

    h2d, _ = run(True, False)
    _, d2h = run(False, True)
    h2d_both, d2h_both = run(True, True)
    return {"h2d": h2d, "d2h": d2h, "h2d_while_d2h": h2d_both, "d2h_while_h2d": d2h_both}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=128)
    ap.add_argument("--min-len", type=int, default=1024)
    ap.add_argument("--max-len", type=int, default=16384)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hbm-frac", type=float, default=0.60)
    ap.add_argument("--window", type=int, default=64)
    ap.add_argument("--slide", type=int, default=2)
    ap.add_argument("--promote-frac", type=float, default=0.10)
    ap.add_argument("--seed", type=int, default=20261125)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_tier needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(0)
    n, total_steps = a.seqs, a.steps + a.warmup
    lens = synth.uniform_ints(a.seed, n, a.min_len, a.max_len).astype(np.int64)
    stride = (a.max_len + total_steps + PAGE) // PAGE + 1
    pages_of = ((lens + total_steps + PAGE) // PAGE).astype(np.int64)      # room for the tokens the run appends
    need = int(pages_of.sum())
    reserve = int(pages_of.max()) + 64                                     # free pages kept for pages in transit
    hbm_pages = int(a.hbm_frac * need)
    host_pages = need - (hbm_pages - reserve) + 2048
    pool = KvPool(0, N_LAYERS, N_KV, HD, hbm_pages)
    pool.zero()
    slot_bytes = 2 * N_LAYERS * pool.half_page_bytes
    tier = C.c_void_p()
    _lib.call("brc_tier_create", pool.handle, host_pages, C.byref(tier))
    perm = synth.permutation(a.seed + 1, n).astype(np.int64)

    # ---- initial placement, in the order of the access pattern: HBM until the cap, then the host tier
    loc = []                       # per sequence: int64 per page; >= 0 HBM page id, < 0 -(slot + 1)
    used = 0
    for s in range(n):
        loc.append(None)
    for s in perm:
        ids = pool.alloc(int(pages_of[s])).astype(np.uint32)
        if used + ids.size <= hbm_pages - reserve:
            used += ids.size
            loc[s] = ids.astype(np.int64)
        else:
            slots = np.zeros(ids.size, np.uint32)
            _lib.call("brc_tier_demote", tier, u32p(ids), ids.size, u32p(slots), None)
            loc[s] = -(slots.astype(np.int64) + 1)
    _lib.call("brc_tier_sync", tier)
    last_decoded = np.full(n, -1, np.int64)
    peaks = pcie_peak()

    dev = "cuda:0"
    gen = torch.Generator(device=dev)
    gen.manual_seed(a.seed)
    W = a.window
    q = (torch.randn((N_LAYERS, W, N_HEAD, HD), generator=gen, device=dev)).half()
    k_new = torch.randn((N_LAYERS, W, N_KV * HD), generator=gen, device=dev) * 0.5
    v_new = torch.randn((N_LAYERS, W, N_KV * HD), generator=gen, device=dev) * 0.5
    out = torch.empty((N_LAYERS, W, N_HEAD, HD), dtype=torch.float32, device=dev)
    ws_bytes = C.c_uint64()
    _lib.call("brc_decode_workspace_bytes", pool.handle, W, N_HEAD, C.byref(ws_bytes))
    scratch = torch.empty(N_LAYERS * ws_bytes.value, dtype=torch.uint8, device=dev)
    # two sets of per-step inputs in pinned memory: the host fills one while the device reads the other
    bt_host = [torch.zeros((W, stride), dtype=torch.int32).pin_memory() for _ in range(2)]
    len_host = [torch.zeros(W, dtype=torch.int32).pin_memory() for _ in range(2)]
    bt_dev = [torch.zeros((W, stride), dtype=torch.int32, device=dev) for _ in range(2)]
    len_dev = [torch.zeros(W, dtype=torch.int32, device=dev) for _ in range(2)]
    pos_dev = torch.zeros(W, dtype=torch.int32, device=dev)
    copied = [torch.cuda.Event() for _ in range(2)]

    def window(t):
        return [int(perm[(a.slide * t + j) % n]) for j in range(W)]

    decoded_tokens = promoted = demoted = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    main = _stream_ptr()
    for t in range(total_steps):
        if t == a.warmup:
            _lib.call("brc_tier_fence", tier, main)
            e0.record()
            decoded_tokens = promoted = demoted = 0
        cur, nxt = window(t), window(t + 1)
        # ---- main stream: decode what is resident of this step's window
        dec = [s for s in cur if loc[s].min() >= 0]
        b = t % 2
        copied[b].synchronize()        # the copies that read this pinned pair two steps ago
        for i, s in enumerate(dec):
            bt_host[b][i, :loc[s].size] = torch.from_numpy(loc[s].astype(np.int32))
            len_host[b][i] = int(lens[s])
        _lib.call("brc_tier_fence", tier, main)
        if dec:
            bt_dev[b].copy_(bt_host[b], non_blocking=True)
            len_dev[b].copy_(len_host[b], non_blocking=True)
            copied[b].record()
            for s in dec:
                lens[s] += 1
                last_decoded[s] = t
            max_after = int(max(lens[s] for s in dec))
            _lib.call("brc_decode_step", pool.handle, 0, N_LAYERS, _ptr(bt_dev[b]), stride, _ptr(len_dev[b]), _ptr(pos_dev), len(dec),
                      max_after, _ptr(q), DTYPE_F16, q.stride(0) * 2, N_HEAD, _ptr(k_new), _ptr(v_new), DTYPE_F32,
                      k_new.stride(0) * 4, None, 0, 0, 1.0 / math.sqrt(HD), _ptr(out), out.stride(0) * 4, _ptr(scratch),
                      scratch.numel(), main)
            decoded_tokens += len(dec)
        # ---- side stream: 10 % of what the next window misses comes in, as much goes out first
        missing = [(s, i) for s in nxt for i in np.nonzero(loc[s] < 0)[0]]
        k = min(int(math.ceil(a.promote_frac * len(missing))), len(missing))
        if k:
            pinned = set(cur) | set(nxt)
            free_now = pool.free_count()
            want_out = max(0, k - (free_now - 64))
            victims = []
            for s in sorted((s for s in range(n) if s not in pinned), key=lambda s: last_decoded[s]):
                if len(victims) >= want_out:
                    break
                res = np.nonzero(loc[s] >= 0)[0]
                take = res[::-1][: want_out - len(victims)]          # from the tail of the sequence
                victims.extend((s, int(i)) for i in take)
            if len(victims) < want_out:
                k = max(0, k - (want_out - len(victims)))
            if victims:
                ids = np.array([loc[s][i] for s, i in victims], np.uint32)
                slots = np.zeros(ids.size, np.uint32)
                _lib.call("brc_tier_demote", tier, u32p(ids), ids.size, u32p(slots), None)
                for (s, i), sl in zip(victims, slots):
                    loc[s][i] = -(int(sl) + 1)
                demoted += ids.size
            if k:
                take = missing[:k]
                slots = np.array([-(loc[s][i]) - 1 for s, i in take], np.uint32)
                ids = np.zeros(k, np.uint32)
                _lib.call("brc_tier_promote", tier, u32p(slots), k, u32p(ids))
                for (s, i), pg in zip(take, ids):
                    loc[s][i] = int(pg)
                promoted += k
    _lib.call("brc_tier_fence", tier, main)
    e1.record()
    torch.cuda.synchronize()
    pool.check()
    ms = e0.elapsed_time(e1)
    sec = ms * 1e-3
    print(json.dumps({
        "metric": "tiered_decode_tok_per_s", "value": decoded_tokens / sec, "unit": "tok/s", "n_gpus": 1, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": ms / a.steps, "higher_is_better": True, "data": "synthetic", "dtype": "f16",
        "decoded_sequences_per_step": decoded_tokens / a.steps,
        "h2d_gb_per_s": promoted * slot_bytes / sec / 1e9, "d2h_gb_per_s": demoted * slot_bytes / sec / 1e9,
        "pages_promoted_per_step": promoted / a.steps, "pages_demoted_per_step": demoted / a.steps,
        "pinned_copy_peak_gb_per_s": peaks,
        "h2d_frac_of_copy_peak": promoted * slot_bytes / sec / 1e9 / peaks["h2d"],
        "d2h_frac_of_copy_peak": demoted * slot_bytes / sec / 1e9 / peaks["d2h"],
        "h2d_frac_of_two_way_peak": promoted * slot_bytes / sec / 1e9 / peaks["h2d_while_d2h"],
        "d2h_frac_of_two_way_peak": demoted * slot_bytes / sec / 1e9 / peaks["d2h_while_h2d"],
        "config": {"workload": f"tiering churn: {n} sequences, context uniform in [{a.min_len}, {a.max_len}], 12 layers, GQA 16q/2kv, "
                               f"head_dim 256, f16 KV; HBM pool {hbm_pages} pages = {a.hbm_frac:.0%} of the {need} needed, "
                               f"{host_pages} pinned host slots of {slot_bytes} B; window {W} sliding by {a.slide} per step, "
                               f"{a.promote_frac:.0%} of the next window's missing pages promoted per step", "seed": a.seed}}),
          flush=True)
    _lib.call("brc_tier_destroy", tier)
    pool.release()


if __name__ == "__main__":
    main()
