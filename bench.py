#!/usr/bin/env python
"""Benchmark of the paged KV decode hot path.

    python bench.py --gpus N --steps K --warmup W            # this library on N GPUs (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores

Headline (`value`): the batched-decode workload.  A step = one decode step of the whole batch: in each of
the 12 attention layers, append one token's K/V per sequence through the block tables, then paged GQA
decode attention over the whole cache - ONE kernel launch per step (brc_decode_step).  Sequences are
independent, so N GPUs each own 32 sequences of the SAME lengths and their own pool (weak scaling, no
data-path collective); torch.distributed is used only for the barrier and the max-over-ranks of the
device time.  Rank 0 prints ONE JSON line, which also carries

    layer_by_layer  the same step as a model's dependent chain sees it (append + attention call per layer);
                    layer_by_layer_fused: one fused launch per layer
    strong          the same 32 sequences dealt round-robin by descending length over the N GPUs
    splitkv         the long-context workload: ONE sequence of 131 072 cells whose KV range is split over the
                    N GPUs, partials stored into the peers' memory by the attention kernel itself and merged there
                    (the only path that communicates), with the output checked against the CPU oracle
    fixed8k         (N = 1) the 32 x 8192 variant of the batched workload
    q8v             (N = 1) the batched workload on a pool whose V page bodies are q8_0
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_LAYERS, N_HEAD, N_KV, HD, PAGE = 12, 16, 2, 256, 16
N_SEQS = 32
TOKEN_BYTES = N_KV * HD * 2 * 2  # K + V of one cell of one layer = 2048 B
SPLITKV_TOKENS = 131072


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "fixed8k"],
                    help="headline workload. cfg2: lengths uniform in [512, 8192]; fixed8k: every sequence at 8192")
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-headline", action="store_true",
                    help="skip the strong / splitkv / fixed8k sub-benchmarks (small profiler captures)")
    ap.add_argument("--only-q8v", action="store_true",
                    help="run the q8_0 V variant of the batched workload alone and print its object (small profiler captures)")
    ap.add_argument("--layers", type=int, default=12,
                    help="attention layers per step (12 = the full workload; fewer only for small profiler captures)")
    return ap.parse_args()


def workload_lengths(kind: str, seed: int) -> np.ndarray:
    from breccia_b200 import synth

    if kind == "fixed8k":
        return np.full(N_SEQS, 8192, np.int64)
    return synth.uniform_ints(seed, N_SEQS, 512, 8192)


def workload_name(kind: str) -> str:
    if kind == "fixed8k":
        return "batched decode: 32 sequences x 8192 context, 12 layers, GQA 16q/2kv, head_dim 256, f16 KV, 16-token pages"
    return ("batched decode: 32 sequences, context uniform in [512, 8192] (seeded), 12 layers, GQA 16q/2kv, "
            "head_dim 256, f16 KV, 16-token pages scattered in a pool of 1.25x need")


def workload_config(kind: str, lens0: np.ndarray, seed: int) -> dict:
    """The `config` object: the same keys and values in both arms."""
    return {"workload": workload_name(kind), "n_seqs_per_gpu": int(lens0.size),
            "sum_context_tokens_per_gpu": int(lens0.sum()), "layers": N_LAYERS, "seed": seed}


def algorithmic_bytes_per_layer(lens: np.ndarray) -> float:
    """Bytes one layer's decode attention must move: every cached K/V byte once, q in, out out, the
    block-table entries."""
    return float(lens.sum() * TOKEN_BYTES + lens.size * (N_HEAD * HD * 2 + N_HEAD * HD * 4)
                 + ((lens + PAGE - 1) // PAGE).sum() * 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def recorded_traffic():
    """DRAM bytes per cached byte of the decode kernel from the committed ncu summary (traffic grows in
    proportion to the pages streamed)."""
    path = os.path.join(ROOT, "profiles", "decode_partial_traffic.json")
    if not os.path.exists(path):
        return None
    try:
        return json.load(open(path))
    except Exception:
        return None


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            time.sleep(0.3)   # the first sample takes a while to appear
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# native arm
# ----------------------------------------------------------------------------------------------
class Ctx:
    """Rank, device and the timing helpers shared by the phases of the native arm."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus != self.world and self.world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, n_warm: int, n_steps: int, before=None) -> float:
        """ms for exactly n_steps calls of fn after n_warm untimed ones: CUDA events on the launching
        stream, a barrier and a device synchronisation on both sides, the max over ranks."""
        torch = self.torch
        if before:
            before()
        for _ in range(n_warm):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))


def make_batch(ctx, lens0, seed, extra_tokens, n_layers=None, v_q8=False):
    """Pool + block tables + lengths of a batch, the cache filled through the append kernel itself
    (f32 sources ~ N(0, 0.5^2), seeded on the device)."""
    import torch

    from breccia_b200 import synth
    from breccia_b200._lib import DTYPE_F16, DTYPE_F32, call
    from breccia_b200.qsa import DecodeBatch, KvPool, _ptr, _stream_ptr

    n_layers = n_layers or N_LAYERS
    tables, n_pool = synth.scattered_tables(seed + 7 + ctx.rank, lens0, page_tokens=PAGE, pool_factor=1.25, extra_tokens=extra_tokens)
    pool = KvPool(ctx.local, n_layers, N_KV, HD, n_pool, v_q8=v_q8)
    batch = DecodeBatch(pool, N_HEAD, tables, lens0, q_dtype=DTYPE_F16)
    gen = torch.Generator(device=ctx.dev)
    gen.manual_seed(seed + ctx.rank)
    n = int(lens0.size)
    cu = np.concatenate([[0], np.cumsum(lens0)]).astype(np.int32)
    cu_dev = torch.as_tensor(cu, device=ctx.dev)
    zeros = torch.zeros(n, dtype=torch.int32, device=ctx.dev)
    total = int(cu[-1])
    for layer in range(n_layers):
        k_src = torch.randn((total, N_KV * HD), generator=gen, device=ctx.dev) * 0.5
        v_src = torch.randn((total, N_KV * HD), generator=gen, device=ctx.dev) * 0.5
        call("brc_kv_append", pool.handle, layer, _ptr(batch.block_tables), batch.table_stride, _ptr(zeros), n, 0,
             _ptr(cu_dev), total, int(lens0.max()), _ptr(k_src), _ptr(v_src), DTYPE_F32, _stream_ptr())
        torch.cuda.synchronize()
        del k_src, v_src
    pool.check()
    q = torch.randn((n_layers, n, N_HEAD, HD), generator=gen, device=ctx.dev).half()
    k_new = torch.randn((n_layers, n, N_KV * HD), generator=gen, device=ctx.dev) * 0.5
    v_new = torch.randn((n_layers, n, N_KV * HD), generator=gen, device=ctx.dev) * 0.5
    out = torch.empty((n_layers, n, N_HEAD, HD), dtype=torch.float32, device=ctx.dev)
    return pool, batch, q, k_new, v_new, out


def bench_batched(ctx, args, kind, steps, warmup, sampler=None, with_cpu=False, repeats=5, full=True):
    """The batched-decode workload on this rank's own 32 sequences: device-resident value, end to end,
    roofline of the step's kernel, the layer-by-layer forms."""
    import ctypes as C

    import torch

    from breccia_b200._lib import DTYPE_F32, call

    lens0 = workload_lengths(kind, args.seed)
    n_warm = max(warmup, 3)
    pool, batch, q, k_new, v_new, out = make_batch(ctx, lens0, args.seed, extra_tokens=n_warm + steps + 2)
    reset = lambda: batch.reset_lengths(lens0)
    step = lambda: batch.step(q, k_new, v_new, out)
    res = {"lens0": lens0}

    # ---- headline: device-resident inputs, one kernel per step
    if sampler:
        sampler.start()
    ms_total = ctx.timed(step, n_warm, steps, before=reset)
    pool.check()
    ms_step = ms_total / steps
    windows = [ms_step]
    for _ in range(repeats if full else 0):
        windows.append(ctx.timed(step, n_warm, steps, before=reset) / steps)
    res["ms_step"], res["windows"] = ms_step, windows
    lens_mid = lens0 + n_warm + (steps + 1) / 2.0
    res["lens_mid"] = lens_mid

    # ---- the same step as a dependent chain sees it: one append call and one attention call per layer
    def chain():
        batch.begin_step()
        for layer in range(N_LAYERS):
            batch.append(layer, k_new[layer], v_new[layer], DTYPE_F32)
            batch.attend(layer, q[layer], out[layer])

    res["ms_chain"] = ctx.timed(chain, 3, steps, before=reset) / steps if full else None

    # ---- the same chain with the append fused into each layer's attention launch (brc_decode_step_part, one layer
    #      per call): 12 launches and one position kernel per step
    def chain_fused():
        for layer in range(N_LAYERS):
            batch.step_part(layer, 1, q, k_new, v_new, out)

    res["ms_chain_fused"] = ctx.timed(chain_fused, 3, steps, before=reset) / steps if full else None

    # ---- one attention launch alone: CUDA events around every launch of the per-layer calls
    iso_us = None
    if full:
        call("brc_timing_enable", pool.handle, 1)
        reset()
        for _ in range(3):
            chain()
        torch.cuda.synchronize()
        launches, total_ms = C.c_uint32(), C.c_double()
        call("brc_timing_read", pool.handle, 1, C.byref(launches), C.byref(total_ms))   # discard the warm-up launches
        n_iso = min(steps, 10)
        for _ in range(n_iso):
            chain()
        call("brc_timing_read", pool.handle, 1, C.byref(launches), C.byref(total_ms))
        call("brc_timing_enable", pool.handle, 0)
        iso_us = total_ms.value / max(launches.value, 1) * 1e3
        res["iso_launches"] = launches.value
        res["lens_iso"] = lens0 + 3 + (n_iso + 1) / 2.0
    res["iso_us"] = iso_us
    clocks = sampler.stop() if sampler else None
    res["clocks"] = clocks

    # ---- end to end: host (pinned) activations in, attention output back to the host, every step
    q_h, k_h, v_h = q.cpu().pin_memory(), k_new.cpu().pin_memory(), v_new.cpu().pin_memory()
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    staging = batch.host_staging(N_LAYERS)
    # q / k / v either read by the kernels where they lie in pinned host memory or uploaded first, the output
    # either stored by the kernels straight into the pinned host buffer or staged on the device and copied down:
    # which is faster depends on the host, so the modes are timed and the best one is reported
    e2e_modes = {}
    for mode, upload, download in (("q/k/v read and output stored in place by the kernels (pinned host memory, nothing staged)", False, False),
                                   ("q/k/v uploaded, output stored by the kernels into the pinned host buffer", True, False),
                                   ("q/k/v uploaded, output staged on the device and copied down", True, True)):
        e2e_modes[mode] = ctx.timed(lambda: batch.step_host(q_h, k_h, v_h, out_h, staging, upload=upload, download=download), 3, steps, before=reset) / steps
    res["e2e_modes"] = e2e_modes
    res["h2d"] = q_h.numel() * 2 + k_h.numel() * 4 + v_h.numel() * 4
    res["d2h"] = out_h.numel() * 4
    pool.check()

    res["cpu"] = cpu_baseline_sample(pool, batch, q) if with_cpu else None
    pool.release()
    del batch, q, k_new, v_new, out, staging
    torch.cuda.empty_cache()
    return res


def roofline_of(res, peak, peak_src):
    """Roofline object of the step's kernel: ONE launch covers the 12 layers of a step, so its duration is
    the timed region divided by the steps in it (which also charges the step's small position kernel to it)."""
    alg = algorithmic_bytes_per_layer(res["lens_mid"]) * N_LAYERS
    dur_s = res["ms_step"] * 1e-3
    achieved = alg / dur_s / 1e9
    traffic = None
    rec = recorded_traffic()
    if rec:
        traffic = rec["dram_bytes_per_cached_byte"] * float(res["lens_mid"].sum()) * TOKEN_BYTES * N_LAYERS
    roof = {"kernel": "decode_partial_kernel<256,f16 q> (one launch = the 12 layers of a step)", "bound": "hbm",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
            "peak_source": peak_src, "algorithmic_bytes_per_launch": alg, "avg_launch_us": dur_s * 1e6,
            "how": "CUDA events around the timed steps on the launching stream / steps (one attention launch per step)",
            "frac_of_nominal_8tbs": achieved / 8000.0}
    if res.get("iso_us"):
        alg1 = algorithmic_bytes_per_layer(res["lens_iso"])
        iso_s = res["iso_us"] * 1e-6
        roof["isolated_launch"] = {"avg_launch_us": res["iso_us"], "achieved": alg1 / iso_s / 1e9, "frac": alg1 / iso_s / 1e9 / peak,
                                   "algorithmic_bytes_per_launch": alg1, "launches_timed": res["iso_launches"],
                                   "how": "one layer per launch (brc_paged_decode_attn), CUDA events around every launch"}
    return roof


Q8_TOKEN_BYTES = N_KV * HD * 2 + N_KV * (HD // 32) * 36   # K binary16 + V q8_0 of one cell of one layer = 1600 B


def bench_q8v(ctx, args, steps, warmup):
    """The batched workload on a pool whose V page bodies are q8_0 (the reference's VLayout::Q8_0): same lengths, same
    step (fused quantising append + attention in 12 layers, one launch); the roofline counts the bytes actually stored."""
    import torch

    lens0 = workload_lengths("cfg2", args.seed)
    n_warm = max(warmup, 3)
    pool, batch, q, k_new, v_new, out = make_batch(ctx, lens0, args.seed, extra_tokens=n_warm + steps + 2, v_q8=True)
    ms = ctx.timed(lambda: batch.step(q, k_new, v_new, out), n_warm, steps, before=lambda: batch.reset_lengths(lens0)) / steps
    pool.check()
    pool.release()
    del batch, q, k_new, v_new, out
    torch.cuda.empty_cache()
    peak, peak_src = measured_peaks()
    lens_mid = lens0 + n_warm + (steps + 1) / 2.0
    alg = float(lens_mid.sum() * Q8_TOKEN_BYTES + lens0.size * (N_HEAD * HD * 2 + N_HEAD * HD * 4) + ((lens_mid + PAGE - 1) // PAGE).sum() * 4) * N_LAYERS
    achieved = alg / (ms * 1e-3) / 1e9
    return {"workload": workload_name("cfg2") + "; V page bodies q8_0 (36 B per 32 values), K binary16: 1600 B per cached cell and layer",
            "value": N_SEQS / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms,
            "roofline": {"kernel": "decode_partial_kernel<256,f16 q,q8_0 V> (one launch = the 12 layers of a step)", "bound": "hbm",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": alg, "avg_launch_us": ms * 1e3}}


def bench_strong(ctx, args, steps):
    """BASELINE's wording of the batched workload: the SAME 32 sequences dealt round-robin by descending
    length over the N GPUs (strong scaling, no collective)."""
    import torch

    lens_all = workload_lengths("cfg2", args.seed)
    order = np.argsort(-lens_all, kind="stable")
    mine = lens_all[order[ctx.rank::ctx.world]]
    pool, batch, q, k_new, v_new, out = make_batch(ctx, mine, args.seed + 31, extra_tokens=steps + 8)
    ms = ctx.timed(lambda: batch.step(q, k_new, v_new, out), 3, steps, before=lambda: batch.reset_lengths(mine)) / steps
    pool.check()
    pool.release()
    del batch, q, k_new, v_new, out
    torch.cuda.empty_cache()
    peak, _ = measured_peaks()
    kv_bytes = float(lens_all.sum() + lens_all.size * (3 + (steps + 1) / 2.0)) * TOKEN_BYTES * N_LAYERS
    return {"value": N_SEQS / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms, "scaling": "strong",
            "seqs_on_rank0": int(mine.size), "context_tokens_on_rank0": int(mine.sum()),
            "kv_gb_per_s": kv_bytes / (ms * 1e-3) / 1e9, "kv_frac_of_hbm_peak_per_gpu": kv_bytes / (ms * 1e-3) / 1e9 / ctx.world / peak,
            "partition": "32 sequences in all, round-robin by descending length, no collective"}


def bench_splitkv(ctx, args, steps):
    """The long-context workload: one sequence of 131 072 cells, 12 layers, KV range split over the ranks;
    per step ONE launch per rank streams the local cells of all layers, pushes the merged (acc, m, l) of every
    (layer, kv-head group) into every peer's receive buffer and merges what the peers pushed."""
    import ctypes as C

    import torch
    import torch.distributed as dist

    import oracle
    from breccia_b200 import _lib, synth
    from breccia_b200._lib import DTYPE_F16, DTYPE_F32
    from breccia_b200.qsa import DecodeBatch, KvPool, _ptr, _stream_ptr
    from breccia_b200.splitkv import SplitKvDecode, kv_range

    dev = ctx.dev

    def filled(n_local, seed):
        n_pages = (n_local + 15) // 16
        pool = KvPool(ctx.local, N_LAYERS, N_KV, HD, n_pages + 8)
        table = synth.permutation(seed, n_pages + 8)[:n_pages]
        bt = torch.as_tensor(table.astype(np.int32), device=dev)
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        for layer in range(N_LAYERS):
            ks = torch.randn((n_local, N_KV * HD), generator=gen, device=dev) * 0.5
            vs = torch.randn((n_local, N_KV * HD), generator=gen, device=dev) * 0.5
            _lib.call("brc_kv_append", pool.handle, layer, _ptr(bt), bt.numel(), _ptr(zero), 1, n_local, None, n_local, n_local,
                      _ptr(ks), _ptr(vs), DTYPE_F32, _stream_ptr())
            torch.cuda.synchronize()
            del ks, vs
        return pool, table, bt

    b, e = kv_range(ctx.rank, ctx.world, SPLITKV_TOKENS)
    n_local = e - b
    pool, table, bt = filled(n_local, 100 + ctx.rank)
    split = SplitKvDecode(pool, N_HEAD, table, n_local, max_layers=N_LAYERS)
    gq = torch.Generator(device=dev)
    gq.manual_seed(99)   # the query is the same on every rank
    q = torch.randn((N_LAYERS, 1, N_HEAD, HD), generator=gq, device=dev).half()
    out = torch.zeros((N_LAYERS, 1, N_HEAD, HD), dtype=torch.float32, device=dev)
    out_chain = torch.zeros_like(out)

    def chain():
        for layer in range(N_LAYERS):
            split.attend(layer, q[layer], out_chain[layer])

    ms_step = ctx.timed(lambda: split.step(q, out), 3, steps) / steps
    ms_chain = ctx.timed(chain, 3, steps) / steps
    pool.check()
    # the same chain recorded once as a CUDA graph and replayed: one driver call per token instead of twelve library
    # calls, which is what bounds the plain loop once a layer's share of the cells streams in a few microseconds
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    ms_chain_graph = ctx.timed(graph.replay, 3, steps) / steps
    pool.check()

    # ---- this rank's share alone (no exchange): the same launch over the local cells through a group of one
    local_comm = C.c_void_p()
    _lib.call("brc_comm_create", pool.handle, 1, 0, N_LAYERS, N_HEAD, C.byref(local_comm))
    sb = split.batch
    out_local = torch.zeros_like(out)
    local_step = lambda: _lib.call("brc_splitkv_step", local_comm, 0, N_LAYERS, _ptr(q), DTYPE_F16, q.stride(0) * q.element_size(), None, 0,
                                   _ptr(sb.block_tables), sb.table_stride, _ptr(sb.seq_lens), 1, sb.capacity, sb.scale, _ptr(out_local),
                                   _ptr(sb.scratch), sb.scratch.numel(), _stream_ptr())
    ms_local = ctx.timed(local_step, 3, steps) / steps
    _lib.call("brc_comm_destroy", local_comm)

    # ---- parity: layers 0 and 11 of rank 0's output against the CPU oracle over the whole sequence (the ranks'
    #      cells are read back through the page-gather kernel and collected on rank 0)
    check_layers = (0, N_LAYERS - 1)
    max_abs = {}
    for layer in check_layers:
        k_loc, v_loc = pool.gather(layer, bt, n_local)
        if ctx.world > 1:
            ks = [torch.empty_like(k_loc) for _ in range(ctx.world)] if ctx.rank == 0 else None
            vs = [torch.empty_like(v_loc) for _ in range(ctx.world)] if ctx.rank == 0 else None
            dist.gather(k_loc, ks, dst=0)
            dist.gather(v_loc, vs, dst=0)
        else:
            ks, vs = [k_loc], [v_loc]
        if ctx.rank == 0:
            k_all = torch.cat(ks).view(torch.int16).cpu().numpy().view(np.uint16)   # [tokens, n_kv, hd]
            v_all = torch.cat(vs).view(torch.int16).cpu().numpy().view(np.uint16)
            to_pool = lambda x: np.ascontiguousarray(x.reshape(-1, PAGE, N_KV, HD).transpose(0, 2, 1, 3)).reshape(-1)
            ident = np.arange(SPLITKV_TOKENS // PAGE, dtype=np.uint32)[None, :]
            want, _ = oracle.decode_batch(to_pool(k_all), to_pool(v_all), ident, np.array([SPLITKV_TOKENS], np.uint32),
                                          q[layer].float().cpu().numpy(), N_HEAD, N_KV, HD, n_threads=os.cpu_count() or 1)
            max_abs[f"layer{layer}"] = {"step": float(np.abs(out[layer].cpu().numpy() - want).max()),
                                        "layer_by_layer": float(np.abs(out_chain[layer].cpu().numpy() - want).max())}
    same = True
    if ctx.world > 1:   # every rank must hold the same output
        ref = out.clone()
        dist.broadcast(ref, 0)
        flag = torch.tensor([1 if torch.equal(ref, out) else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        same = bool(flag.item())
    split.close()
    pool.release()
    torch.cuda.empty_cache()

    # ---- the whole sequence on ONE GPU in the same run (rank 0), the reference point of the speed-up
    ms_one = ms_step
    if ctx.world > 1:
        if ctx.rank == 0:
            pool1, table1, _ = filled(SPLITKV_TOKENS, 100)
            batch1 = DecodeBatch(pool1, N_HEAD, table1[None, :], [SPLITKV_TOKENS], q_dtype=DTYPE_F16)
            comm1 = C.c_void_p()
            _lib.call("brc_comm_create", pool1.handle, 1, 0, N_LAYERS, N_HEAD, C.byref(comm1))
            one = lambda: _lib.call("brc_splitkv_step", comm1, 0, N_LAYERS, _ptr(q), DTYPE_F16, q.stride(0) * q.element_size(), None, 0,
                                    _ptr(batch1.block_tables), batch1.table_stride, _ptr(batch1.seq_lens), 1, batch1.capacity, batch1.scale,
                                    _ptr(out_local), _ptr(batch1.scratch), batch1.scratch.numel(), _stream_ptr())
            for _ in range(3):
                one()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            ms_one = e0.elapsed_time(e1) / steps
            _lib.call("brc_comm_destroy", comm1)
            pool1.release()
            del batch1
            torch.cuda.empty_cache()
        ctx.barrier()
    peak, _ = measured_peaks()
    kv_bytes = float(SPLITKV_TOKENS) * TOKEN_BYTES * N_LAYERS
    form = lambda ms: {"value": 1e3 / ms, "unit": "tok/s", "ms_per_step": ms, "us_per_layer": ms * 1e3 / N_LAYERS,
                       "kv_gb_per_s": kv_bytes / (ms * 1e-3) / 1e9, "kv_frac_of_hbm_peak_per_gpu": kv_bytes / (ms * 1e-3) / 1e9 / ctx.world / peak}
    return {"workload": f"1 sequence x {SPLITKV_TOKENS} cells, 12 layers, GQA 16q/2kv, head_dim 256, f16 KV; KV range split over {ctx.world} GPU(s)",
            "scaling": "strong", "n_gpus": ctx.world,
            "step": dict(form(ms_step), how="brc_splitkv_step: one launch per rank and token; the layers' attention calls do not depend on one another"),
            "layer_by_layer": dict(form(ms_chain), how="brc_splitkv_attend per layer, each ordered after the one before (a model's dependency chain)"),
            "layer_by_layer_graph": dict(form(ms_chain_graph), how="the same twelve calls captured once in a CUDA graph, one replay per token"),
            "local_share_alone_ms_per_step": ms_local,
            "exchange_and_merge_ms_per_step": ms_step - ms_local,
            "one_gpu_same_run_ms_per_step": ms_one, "speedup_vs_one_gpu_same_run": ms_one / ms_step,
            "exchange": "merged (acc, m, l) of each (layer, kv-head group) stored into every peer's receive buffer by the attention "
                        "kernel (16 512 B per layer per peer, plain stores over NVLink, no flags or fences: an empty slot holds 0xFFFFFFFF "
                        "words and the consumer polls the segment it needs), merged by the CTAs of the unit in the same launch; no NCCL "
                        "collective on the data path",
            "max_abs_vs_cpu_oracle": max_abs, "identical_on_all_ranks": same, "tolerance": "max-abs 2e-3 (measured ~1e-8)"}


def run_native(args):
    ctx = Ctx(args)
    steps, warmup = args.steps, max(args.warmup, 0)
    if args.only_q8v:
        print(json.dumps(bench_q8v(ctx, args, steps, warmup)), flush=True)
        return
    peak, peak_src = measured_peaks()
    full = not args.only_headline
    sampler = ClockSampler(ctx.local) if ctx.rank == 0 else None
    res = bench_batched(ctx, args, args.workload, steps, warmup, sampler=sampler,
                        with_cpu=(ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline and full), full=full)
    lens0, ms_step = res["lens0"], res["ms_step"]
    e2e_mode = min(res["e2e_modes"], key=res["e2e_modes"].get)
    ms_e2e = res["e2e_modes"][e2e_mode]
    kv_bytes_step = float(res["lens_mid"].sum()) * TOKEN_BYTES * N_LAYERS * ctx.world
    kv_gbs = kv_bytes_step / (ms_step * 1e-3) / 1e9
    tok = lambda ms: N_SEQS * ctx.world / (ms * 1e-3)
    line = {
        "metric": "decode_tok_per_s", "value": tok(ms_step), "unit": "tok/s", "n_gpus": ctx.world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args.workload, lens0, args.seed),
        "notes": {"l2": "inputs larger than L2 (%.0f MB of KV per layer, %.1f GB per step and GPU)" % (
                      lens0.sum() * TOKEN_BYTES / 1e6, lens0.sum() * TOKEN_BYTES * N_LAYERS / 1e9),
                  "partition": "every GPU owns 32 sequences of the same lengths and its own pool; no collective",
                  "value": "one launch per step covers the 12 layers (their q / k / v are given up front); a model whose layer "
                           "i+1 depends on layer i sees `layer_by_layer`"},
        "value_windows": {"n": len(res["windows"]), "median": tok(statistics.median(res["windows"])),
                          "min": tok(max(res["windows"])), "max": tok(min(res["windows"])),
                          "how": "the timed window repeated after resetting the lengths; `value` is the first"},
        "kv_gb_per_s": kv_gbs, "kv_frac_of_hbm_peak": kv_gbs / ctx.world / peak,
        "clocks": res["clocks"],
        "e2e": {"value": tok(ms_e2e), "unit": "tok/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                "how": "brc_decode_step_host per step, " + e2e_mode + "; the call returns when the output is complete",
                "ms_per_step_by_mode": res["e2e_modes"]},
        "gpu_launches": steps * 2,
        "roofline": roofline_of(res, peak, peak_src),
        "cpu_baseline": res["cpu"],
    }
    if res["ms_chain"]:
        line["layer_by_layer"] = {"value": tok(res["ms_chain"]), "unit": "tok/s", "ms_per_step": res["ms_chain"],
                                  "us_per_layer": res["ms_chain"] * 1e3 / N_LAYERS,
                                  "how": "per layer brc_kv_append then brc_paged_decode_attn on one stream (24 launches per step): what a "
                                         "model sees whose next layer's query depends on this layer's output"}
        line["layer_by_layer_fused"] = {"value": tok(res["ms_chain_fused"]), "unit": "tok/s", "ms_per_step": res["ms_chain_fused"],
                                        "us_per_layer": res["ms_chain_fused"] * 1e3 / N_LAYERS,
                                        "how": "per layer ONE launch that appends and attends (brc_decode_step_part with one layer per "
                                               "call; 13 launches per step): the same dependency chain through the fused entry point"}
    if full:
        if args.workload == "cfg2":
            line["strong"] = bench_strong(ctx, args, steps)
            if ctx.world == 1:
                r8 = bench_batched(ctx, args, "fixed8k", steps, warmup, full=False)
                m8 = min(r8["e2e_modes"], key=r8["e2e_modes"].get)
                line["q8v"] = bench_q8v(ctx, args, steps, warmup)
                line["fixed8k"] = {"workload": workload_name("fixed8k"), "value": N_SEQS / (r8["ms_step"] * 1e-3), "unit": "tok/s",
                                   "ms_per_step": r8["ms_step"], "roofline": roofline_of(r8, peak, peak_src),
                                   "e2e": {"value": N_SEQS / (r8["e2e_modes"][m8] * 1e-3), "unit": "tok/s",
                                           "ms_per_step": r8["e2e_modes"][m8], "h2d_bytes_per_step": r8["h2d"], "d2h_bytes_per_step": r8["d2h"]}}
        line["splitkv"] = bench_splitkv(ctx, args, steps)
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)
    if ctx.world > 1:
        ctx.dist.destroy_process_group()


def cpu_baseline_sample(pool, batch, q):
    """Times the oracle (C restatement of the reference's f64 CPU attention) on the box's cores over a
    bounded sample: whole layers of one decode step of this same batch, read back from the GPU pool."""
    import oracle

    threads = os.cpu_count() or 1
    tables = batch.block_tables.cpu().numpy().astype(np.uint32)
    lens = batch.seq_lens.cpu().numpy().astype(np.uint32)
    spent, layers_done = 0.0, 0
    while spent < 12.0 and layers_done < 10 * N_LAYERS:   # about 12 s of CPU work, layers taken round-robin
        layer = layers_done % N_LAYERS
        kp = pool.read(0, layer).reshape(-1)
        vp = pool.read(1, layer).reshape(-1)
        ql = q[layer].float().cpu().numpy()
        t0 = time.perf_counter()
        _, used = oracle.decode_batch(kp, vp, tables, lens, ql, N_HEAD, N_KV, HD, n_threads=threads)
        spent += time.perf_counter() - t0
        layers_done += 1
        threads = used
    per_layer = spent / layers_done
    return {"value": N_SEQS / (per_layer * N_LAYERS), "unit": "tok/s", "cores": threads, "kind": "port",
            "sample": f"{layers_done} layer-passes (of the {N_LAYERS} layers of one decode step) over the same 32 sequences "
                      f"({spent:.1f} s of CPU work), scaled to 12 layers; f64 attention as in qsa/cpu.rs"}


# ----------------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation of the path (its f64 oracle algorithm; the Rust
# original cannot be built here, so this is the C port), all host threads; every timed step is a whole
# decode step (append + attention in all 12 layers) of the same 32 sequences
# ----------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from breccia_b200 import synth

    threads = os.cpu_count() or 1
    steps, warmup = args.steps, max(args.warmup, 0)
    lens0 = workload_lengths(args.workload, args.seed)
    tables, n_pool = synth.scattered_tables(args.seed + 7, lens0, page_tokens=PAGE, pool_factor=1.25,
                                            extra_tokens=warmup + steps + 2)
    rng = np.random.default_rng(args.seed)
    n = n_pool * N_KV * PAGE * HD

    def pool_bits():
        out = np.empty(n, np.uint16)
        for at in range(0, n, 1 << 22):  # chunked: the NumPy codec makes 64-bit temporaries
            m = min(1 << 22, n - at)
            x = rng.standard_normal(m, dtype=np.float32)
            x *= np.float32(0.5)
            out[at:at + m] = oracle.f32_to_f16_bits_np(x)
        return out

    # One layer's pools stand for all twelve (the layers' contents are statistically alike and the algorithm
    # does the same work in each): every timed step runs the append and the attention twelve times over them.
    kp, vp = pool_bits(), pool_bits()
    q = oracle.to_f16(rng.standard_normal((N_SEQS, N_HEAD, HD), dtype=np.float32))
    k_new = (rng.standard_normal((N_SEQS, N_KV * HD), dtype=np.float32) * np.float32(0.5))
    v_new = (rng.standard_normal((N_SEQS, N_KV * HD), dtype=np.float32) * np.float32(0.5))
    lens = lens0.copy()
    kw, vw = kp.view(np.uint32), vp.view(np.uint32)

    def one_step():
        used = threads
        for _ in range(N_LAYERS):
            for s in range(N_SEQS):
                oracle.kv_append(kw, vw, tables[s], k_new[s], v_new[s], int(lens[s]), N_KV, HD)
            _, used = oracle.decode_batch(kp, vp, tables, (lens + 1).astype(np.uint32), q, N_HEAD, N_KV, HD, n_threads=threads)
        lens[:] += 1
        return used

    used = threads
    for _ in range(warmup):
        used = one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        used = one_step()
    dt = time.perf_counter() - t0
    ms_step = dt / steps * 1e3
    tok_s = N_SEQS / (ms_step * 1e-3)
    sample = (f"each timed step = a whole decode step of the 32 sequences: append + f64 attention "
              f"(crates/breccia-kernels/src/qsa/cpu.rs) in all {N_LAYERS} layers, one layer's pools standing for all")
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(args.workload, lens0, args.seed),
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference GPU path is Vulkan compute: unavailable on this box; this is its CPU algorithm "
                "(C port of the Rust oracle, which cannot be compiled here)",
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse_args()
    N_LAYERS = a.layers
    if a.impl == "reference":
        run_reference(a)
    else:
        run_native(a)
