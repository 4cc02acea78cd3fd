#!/usr/bin/env python
"""Benchmark of the paged KV decode hot path (the batched-decode workload).

    python bench.py --gpus N --steps K --warmup W            # this library on N GPUs (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU algorithm on the host cores

A step = one decode step of the whole batch: in each of the 12 attention layers, append one token's
K/V per sequence through the block tables, then paged GQA decode attention over the whole cache.
Prints ONE JSON line (rank 0).  Sequences are independent, so N GPUs each own their own 32
sequences and pool (weak scaling, no data-path collective); torch.distributed is used only for the
barrier and the max-over-ranks of the device time.
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "fixed8k"],
                    help="cfg2: lengths uniform in [512, 8192]; fixed8k: every sequence at 8192")
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=12,
                    help="attention layers per step (12 = the full workload; fewer only for small profiler captures)")
    return ap.parse_args()


def workload_lengths(kind: str, seed: int, rank: int) -> np.ndarray:
    from breccia_b200 import synth

    if kind == "fixed8k":
        return np.full(N_SEQS, 8192, np.int64)
    return synth.uniform_ints(seed + 1000 * rank, N_SEQS, 512, 8192)


def workload_name(kind: str) -> str:
    if kind == "fixed8k":
        return "batched decode: 32 sequences x 8192 context, 12 layers, GQA 16q/2kv, head_dim 256, f16 KV, 16-token pages"
    return ("batched decode: 32 sequences, context uniform in [512, 8192] (seeded), 12 layers, GQA 16q/2kv, "
            "head_dim 256, f16 KV, 16-token pages scattered in a pool of 1.25x need")


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
    """DRAM bytes per launch of the decode partial kernel from the committed ncu summary, scaled to this
    workload by cached bytes (traffic grows in proportion to the pages streamed)."""
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
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
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
def run_native(args):
    import torch
    import torch.distributed as dist

    from breccia_b200 import synth
    from breccia_b200._lib import DTYPE_F16, DTYPE_F32, call
    from breccia_b200.qsa import DecodeBatch, KvPool, _ptr, _stream_ptr
    import ctypes as C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ["NCCL_DEBUG"] = "WARN"   # no version banner on stdout: rank 0 prints exactly one JSON line
        dist.init_process_group("nccl", device_id=dev)

    steps, warmup = args.steps, max(args.warmup, 0)
    lens0 = workload_lengths(args.workload, args.seed, rank)
    passes_steps = warmup + steps + 2
    tables, n_pool = synth.scattered_tables(args.seed + 7 + rank, lens0, page_tokens=PAGE, pool_factor=1.25,
                                            extra_tokens=passes_steps)
    pool = KvPool(local_rank, N_LAYERS, N_KV, HD, n_pool)
    batch = DecodeBatch(pool, N_HEAD, tables, lens0, q_dtype=DTYPE_F16)

    # ---- fill the cache through the append kernel itself (f32 sources ~ N(0, 0.5^2), seeded on the device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed + rank)
    cu = np.concatenate([[0], np.cumsum(lens0)]).astype(np.int32)
    cu_dev = torch.as_tensor(cu, device=dev)
    zeros = torch.zeros(N_SEQS, dtype=torch.int32, device=dev)
    total = int(cu[-1])
    for layer in range(N_LAYERS):
        k_src = torch.randn((total, N_KV * HD), generator=gen, device=dev) * 0.5
        v_src = torch.randn((total, N_KV * HD), generator=gen, device=dev) * 0.5
        call("brc_kv_append", pool.handle, layer, _ptr(batch.block_tables), batch.table_stride, _ptr(zeros), N_SEQS, 0,
             _ptr(cu_dev), total, int(lens0.max()), _ptr(k_src), _ptr(v_src), DTYPE_F32, _stream_ptr())
        torch.cuda.synchronize()
        del k_src, v_src
    pool.check()

    q = (torch.randn((N_LAYERS, N_SEQS, N_HEAD, HD), generator=gen, device=dev)).half()
    k_new = torch.randn((N_LAYERS, N_SEQS, N_KV * HD), generator=gen, device=dev) * 0.5
    v_new = torch.randn((N_LAYERS, N_SEQS, N_KV * HD), generator=gen, device=dev) * 0.5
    out = torch.empty((N_LAYERS, N_SEQS, N_HEAD, HD), dtype=torch.float32, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n_warm, n_steps, sampler=None):
        batch.reset_lengths(lens0)
        for _ in range(n_warm):
            fn()
        barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler else None
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    # ---- headline: device-resident inputs
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_total, clocks = timed(lambda: batch.step(q, k_new, v_new, out), max(warmup, 3), steps, sampler)
    pool.check()
    ms_step = ms_total / steps
    tok_s = N_SEQS * world / (ms_step * 1e-3)
    lens_mid = lens0 + max(warmup, 3) + (steps + 1) / 2.0
    kv_bytes_step = float(lens_mid.sum()) * TOKEN_BYTES * N_LAYERS * world
    kv_gbs = kv_bytes_step / (ms_step * 1e-3) / 1e9

    # ---- end to end: host (pinned) activations in, attention output back to the host, every step
    q_h = q.cpu().pin_memory()
    k_h = k_new.cpu().pin_memory()
    v_h = v_new.cpu().pin_memory()
    out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    staging = batch.host_staging(N_LAYERS)
    e2e_steps = steps
    # the output either stored by the kernels straight into the pinned host buffer, or staged on the device and
    # copied down: which is faster depends on the host, so both are timed and the better one is reported
    e2e_modes = {}
    for mode, download in (("stored by the kernels into the pinned host buffer", False), ("staged on the device and copied down", True)):
        ms_mode, _ = timed(lambda: batch.step_host(q_h, k_h, v_h, out_h, staging, download=download), 3, e2e_steps)
        e2e_modes[mode] = ms_mode / e2e_steps
    e2e_mode = min(e2e_modes, key=e2e_modes.get)
    ms_e2e = e2e_modes[e2e_mode]
    h2d = q_h.numel() * 2 + k_h.numel() * 4 + v_h.numel() * 4
    d2h = out_h.numel() * 4

    # ---- roofline of the dominant kernel (the split-KV partial kernel), timed by CUDA events around each
    #      of its launches on the launching stream
    call("brc_timing_enable", pool.handle, 1)
    prof_steps = min(steps, 20)
    timed(lambda: batch.step(q, k_new, v_new, out), 3, prof_steps)
    launches, total_ms = C.c_uint32(), C.c_double()
    stage_ms = {}
    for name, sid in (("kv_append", 0), ("attn_partial", 1), ("attn_combine", 2)):
        call("brc_timing_read", pool.handle, sid, C.byref(launches), C.byref(total_ms))
        stage_ms[name] = (launches.value, total_ms.value)
    call("brc_timing_enable", pool.handle, 0)
    n_part, ms_part = stage_ms["attn_partial"]
    # the timing pass started again from lens0: 3 warm-up steps, then prof_steps; lengths at step i
    lens_prof = lens0 + 3 + (prof_steps + 1) / 2.0
    # events of the warm-up steps were recorded too; lengths differ by < 0.1 %, average over all recorded
    lens_prof = lens0 + (3 + prof_steps + 1) / 2.0
    alg_bytes = algorithmic_bytes_per_layer(lens_prof)
    iso_s = ms_part / max(n_part, 1) * 1e-3       # one launch alone (events around it serialise the stream)
    peak, peak_src = measured_peaks()
    # In a decode step the layers' kernels overlap (each starts on the SMs the previous one has left), so
    # a launch's duration is taken from the timed region of the headline pass: CUDA events around all
    # `steps` steps, divided by the attention launches in it.  This charges the small position-advance
    # kernel of every step to the attention launches too.
    alg_bytes_mid = algorithmic_bytes_per_layer(lens_mid)
    dur_s = ms_step * 1e-3 / N_LAYERS
    achieved = alg_bytes_mid / dur_s / 1e9
    traffic = None
    rec = recorded_traffic()
    if rec:
        traffic = rec["dram_bytes_per_cached_byte"] * float(lens_prof.sum()) * TOKEN_BYTES

    # ---- the reference's CPU algorithm on this box's cores, bounded sample (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample(pool, batch, q)

    if rank == 0:
        line = {
            "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(args.workload), "n_seqs_per_gpu": N_SEQS,
                       "sum_context_tokens_per_gpu": int(lens0.sum()), "layers": N_LAYERS,
                       "l2": "inputs larger than L2 (%.0f MB of KV per layer, %.1f GB per step)" % (
                           lens0.sum() * TOKEN_BYTES / 1e6, lens0.sum() * TOKEN_BYTES * N_LAYERS / 1e9),
                       "partition": "sequences sharded per GPU, no collective", "seed": args.seed},
            "kv_gb_per_s": kv_gbs, "kv_frac_of_hbm_peak": kv_gbs / world / peak,
            "clocks": clocks,
            "e2e": {"value": N_SEQS * world / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "brc_decode_step_host per step: pinned q/k/v uploaded, output " + e2e_mode +
                           ", call returns when it is complete",
                    "ms_per_step_by_output_mode": e2e_modes},
            "gpu_launches": steps * (1 + N_LAYERS),
            "roofline": {"kernel": "decode_partial_kernel<256,f16 q>", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": alg_bytes_mid, "avg_launch_us": dur_s * 1e6,
                         "launches_timed": steps * N_LAYERS,
                         "how": "timed region of the headline pass / attention launches in it (layers of a step overlap)",
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         "isolated_launch": {"avg_launch_us": iso_s * 1e6, "achieved": alg_bytes / iso_s / 1e9,
                                             "frac": alg_bytes / iso_s / 1e9 / peak, "launches_timed": n_part,
                                             "how": "CUDA events around every launch (no overlap between layers)"},
                         "stage_us_per_launch": {k: (v[1] / max(v[0], 1)) * 1e3 for k, v in stage_ms.items()}},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    pool.release()
    if world > 1:
        dist.destroy_process_group()


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
# original cannot be built here, so this is the C port), all host threads, bounded sample per step
# ----------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from breccia_b200 import synth

    threads = os.cpu_count() or 1
    steps, warmup = args.steps, max(args.warmup, 0)
    lens0 = workload_lengths(args.workload, args.seed, 0)
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

    kp, vp = pool_bits(), pool_bits()
    q = oracle.to_f16(rng.standard_normal((N_SEQS, N_HEAD, HD), dtype=np.float32))
    k_new = (rng.standard_normal((N_SEQS, N_KV * HD), dtype=np.float32) * np.float32(0.5))
    v_new = (rng.standard_normal((N_SEQS, N_KV * HD), dtype=np.float32) * np.float32(0.5))
    lens = lens0.copy()
    kw, vw = kp.view(np.uint32), vp.view(np.uint32)

    def one_layer_step():
        # the layer's share of a decode step: append one token per sequence, then attention
        for s in range(N_SEQS):
            oracle.kv_append(kw, vw, tables[s], k_new[s], v_new[s], int(lens[s]), N_KV, HD)
        lens[:] += 1
        _, used = oracle.decode_batch(kp, vp, tables, lens.astype(np.uint32), q, N_HEAD, N_KV, HD, n_threads=threads)
        return used

    used = threads
    for _ in range(warmup):
        used = one_layer_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        used = one_layer_step()
    dt = time.perf_counter() - t0
    per_layer = dt / steps
    ms_step = per_layer * N_LAYERS * 1e3
    tok_s = N_SEQS / (ms_step * 1e-3)
    sample = (f"each timed step = 1 of {N_LAYERS} layers of one decode step of the 32 sequences (append + f64 "
              f"attention, crates/breccia-kernels/src/qsa/cpu.rs), scaled x{N_LAYERS}")
    line = {
        "impl": "reference", "metric": "decode_tok_per_s", "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": workload_name(args.workload), "n_seqs_per_gpu": N_SEQS,
                   "sum_context_tokens_per_gpu": int(lens0.sum()), "layers": N_LAYERS, "seed": args.seed},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": used, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference GPU path is Vulkan compute: unavailable on this box; this is its CPU algorithm "
                "(C port of the Rust oracle, which cannot be compiled here)",
    }
    print(json.dumps(line))


if __name__ == "__main__":
    a = parse_args()
    N_LAYERS = a.layers
    if a.impl == "reference":
        run_reference(a)
    else:
        run_native(a)
