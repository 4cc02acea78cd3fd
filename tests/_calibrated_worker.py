"""Worker of test_decode_gpu.py::test_shares_in_proportion_to_measured_rates_when_asked (run with
BRC_DECODE_CALIBRATE=1): a pool of more than 1 GiB measures
the streaming rates of the device's SMs, the decode launches then cut their work in proportion, and the attention
output still matches the oracle.  Prints one line and exits 0 / 1."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from breccia_b200 import _lib, synth  # noqa: E402
from breccia_b200._lib import DTYPE_F16  # noqa: E402
from breccia_b200.qsa import DecodeBatch, KvPool  # noqa: E402


def main():
    n_head, n_kv, hd = 16, 2, 256
    n_pool = 70000                                     # x 16 KiB = 1.07 GiB of K: large enough to be measured
    pool = KvPool(0, 1, n_kv, hd, n_pool)
    rates = (C.c_float * 256)()
    n = C.c_uint32()
    _lib.call("brc_decode_share_rates", pool.handle, rates, 256, C.byref(n))
    r = np.array(rates[:n.value])
    ok = n.value == torch.cuda.get_device_properties(0).multi_processor_count and bool((r >= 0.75).all() and (r <= 1.25).all())
    ok = ok and abs(float(r.mean()) - 1.0) < 0.02 and len(set(r.tolist())) > 1
    lens = np.array([9000, 33, 4097, 700, 12000, 16, 2049, 5000], np.int64)
    used = 4096                                        # the sequences' pages are scattered over the pool's first 4096
    need = int(((lens + 15) // 16).sum())
    ids = synth.permutation(5, used)[:need].astype(np.uint32)
    tables = np.zeros((lens.size, int((lens.max() + 15) // 16)), np.uint32)
    at = 0
    for s, ln in enumerate(lens):
        npg = int((ln + 15) // 16)
        tables[s, :npg] = ids[at:at + npg]
        at += npg
    k = oracle.f32_to_f16_bits_np(synth.normal(11, used * n_kv * 16 * hd, 0.5))
    v = oracle.f32_to_f16_bits_np(synth.normal(12, used * n_kv * 16 * hd, 0.5))
    pool.write(0, 0, k)
    pool.write(1, 0, v)
    q32 = oracle.to_f16(synth.normal(13, lens.size * n_head * hd)).reshape(lens.size, n_head, hd)
    batch = DecodeBatch(pool, n_head, tables, lens, q_dtype=DTYPE_F16)
    qd = torch.from_numpy(q32).cuda().half()
    out = torch.full((lens.size, n_head, hd), float("nan"), device="cuda")
    out2 = torch.full_like(out, float("nan"))
    batch.attend(0, qd, out)
    batch.attend(0, qd, out2)
    pool.check()
    got = out.cpu().numpy()
    want, _ = oracle.decode_batch(k, v, tables, lens, q32, n_head, n_kv, hd)
    err = float(np.abs(got - want).max())
    same = bool(torch.equal(out, out2))
    ok = ok and bool(np.isfinite(got).all()) and err <= 2e-3 and same
    print(f"calibrated shares: {n.value} rates in [{r.min():.3f}, {r.max():.3f}], max_abs vs oracle {err:.2e}, two launches identical {same}",
          flush=True)
    pool.release()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
