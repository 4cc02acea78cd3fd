"""Generates tests/golden/cfg1_golden.npz: the oracle's results for the CPU-runnable conformance
configuration (1 layer, 1 sequence, GQA 16q/2kv, head_dim 256, 16-cell pages, context 1024 through a
seeded permutation of a 256-page pool, append one token, one decode-attention step).

The reference itself cannot run here (Rust + GLSL, neither toolchain present), so the vectors come
from the C restatement in oracle/, which is pinned by the reference's known-answer tests.

    python tests/golden/make_cfg1_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from breccia_b200 import synth  # noqa: E402

N_HEAD, N_KV, HD, PAGE, POOL_PAGES, CONTEXT = 16, 2, 256, 16, 256, 1024
SEED = 0xC0FFEE


def cfg1_inputs():
    """Everything the configuration needs, from fixed seeds."""
    table = synth.permutation(SEED, POOL_PAGES)[:CONTEXT // PAGE + 1]       # 65 entries
    row = N_KV * HD
    k_ctx = synth.normal(SEED + 1, CONTEXT * row, 0.5).reshape(CONTEXT, row)
    v_ctx = synth.normal(SEED + 2, CONTEXT * row, 0.5).reshape(CONTEXT, row)
    k_new = synth.normal(SEED + 3, row, 0.5).reshape(1, row)
    v_new = synth.normal(SEED + 4, row, 0.5).reshape(1, row)
    q = oracle.to_f16(synth.normal(SEED + 5, N_HEAD * HD, 1.0)).reshape(N_HEAD, HD)  # f16 query
    return table, k_ctx, v_ctx, k_new, v_new, q


def cfg1_expected():
    table, k_ctx, v_ctx, k_new, v_new, q = cfg1_inputs()
    words = POOL_PAGES * N_KV * PAGE * HD // 2
    kp = np.zeros(words, np.uint32)
    vp = np.zeros(words, np.uint32)
    assert oracle.kv_append(kp, vp, table, k_ctx, v_ctx, 0, N_KV, HD) == 0
    assert oracle.kv_append(kp, vp, table, k_new, v_new, CONTEXT, N_KV, HD) == 0
    _, kf = oracle.gather(kp.view(np.uint16), table, CONTEXT + 1, N_KV, HD)
    _, vf = oracle.gather(vp.view(np.uint16), table, CONTEXT + 1, N_KV, HD)
    out = oracle.attend(q, kf, vf, np.arange(CONTEXT + 1, dtype=np.uint32), CONTEXT, N_HEAD, N_KV, HD)
    return kp, vp, out


if __name__ == "__main__":
    kp, vp, out = cfg1_expected()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cfg1_golden.npz")
    np.savez_compressed(path, out=out,
                        k_pool_sha256=np.frombuffer(hashlib.sha256(kp.tobytes()).digest(), np.uint8),
                        v_pool_sha256=np.frombuffer(hashlib.sha256(vp.tobytes()).digest(), np.uint8),
                        last_page_k=kp.view(np.uint16).reshape(POOL_PAGES, N_KV, PAGE, HD)[cfg1_inputs()[0][64]])
    print(path, os.path.getsize(path), "bytes")
