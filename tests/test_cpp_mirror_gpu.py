"""The conformance configuration driven from C++ through include/breccia_qsa.hpp (QsaState / QsaWorkspace / Qsa with
the reference's call sequence: kv_append in chunks, one more token, topk_dense, attend, apply).  The
program's cache pages must be bit-exact and its output in tolerance against the committed golden
vectors of the oracle."""
import hashlib
import os
import subprocess
import sys

import numpy as np
import pytest

from cpp_build import build_mirror_test
from helpers import ATTN_MAX_ABS, ATTN_MAX_REL, attention_errors

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_cfg1_golden import CONTEXT, cfg1_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def test_cfg1_through_the_cpp_mirror(cuda_device, tmp_path):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "cfg1_golden.npz"))
    table, k_ctx, v_ctx, k_new, v_new, q = cfg1_inputs()
    d = str(tmp_path)
    np.asarray(table[:65], np.uint32).tofile(os.path.join(d, "table.u32"))
    np.asarray(k_ctx[:CONTEXT], np.float32).tofile(os.path.join(d, "k_ctx.f32"))
    np.asarray(v_ctx[:CONTEXT], np.float32).tofile(os.path.join(d, "v_ctx.f32"))
    np.asarray(k_new, np.float32).tofile(os.path.join(d, "k_new.f32"))
    np.asarray(v_new, np.float32).tofile(os.path.join(d, "v_new.f32"))
    np.asarray(q, np.float32).tofile(os.path.join(d, "q.f32"))
    exe = build_mirror_test(tmp_path)
    r = subprocess.run([exe["path"], "gpu", d], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    kp = np.fromfile(os.path.join(d, "k_pool.u16"), np.uint16)
    vp = np.fromfile(os.path.join(d, "v_pool.u16"), np.uint16)
    assert hashlib.sha256(kp.tobytes()).digest() == bytes(g["k_pool_sha256"])
    assert hashlib.sha256(vp.tobytes()).digest() == bytes(g["v_pool_sha256"])
    out = np.fromfile(os.path.join(d, "out.f32"), np.float32).reshape(g["out"].shape)
    max_abs, max_rel, _ = attention_errors(out, g["out"])
    assert max_abs <= ATTN_MAX_ABS and max_rel <= ATTN_MAX_REL
