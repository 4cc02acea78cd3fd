"""The committed cfg1 vectors still match what the oracle produces (guards fixture and oracle drift)."""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_cfg1_golden import cfg1_expected  # noqa: E402


def test_cfg1_golden_matches_oracle():
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "cfg1_golden.npz"))
    kp, vp, out = cfg1_expected()
    assert np.array_equal(g["out"], out)
    assert bytes(g["k_pool_sha256"]) == hashlib.sha256(kp.tobytes()).digest()
    assert bytes(g["v_pool_sha256"]) == hashlib.sha256(vp.tobytes()).digest()
