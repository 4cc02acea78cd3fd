"""Split-KV decode across GPUs (NCCL all-gather of the partials + merge).  Needs at least two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("n_tokens", [5000, 33])
def test_split_kv_across_gpus_equals_the_whole(cuda_device, n_tokens):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + n_tokens % 97), os.path.join(HERE, "_splitkv_worker.py"), str(n_tokens)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0
