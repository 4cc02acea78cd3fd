"""The C++ host-side mirror (include/breccia_qsa.hpp) compiles against the C ABI and its host logic
(allocator, refcounts, shared tables, capacity refusal) works without a GPU."""
import os
import subprocess

from cpp_build import build_mirror_test


def test_cpp_mirror_host_logic(tmp_path):
    exe = build_mirror_test(tmp_path)
    env = dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(exe["lib"]) + ":" + os.environ.get("LD_LIBRARY_PATH", ""))
    r = subprocess.run([exe["path"], "cpu"], capture_output=True, text=True, timeout=60, env=env)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == "ok"
