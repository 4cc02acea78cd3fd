"""Builds tests/cpp/qsa_mirror_test.cpp against the in-tree library (g++, CUDA runtime headers)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_mirror_test(out_dir) -> dict:
    from breccia_b200 import _lib

    _lib.load()   # fails loudly when the library has not been built
    lib = _lib.LIB_PATH
    exe = os.path.join(str(out_dir), "qsa_mirror_test")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           os.path.join(ROOT, "tests", "cpp", "qsa_mirror_test.cpp"), "-o", exe, "-L", os.path.dirname(lib),
           "-l:" + os.path.basename(lib), "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.dirname(lib), "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    return {"path": exe, "lib": lib}
