"""breccia_b200 — B200 (sm_100a) paged KV-cache hot path behind the breccia `qsa` operator surface.

`_lib` binds the C ABI of include/breccia_kv.h; `qsa` mirrors the reference's host interface on top
of it; `synth` generates the seeded synthetic workloads; `build` compiles the CUDA library in-tree.
"""
from . import _lib  # noqa: F401
from ._lib import BrcError, DTYPE_F16, DTYPE_F32  # noqa: F401
