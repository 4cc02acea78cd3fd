"""ctypes binding of libbreccia_kv.so — the declarations of include/breccia_kv.h, nothing else.

The library must be present (``python -m breccia_b200.build``); there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libbreccia_kv.so")

OK = 0
ERR_INVALID = -1
ERR_CAPACITY = -2
ERR_CUDA = -3
ERR_NO_PAGES = -4
ERR_TIMEOUT = -5
ERR_DEVICE_CHECK = -6
ERR_UNSUPPORTED = -7
ERR_NOT_RESIDENT = -8

DTYPE_F32 = 0
DTYPE_F16 = 1


class BrcError(RuntimeError):
    """A libbreccia_kv entry point returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class Geometry(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("n_kv_head", C.c_uint32), ("head_dim", C.c_uint32),
                ("page_tokens", C.c_uint32), ("n_pages", C.c_uint32), ("device", C.c_int32),
                ("half_page_bytes", C.c_uint64), ("total_bytes", C.c_uint64)]


_vp = C.c_void_p
_u32 = C.c_uint32
_u64 = C.c_uint64
_i32 = C.c_int32
_f32 = C.c_float
_u32p = C.POINTER(C.c_uint32)
_u64p = C.POINTER(C.c_uint64)
_vpp = C.POINTER(C.c_void_p)

# name -> (argtypes); every function returns brc_status unless listed in _SPECIAL.
SIGNATURES = {
    "brc_pool_create": [_i32, _u32, _u32, _u32, _u32, _u32, _vpp],
    "brc_pool_create_bookkeeping": [_u32, _u32, _u32, _u32, _u32, _vpp],
    "brc_pool_destroy": [_vp],
    "brc_pool_geometry": [_vp, C.POINTER(Geometry)],
    "brc_pool_bytes": [_vp, _u64p],
    "brc_pool_zero": [_vp, _vp],
    "brc_pool_poison_nan": [_vp, _vp],
    "brc_pool_k_ptr": [_vp, _u32, _vpp],
    "brc_pool_v_ptr": [_vp, _u32, _vpp],
    "brc_pool_read": [_vp, _i32, _u32, _u64, _vp, _u64, _vp],
    "brc_pool_write": [_vp, _i32, _u32, _u64, _vp, _u64, _vp],
    "brc_pool_check": [_vp, _vp],
    "brc_pages_alloc": [_vp, _u32, _u32p],
    "brc_pages_retain": [_vp, _u32p, _u32],
    "brc_pages_release": [_vp, _u32p, _u32],
    "brc_page_refcount": [_vp, _u32, _u32p],
    "brc_pages_free_count": [_vp, _u32p],
    "brc_kv_append": [_vp, _u32, _vp, _u32, _vp, _u32, _u32, _vp, _u32, _u32, _vp, _vp, _i32, _vp],
    "brc_page_gather": [_vp, _u32, _vp, _u32, _u32, _vp, _vp, _vp],
    "brc_page_copy": [_vp, _vp, _vp, _u32, _vp],
    "brc_seq_fork": [_vp, _u32p, _u32, _u32p, _u32p, _vp],
    "brc_decode_workspace_bytes": [_vp, _u32, _u32, _u64p],
    "brc_decode_share_rates": [_vp, C.POINTER(C.c_float), _u32, _u32p],
    "brc_paged_decode_attn": [_vp, _u32, _vp, _i32, _u32, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _f32, _vp, _vp,
                              _u64, _vp],
    "brc_paged_decode_attn_static": [_vp, _u32, _vp, _i32, _u32, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _f32, _vp, _vp],
    "brc_decode_partial_bytes": [_u32, _u32, _u32, _u64p],
    "brc_decode_partial": [_vp, _u32, _vp, _i32, _u32, _vp, _u32, _vp, _u32, _u32, _f32, _vp, _vp, _u64, _vp],
    "brc_decode_combine": [_i32, _vp, _u32, _u64, _u32, _u32, _u32, _vp, _u32, _vp, _vp],
    "brc_decode_step": [_vp, _u32, _u32, _vp, _u32, _vp, _vp, _u32, _u32, _vp, _i32, _u64, _u32, _vp, _vp, _i32, _u64,
                        _vp, _u32, _u64, _f32, _vp, _u64, _vp, _u64, _vp],
    "brc_decode_step_part": [_vp, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _vp, _u32, _u32, _vp, _i32, _u64, _u32, _vp, _vp,
                             _i32, _u64, _vp, _u32, _u64, _f32, _vp, _u64, _vp, _u64, _vp],
    "brc_topk_blocks": [_vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _i32, _vp, _vp, _vp],
    "brc_cold_open": [_vp, C.c_char_p, _u32, _i32, _vpp],
    "brc_cold_close": [_vp],
    "brc_cold_spill": [_vp, _u32p, _u64p, _u32, _u32p],
    "brc_cold_fetch": [_vp, _u32p, _u32, _i32, _u32p],
    "brc_cold_find": [_vp, _u64, _u32p],
    "brc_cold_stats": [_vp, _u32p, _u32p, _u64p, _u64p],
    "brc_idx_pool": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _f32, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _u32, _vp],
    "brc_idx_tail": [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp, _vp],
    "brc_idx_score": [_vp, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _u32, _u32, _u32, _f32, _vp, _vp],
    "brc_pool_create_q8v": [_i32, _u32, _u32, _u32, _u32, _u32, _vpp],
    "brc_pool_v_layout": [_vp, C.POINTER(C.c_int32)],
    "brc_decode_step_host_staging_bytes": [_vp, _u32, _u32, _u32, _i32, _i32, _u64p],
    "brc_decode_step_host": [_vp, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _vp, _u32, _u32, _vp, _i32, _u32, _vp, _vp, _i32, _f32,
                             _vp, _vp, _u64, _vp, _u64, _vp],
    "brc_paged_prefill_attn": [_vp, _u32, _vp, _i32, _u32, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _u32, _f32, _vp, _vp],
    "brc_radix_create": [_vp, _vpp],
    "brc_radix_destroy": [_vp],
    "brc_radix_match": [_vp, _u32p, _u32, _u32p, _u32, _u32p],
    "brc_radix_insert": [_vp, _u32p, _u32, _u32p, _u32, _u32p],
    "brc_radix_evict": [_vp, _u32, _u32p],
    "brc_radix_release": [_vp, _u32p, _u32],
    "brc_radix_prefix_tags": [_u32p, _u32, _u32, _u64p, _u32, _u32p],
    "brc_radix_stats": [_vp, _u64p, _u64p, _u64p, _u64p],
    "brc_tier_create": [_vp, _u32, _vpp],
    "brc_tier_destroy": [_vp],
    "brc_tier_demote": [_vp, _u32p, _u32, _u32p, _vp],
    "brc_tier_promote": [_vp, _u32p, _u32, _u32p],
    "brc_tier_fence": [_vp, _vp],
    "brc_tier_sync": [_vp],
    "brc_tier_touch": [_vp, _u32p, _u32],
    "brc_tier_lru": [_vp, _u32, _u32p, _u32p],
    "brc_tier_stats": [_vp, _u64p, _u64p, _u64p, _u64p, _u32p],
    "brc_comm_create": [_vp, _u32, _u32, _u32, _u32, _vpp],
    "brc_comm_ipc_handle": [_vp, _vp],
    "brc_comm_connect_ipc": [_vp, _vp, _u32],
    "brc_comm_connect_local": [_vp, _vpp, _u32],
    "brc_comm_set_wait_ms": [_vp, _u32],
    "brc_comm_reset": [_vp, _vp],
    "brc_comm_destroy": [_vp],
    "brc_splitkv_exchange_combine": [_vp, _vp, _u32, _vp, _u32, _vp, _vp],
    "brc_splitkv_attend": [_vp, _u32, _vp, _i32, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _f32, _vp, _vp, _u64, _vp],
    "brc_splitkv_step": [_vp, _u32, _u32, _vp, _i32, _u64, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _f32, _vp, _vp, _u64, _vp],
    "brc_state_dump": [_vp, _u32, _u32p, _u32, _u32, _u32, C.c_char_p, _vp],
    "brc_state_load": [_vp, _u32, _u32p, _u32, _u32, _u32, C.c_char_p, _vp],
    "brc_qk_prepare_append": [_vp, _u32, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _f32, _vp, _u32, _u32, _vp, _u32, _vp, _u32, _u32,
                              _u32, _vp, _i32, _vp],
    "brc_paged_sparse_attn": [_vp, _u32, _vp, _i32, _u32, _vp, _u32, _vp, _u32, _vp, _u32, _u32, _vp, _u32, _vp, _u32, _f32, _vp, _vp],
    "brc_timing_enable": [_vp, _i32],
    "brc_timing_read": [_vp, _i32, _u32p, C.POINTER(C.c_double)],
}
_SPECIAL = {
    "brc_last_error": ([], C.c_char_p),
    "brc_abi_version": ([], C.c_int32),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m breccia_b200.build` "
                          "(there is no fallback path)")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int32
    for name, (args, res) in _SPECIAL.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise BrcError(status, load().brc_last_error().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))
