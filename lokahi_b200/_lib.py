"""ctypes binding of libstrata_b200.so (the C ABI declared in include/strata_b200.h).

There is no fallback: importing this module without the built library raises, and so does
every compute call without a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstrata_b200.so")

# status codes (include/strata_b200.h)
OK, ERR_BAD_ARG, ERR_REPLAY, ERR_OUT_OF_PAGES, ERR_NOT_RESIDENT = 0, -1, -2, -3, -4
ERR_TIMEOUT, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_FLAG = -5, -6, -7, -8
F32, BF16 = 0, 1
PAGE_UNASSIGNED = -1
ABI_VERSION = 2
STATIC_SCRATCH_BYTES = 16 << 20
MAX_TOKENS_PER_SEQ = 262144
XCHG_HEAD_GATHER, XCHG_SEQ_MERGE = 1, 2
STEP_CONSECUTIVE = 1


class OutOfPagesError(RuntimeError):
    """The page, sequence or host-slot allocator cannot satisfy the request; nothing was changed."""


class NotResidentError(RuntimeError):
    """A page needed by the call is parked in host memory."""


class DeviceFlagError(RuntimeError):
    """A kernel recorded a bad page id, length or sequence id in the pool's status word."""


class SkvConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "device", "dtype", "num_layers", "num_kv_heads", "head_dim", "page_size", "num_pages",
        "max_seqs", "max_pages_per_seq", "host_pages")]


class SkvAppendArgs(C.Structure):
    _fields_ = [
        ("layer", C.c_int32), ("n_seqs", C.c_int32),
        ("seq_ids", C.POINTER(C.c_int32)), ("start_pos", C.POINTER(C.c_int32)),
        ("n_new", C.c_int32),
        ("k", C.c_void_p), ("v", C.c_void_p),
        ("kv_stride_seq", C.c_int64), ("kv_stride_head", C.c_int64), ("kv_stride_tok", C.c_int64),
        ("rope_k", C.c_int32),
        ("q_in", C.c_void_p), ("q_out", C.c_void_p), ("n_q_heads", C.c_int32),
        ("q_stride_seq", C.c_int64), ("q_stride_head", C.c_int64), ("q_stride_tok", C.c_int64),
    ]


class SkvExchange(C.Structure):
    _fields_ = [("mode", C.c_int32), ("rank", C.c_int32), ("world", C.c_int32), ("epoch", C.c_uint32),
                ("recv_ptrs", C.POINTER(C.c_void_p)), ("out", C.c_void_p)]


class SkvStepArgs(C.Structure):
    _fields_ = [
        ("layer", C.c_int32), ("n_seqs", C.c_int32),
        ("seq_ids", C.POINTER(C.c_int32)),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("q_row_stride", C.c_int64), ("k_row_stride", C.c_int64), ("v_row_stride", C.c_int64), ("out_row_stride", C.c_int64),
        ("n_q_heads", C.c_int32), ("eps", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("xchg", C.POINTER(SkvExchange)), ("partial_out", C.c_void_p),
        ("positions", C.POINTER(C.c_int32)), ("store", C.POINTER(C.c_uint8)),
        ("flags", C.c_uint32),
    ]


_i32, _i64, _vp, _f = C.c_int32, C.c_int64, C.c_void_p, C.c_float
_pi32 = C.POINTER(C.c_int32)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "skv_abi_version": (_i32, []),
    "skv_create": (_i32, [C.POINTER(SkvConfig), C.POINTER(_vp)]),
    "skv_destroy": (_i32, [_vp]),
    "skv_last_error": (C.c_char_p, [_vp]),
    "skv_status_string": (C.c_char_p, [_i32]),
    "skv_launch_count": (_i64, []),
    "skv_alloc_sequence": (_i32, [_vp, _pi32]),
    "skv_reload_env": (None, []),
    "skv_free_sequence": (_i32, [_vp, _i32, _vp]),
    "skv_reserve": (_i32, [_vp, _i32, _i32, _vp]),
    "skv_set_page_table": (_i32, [_vp, _i32, _pi32, _i32, _i32, _vp]),
    "skv_truncate": (_i32, [_vp, _i32, _pi32, _i32, _i32, _vp]),
    "skv_length": (_i32, [_vp, _i32, _i32, _pi32]),
    "skv_lengths": (_i32, [_vp, _i32, _pi32, _i32]),
    "skv_page_table": (_i32, [_vp, _i32, _pi32, _i32, _pi32]),
    "skv_pool_counters": (_i32, [_vp, C.POINTER(_i64)]),
    "skv_pool_pointers": (_i32, [_vp, _i32, C.POINTER(_vp), C.POINTER(_vp)]),
    "skv_device_tables": (_i32, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "skv_set_rope": (_i32, [_vp, C.POINTER(_f), _i32, _f]),
    "skv_append": (_i32, [_vp, C.POINTER(SkvAppendArgs), _vp]),
    "skv_gather": (_i32, [_vp, _i32, _pi32, _i32, _vp, _vp, _i32, _vp]),
    "skv_decode_workspace_bytes": (C.c_size_t, [_vp, _i32, _i32]),
    "skv_decode_attn": (_i32, [_vp, _i32, _pi32, _i32, _vp, _vp, _pi32, _i32, _f, _vp, C.c_size_t, _vp]),
    "skv_exchange_bytes": (C.c_size_t, [_i32, _i32, _i32, _i32, _i32, _i32]),
    "skv_decode_attn_xchg": (_i32, [_vp, _i32, _pi32, _i32, _vp, _pi32, _i32, _f, _vp, C.c_size_t, C.POINTER(SkvExchange), _vp]),
    "skv_decode_step_ex": (_i32, [_vp, C.POINTER(SkvStepArgs), _vp]),
    "skv_decode_step_xchg": (_i32, [_vp, _i32, _pi32, _i32, _vp, _vp, _vp, _i32, _f, _vp, C.c_size_t, C.POINTER(SkvExchange), _vp]),
    "skv_decode_partial": (_i32, [_vp, _i32, _pi32, _i32, _vp, _pi32, _i32, _vp, C.c_size_t, _vp, _vp]),
    "skv_merge_partials": (_i32, [_vp, _i32, _i64, _i32, _i32, _f, _vp, _i32, _vp]),
    "skv_decode_step": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _f, _vp, C.c_size_t, _vp]),
    "skv_decode_step_seqs": (_i32, [_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _f, _vp, C.c_size_t, _vp]),
    "skv_decode_attn_static": (_i32, [_vp, _i32, _pi32, _i32, _vp, _vp, _pi32, _i32, _f, _vp]),
    "skv_attn_dense": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f, _vp, _vp]),
    "skv_prefill_attn_paged": (_i32, [_vp, _i32, _pi32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _f, _vp]),
    "skv_evict": (_i32, [_vp, _i32, _i32, _i32, _vp]),
    "skv_prefetch": (_i32, [_vp, _i32, _i32, _i32, _vp]),
    "skv_sync_transfers": (_i32, [_vp, _vp]),
    "skv_wait_resident": (_i32, [_vp, _i32]),
    "skv_check_device_status": (_i32, [_vp, _vp, _pi32]),
    "skv_rope_rows": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _f, _i32, _vp]),
    "skv_rmsnorm": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f, _i32, _vp]),
    "skv_swiglu": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "skv_swiglu_rows": (_i32, [_vp, _vp, _vp, _i64, _i32, _i64, _i64, _i64, _i32, _vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python lokahi_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.skv_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI {lib.skv_abi_version()}, binding expects {ABI_VERSION}")
    return lib


lib = _load()


def raise_for_status(status: int, pool_handle=None) -> None:
    """Map a status code to the exception type the reference raises for the same condition."""
    if status == OK:
        return
    msg = ""
    if pool_handle:
        raw = lib.skv_last_error(pool_handle)
        msg = raw.decode() if raw else ""
    if not msg:
        msg = lib.skv_status_string(status).decode()
    if status in (ERR_BAD_ARG, ERR_REPLAY):
        raise ValueError(msg)
    if status == ERR_OUT_OF_PAGES:
        raise OutOfPagesError(msg)
    if status == ERR_NOT_RESIDENT:
        raise NotResidentError(msg)
    if status == ERR_TIMEOUT:
        raise TimeoutError(msg)
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    if status == ERR_DEVICE_FLAG:
        raise DeviceFlagError(msg)
    raise RuntimeError(f"strata_b200: {msg} (status {status})")


def i32_array(values):
    """ctypes int32 array (or None) from a sequence of ints."""
    if values is None:
        return None
    values = list(values)
    return (C.c_int32 * len(values))(*values)
