"""ctypes binding of libtitan_kv.so (the C ABI declared in include/titan_kv.h).

There is no fallback: if the shared library is missing the import fails.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtitan_kv.so")

TK_OK, TK_INVALID_ARG, TK_OUT_OF_PAGES, TK_CUDA_ERROR, TK_TIMEOUT, TK_OUT_OF_SEQS, TK_UNSUPPORTED = range(7)
TK_FP32, TK_FP16, TK_BF16, TK_FP8_E4M3 = 0, 1, 2, 3
TK_DECODE_AUTO, TK_DECODE_SIMT, TK_DECODE_MMA = 0, 1, 2
TK_MERGE_IN_KERNEL, TK_MERGE_SEPARATE = 0, 1
TK_OVERLAP_AUTO, TK_OVERLAP_OFF = 0, 1
TK_PREFILL_AUTO, TK_PREFILL_MMA_SYNC = 0, 1
TK_DEVICE_NONE = -2
TK_PEER_HANDLE_BYTES = 64


class KvConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_layers", "num_heads", "num_kv_heads", "head_dim", "page_size", "dtype", "io_dtype",
        "num_pages", "max_seqs", "max_pages_per_seq", "max_step_tokens", "chunk_tokens",
        "decode_impl", "device", "hot_window", "cold_pages", "v_head_dim", "merge_impl", "launch_overlap", "prefill_impl")]


class KvStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "pages_total", "pages_free", "pages_cold", "page_allocs", "page_frees", "seq_allocs",
        "seq_frees", "evictions", "prefetch_hits", "prefetch_misses", "bytes_h2d", "bytes_d2h",
        "steps", "tokens_appended", "pages_sealed", "evictions_refused")]


class SchedConfig(C.Structure):
    _fields_ = [("max_batch_size", C.c_int32), ("max_prefill_tokens", C.c_int32), ("reserved", C.c_int32 * 6)]


class SchedStats(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("active_requests", "queued_requests", "completed_requests", "cancelled_requests")] + \
               [(n, C.c_int64) for n in ("total_tokens_generated", "total_prompt_tokens", "iterations", "preemptions")] + \
               [(n, C.c_float) for n in ("avg_ttft_ms", "avg_tps", "batch_utilization")]


_P = C.c_void_p
_I32P = C.POINTER(C.c_int32)

# name -> (restype, argtypes); every symbol include/titan_kv.h declares
SIGNATURES = {
    "tk_status_str": (C.c_char_p, [C.c_int]),
    "tk_kv_last_error": (C.c_char_p, [_P]),
    "tk_kv_config_default": (None, [C.POINTER(KvConfig)]),
    "tk_kv_arena_bytes": (C.c_size_t, [C.POINTER(KvConfig)]),
    "tk_kv_create": (C.c_int, [C.POINTER(KvConfig), C.POINTER(_P)]),
    "tk_kv_create_external": (C.c_int, [C.POINTER(KvConfig), _P, C.c_size_t, C.POINTER(_P)]),
    "tk_kv_destroy": (C.c_int, [_P]),
    "tk_kv_get_config": (C.c_int, [_P, C.POINTER(KvConfig)]),
    "tk_kv_memory_bytes": (C.c_size_t, [_P]),
    "tk_kv_layer_ptrs": (C.c_int, [_P, C.c_int, C.POINTER(_P), C.POINTER(_P), C.POINTER(_P)]),
    "tk_kv_seq_alloc": (C.c_int, [_P, _I32P]),
    "tk_kv_seq_free": (C.c_int, [_P, C.c_int32]),
    "tk_kv_reserve": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "tk_kv_truncate": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "tk_kv_seq_adopt": (C.c_int, [_P, C.c_int32, _I32P, C.c_int32, C.c_int32]),
    "tk_kv_seq_fork": (C.c_int, [_P, C.c_int32, _I32P, _P]),
    "tk_kv_seq_set_tail": (C.c_int, [_P, C.c_int32, C.c_int32]),
    "tk_kv_seq_len": (C.c_int, [_P, C.c_int32]),
    "tk_kv_num_free_pages": (C.c_int, [_P]),
    "tk_kv_page_table": (C.c_int, [_P, C.c_int32, _I32P, C.c_int32, _I32P]),
    "tk_kv_slot": (C.c_int64, [_P, C.c_int32, C.c_int32]),
    "tk_kv_state_digest": (C.c_uint64, [_P]),
    "tk_kv_state_save": (C.c_int, [_P, _I32P, C.c_int64, C.POINTER(C.c_int64)]),
    "tk_kv_state_load": (C.c_int, [_P, _I32P, C.c_int64]),
    "tk_kv_get_stats": (C.c_int, [_P, C.POINTER(KvStats)]),
    "tk_kv_step_begin": (C.c_int, [_P, C.c_int32, _I32P, _I32P, _P]),
    "tk_kv_step_begin_capped": (C.c_int, [_P, C.c_int32, _I32P, _I32P, _I32P, _P]),
    "tk_kv_set_num_heads": (C.c_int, [_P, C.c_int32]),
    "tk_kv_decode_ex": (C.c_int, [_P, C.c_int32, _P, C.c_int32, _P, C.c_int32, _P]),
    "tk_kv_step_num_tokens": (C.c_int, [_P]),
    "tk_kv_step_num_work_items": (C.c_int, [_P]),
    "tk_kv_step_chunk_tokens": (C.c_int, [_P]),
    "tk_kv_step_prefill_plan": (C.c_int, [_P, C.c_int32, _I32P, _I32P, _I32P, _I32P]),
    "tk_kv_append": (C.c_int, [_P, C.c_int32, _P, _P, _P, _P]),
    "tk_kv_decode": (C.c_int, [_P, C.c_int32, _P, _P, _P]),
    "tk_kv_append_decode": (C.c_int, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "tk_kv_rope_append_decode": (C.c_int, [_P, C.c_int32, _P, _P, _P, _P, C.c_float, C.c_float, _P]),
    "tk_kv_decode_partial": (C.c_int, [_P, C.c_int32, _P, _P, _P]),
    "tk_combine_partials": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, _P, C.c_int32, _P]),
    "tk_kv_append_decode_host": (C.c_int, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "tk_kv_append_decode_host_async": (C.c_int, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "tk_kv_host_wait": (C.c_int, [_P, _P]),
    "tk_peer_create": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(_P)]),
    "tk_peer_destroy": (None, [_P]),
    "tk_peer_last_error": (C.c_char_p, [_P]),
    "tk_peer_export": (C.c_int, [_P, C.c_void_p]),
    "tk_peer_connect": (C.c_int, [_P, C.c_void_p]),
    "tk_peer_mailbox": (C.c_void_p, [_P]),
    "tk_peer_mailbox_bytes": (C.c_size_t, [_P]),
    "tk_peer_connect_ptrs": (C.c_int, [_P, C.POINTER(C.c_void_p)]),
    "tk_peer_set_wait_limit_ms": (C.c_int, [_P, C.c_int32]),
    "tk_peer_exchange_combine": (C.c_int, [_P, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "tk_peer_send": (C.c_int, [_P, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "tk_peer_recv_combine": (C.c_int, [_P, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "tk_peer_status": (C.c_int, [_P, C.c_void_p]),
    "tk_kv_decode_multi": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tk_kv_decode_multi_ex": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "tk_kv_append_decode_multi": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tk_kv_decode_exchange": (C.c_int, [_P, C.c_int32, C.c_void_p, _P, C.c_void_p, C.c_void_p]),
    "tk_kv_profile_enable": (C.c_int, [_P, C.c_int32]),
    "tk_kv_profile_read": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "tk_kv_profile_read_each": (C.c_int, [_P, C.POINTER(C.c_float), C.c_int32, C.POINTER(C.c_int32)]),
    "tk_paged_decode_static": (C.c_int, [_P, C.c_int32, C.c_int32, _P, C.c_int32, _I32P, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_int32, _P, _P, _P]),
    "tk_kv_device_status": (C.c_int, [_P, _P]),
    "tk_kv_selftest_bounded_wait": (C.c_int, [_P, C.c_int32, _P]),
    "tk_kv_selftest_set_status": (C.c_int, [_P, C.c_int32, _P]),
    "tk_kv_check_canaries": (C.c_int, [_P, _P]),
    "tk_peer_check_canaries": (C.c_int, [_P, _P]),
    "tk_kv_launch_count": (C.c_int64, [_P]),
    "tk_sched_create": (C.c_int, [_P, C.POINTER(SchedConfig), C.POINTER(_P)]),
    "tk_sched_destroy": (C.c_int, [_P]),
    "tk_sched_submit": (C.c_int, [_P, C.c_int32, C.c_int32, _I32P]),
    "tk_sched_cancel": (C.c_int, [_P, C.c_int32]),
    "tk_sched_next": (C.c_int, [_P, C.c_int32, _I32P, _I32P, _I32P, _I32P, _I32P, _P]),
    "tk_sched_commit": (C.c_int, [_P, C.c_int32, _I32P]),
    "tk_sched_request_state": (C.c_int, [_P, C.c_int32, _I32P, _I32P, _I32P, _I32P]),
    "tk_sched_last_events": (C.c_int, [_P, C.c_int32, C.c_int32, _I32P, _I32P]),
    "tk_sched_get_stats": (C.c_int, [_P, C.POINTER(SchedStats)]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m titan_engine_b200.build` "
                "(there is no non-CUDA implementation to fall back to)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib
