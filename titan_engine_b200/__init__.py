"""B200 (sm_100a) paged KV-cache hot path: page manager, K/V append, paged GQA decode attention.

The compute lives in libtitan_kv.so (hand-written CUDA behind the C ABI of include/titan_kv.h);
this package is the host-side mirror of that interface.
"""
from ._lib import (TK_OK, TK_INVALID_ARG, TK_OUT_OF_PAGES, TK_CUDA_ERROR, TK_TIMEOUT, TK_OUT_OF_SEQS,
                   TK_UNSUPPORTED, TK_FP16, TK_BF16, TK_FP8_E4M3, lib)
from .kv import KvError, PagedKVCache

__all__ = ["PagedKVCache", "KvError", "lib"]
