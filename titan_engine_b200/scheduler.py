"""Continuous batching over the paged KV cache: thin object over the tk_sched_* C ABI.

Stands where the reference has `BatchScheduler` (src/inference/batch.h:75-140); the scheduling
itself is C++ (titan_engine_b200/csrc/kv_scheduler.cpp)."""
from __future__ import annotations

import ctypes as C
from typing import List, NamedTuple, Sequence

import numpy as np

from . import _lib as L
from .kv import KvError, PagedKVCache

STATES = ("queued", "prefilling", "decoding", "finished", "cancelled")


class Row(NamedTuple):
    req_id: int
    seq: int
    n_new: int
    samples: bool


class BatchScheduler:
    def __init__(self, cache: PagedKVCache, max_batch_size: int = 8, max_prefill_tokens: int = 2048):
        self._lib, self.cache = L.lib(), cache
        cfg = L.SchedConfig(max_batch_size, max_prefill_tokens)
        self._h = C.c_void_p()
        st = self._lib.tk_sched_create(cache._h, C.byref(cfg), C.byref(self._h))
        if st != L.TK_OK:
            raise KvError(st, "tk_sched_create: bad configuration (max_prefill_tokens + max_batch_size must fit "
                              "the cache's max_step_tokens)")
        self._cap = max_batch_size
        self._n_rows = 0

    def close(self):
        if self._h.value:
            self._lib.tk_sched_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, prompt_tokens: int, max_output_tokens: int) -> int:
        rid = C.c_int32(-1)
        st = self._lib.tk_sched_submit(self._h, prompt_tokens, max_output_tokens, C.byref(rid))
        if st != L.TK_OK:
            raise KvError(st, f"submit({prompt_tokens}, {max_output_tokens}): does not fit a sequence of this cache")
        return rid.value

    def cancel(self, request_id: int) -> bool:
        return self._lib.tk_sched_cancel(self._h, request_id) == L.TK_OK

    def next(self) -> List[Row]:
        """One scheduling iteration; the step is begun on the cache (current stream)."""
        a = [np.zeros(self._cap, dtype=np.int32) for _ in range(4)]
        n = C.c_int32(0)
        p = [x.ctypes.data_as(C.POINTER(C.c_int32)) for x in a]
        stream = None if self.cache.host_only else self.cache._stream()
        st = self._lib.tk_sched_next(self._h, self._cap, p[0], p[1], p[2], p[3], C.byref(n), stream)
        if st != L.TK_OK:
            raise KvError(st, self._lib.tk_kv_last_error(self.cache._h).decode())
        self._n_rows = n.value
        self.cache._n_seqs = n.value
        self.cache._n_tokens = self._lib.tk_kv_step_num_tokens(self.cache._h)
        return [Row(int(a[0][i]), int(a[1][i]), int(a[2][i]), bool(a[3][i])) for i in range(n.value)]

    def commit(self, finished: Sequence[bool]) -> None:
        f = np.ascontiguousarray(np.asarray(finished, dtype=np.int32))
        assert len(f) == self._n_rows
        st = self._lib.tk_sched_commit(self._h, len(f), f.ctypes.data_as(C.POINTER(C.c_int32)))
        if st != L.TK_OK:
            raise KvError(st, "commit: row count does not match the last step")

    def request(self, request_id: int) -> dict:
        v = [C.c_int32(0) for _ in range(4)]
        st = self._lib.tk_sched_request_state(self._h, request_id, *[C.byref(x) for x in v])
        if st != L.TK_OK:
            raise KvError(st, f"unknown request {request_id}")
        return {"state": STATES[v[0].value], "seq": v[1].value, "prefill_pos": v[2].value, "output_tokens": v[3].value}

    def last_events(self) -> dict:
        out = {}
        for which, name in enumerate(("retired", "admitted", "preempted")):
            buf = np.zeros(4096, dtype=np.int32)
            n = C.c_int32(0)
            self._lib.tk_sched_last_events(self._h, which, len(buf), buf.ctypes.data_as(C.POINTER(C.c_int32)), C.byref(n))
            out[name] = buf[:n.value].tolist()
        return out

    def stats(self) -> dict:
        s = L.SchedStats()
        self._lib.tk_sched_get_stats(self._h, C.byref(s))
        return {n: getattr(s, n) for n, _ in L.SchedStats._fields_}
