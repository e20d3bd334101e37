"""ctypes/numpy binding of the CPU oracle (oracle/tk_oracle.c) and of the compiled
reference harness (oracle/ref_harness.cu).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of the benchmark.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_ref", "libtk_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libtitan_ref.so")

FP16, BF16, FP8 = 1, 2, 3
OK, INVALID_ARG, OUT_OF_PAGES = 0, 1, 2


def reference_root() -> str:
    """Root of the reference tree as BASELINE.json names it (`reference_path`), or "" when that
    file or that directory is absent (e.g. on a GPU box, which only has the prebuilt files)."""
    import json
    try:
        path = json.load(open(os.path.join(HERE, "..", "BASELINE.json"))).get("reference_path", "")
    except (OSError, ValueError):
        return ""
    return path if path and os.path.isdir(os.path.join(path, "src")) else ""


def build(ref: bool = True) -> None:
    """Compile the oracle (and, when the reference tree is present, the reference harness)."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    root = reference_root()
    if ref and root:
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={root}"], check=True)


class View(C.Structure):
    _fields_ = [("dtype", C.c_int), ("carrier_dtype", C.c_int), ("num_heads", C.c_int),
                ("num_kv_heads", C.c_int), ("head_dim", C.c_int), ("page_size", C.c_int),
                ("pool", C.c_void_p), ("scales", C.c_void_p), ("open_pages", C.c_void_p),
                ("page_table", C.c_void_p), ("max_pages_per_seq", C.c_int), ("v_head_dim", C.c_int)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        l = C.CDLL(ORACLE_SO)
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        sig = {
            "tko_e4m3_decode": (C.c_float, [C.c_uint8]),
            "tko_e4m3_encode": (C.c_uint8, [C.c_float]),
            "tko_f32_to_16": (None, [vp, vp, C.c_size_t, i]),
            "tko_16_to_f32": (None, [vp, vp, C.c_size_t, i]),
            "tko_kv_update_f32": (i, [vp, vp, i, i, i, i, i, i, vp, vp, i]),
            "tko_attention_decode_f32": (None, [vp, vp, vp, vp, i, i, i, i]),
            "tko_attention_decode_mla_f32": (None, [vp, vp, vp, vp, i, i, i, i, i]),
            "tko_append_16_kv": (None, [vp, i, i, i, i, vp, i, i, vp, vp, vp, vp, vp]),
            "tko_mgr_create": (vp, [i, i, i, i]),
            "tko_mgr_destroy": (None, [vp]),
            "tko_seq_alloc": (i, [vp]),
            "tko_seq_free": (i, [vp, i]),
            "tko_reserve": (i, [vp, i, i]),
            "tko_truncate": (i, [vp, i, i]),
            "tko_adopt": (i, [vp, i, vp, i, i]),
            "tko_mgr_enable_cold": (i, [vp, i, i]),
            "tko_evict_cold": (i, [vp, i, i]),
            "tko_num_cold_used": (i, [vp]),
            "tko_set_tail": (i, [vp, i, i]),
            "tko_fork": (i, [vp, i, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
            "tko_seq_len": (i, [vp, i]),
            "tko_seq_num_pages": (i, [vp, i]),
            "tko_num_free_pages": (i, [vp]),
            "tko_page_table": (C.POINTER(C.c_int32), [vp]),
            "tko_seq_lens": (C.POINTER(C.c_int32), [vp]),
            "tko_slot": (C.c_int64, [vp, i, i]),
            "tko_state_digest": (C.c_uint64, [vp]),
            "tko_append_16": (None, [vp, i, i, i, vp, i, i, vp, vp, vp, vp, vp]),
            "tko_append_fp8": (None, [vp, vp, vp, i, i, i, i, vp, i, i, vp, vp, vp, vp, vp]),
            "tko_gather_f32": (None, [C.POINTER(View), i, i, i, i, i, vp, vp]),
            "tko_decode_paged": (None, [C.POINTER(View), i, vp, vp, vp, vp]),
            "tko_decode_partial": (None, [C.POINTER(View), i, i, i, i, vp, vp, vp, vp]),
            "tko_combine": (None, [i, vp, vp, vp, i, vp]),
            "tko_rope_f32": (None, [vp, vp, i, i, i, i, f, f]),
            "tko_rope_mla_f32": (None, [vp, vp, i, i, i, i, i, f]),
            "tko_num_threads": (i, []),
            "tko_set_num_threads": (None, [i]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data


def _c(a, dt) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=dt)
    return a


# ---- conversions ------------------------------------------------------------------------
def f32_to_16(x: np.ndarray, dtype: int) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().tko_f32_to_16(_p(x), _p(out), x.size, dtype)
    return out


def to_f32(x: np.ndarray, dtype: int) -> np.ndarray:
    x = _c(x, np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().tko_16_to_f32(_p(x), _p(out), x.size, dtype)
    return out


def e4m3_decode_all() -> np.ndarray:
    return np.array([lib().tko_e4m3_decode(c) for c in range(256)], dtype=np.float32)


def e4m3_encode(x) -> np.ndarray:
    x = np.atleast_1d(np.asarray(x, dtype=np.float32))
    return np.array([lib().tko_e4m3_encode(float(v)) for v in x.ravel()], dtype=np.uint8).reshape(x.shape)


# ---- tier 1 -------------------------------------------------------------------------------
def attention_decode_f32(q, k_cache, v_cache, H, Hkv, D, seq_len) -> np.ndarray:
    q, k_cache, v_cache = _c(q, np.float32), _c(k_cache, np.float32), _c(v_cache, np.float32)
    out = np.empty((H, D), dtype=np.float32)
    lib().tko_attention_decode_f32(_p(q), _p(k_cache), _p(v_cache), _p(out), H, Hkv, D, seq_len)
    return out


def attention_decode_mla_f32(q, k_cache, v_cache, H, Hkv, Dk, Dv, seq_len) -> np.ndarray:
    q, k_cache, v_cache = _c(q, np.float32), _c(k_cache, np.float32), _c(v_cache, np.float32)
    out = np.empty((H, Dv), dtype=np.float32)
    lib().tko_attention_decode_mla_f32(_p(q), _p(k_cache), _p(v_cache), _p(out), H, Hkv, Dk, Dv, seq_len)
    return out


def kv_update_f32(k_data, v_data, L, max_seq, Hkv, D, layer, pos, key, value, seq_len) -> int:
    key, value = _c(key, np.float32), _c(value, np.float32)
    assert k_data.dtype == np.float32 and k_data.flags.c_contiguous
    return lib().tko_kv_update_f32(_p(k_data), _p(v_data), L, max_seq, Hkv, D, layer, pos, _p(key), _p(value), seq_len)


def rope_f32(q, k, H, Hkv, D, position, theta, scaling=1.0):
    q, k = _c(q, np.float32).copy(), _c(k, np.float32).copy()
    lib().tko_rope_f32(_p(q), _p(k), H, Hkv, D, position, theta, scaling)
    return q, k


def rope_mla_f32(q, k, H, Hkv, nope, rope, position, theta):
    q, k = _c(q, np.float32).copy(), _c(k, np.float32).copy()
    lib().tko_rope_mla_f32(_p(q), _p(k), H, Hkv, nope, rope, position, theta)
    return q, k


# ---- tier 2: manager ----------------------------------------------------------------------
class Manager:
    def __init__(self, num_pages, max_seqs, max_pages_per_seq, page_size=16):
        self.l = lib()
        self.num_pages, self.max_seqs, self.mpps, self.ps = num_pages, max_seqs, max_pages_per_seq, page_size
        self.h = self.l.tko_mgr_create(num_pages, max_seqs, max_pages_per_seq, page_size)
        assert self.h

    def __del__(self):
        if getattr(self, "h", None):
            self.l.tko_mgr_destroy(self.h)
            self.h = None

    def seq_alloc(self): return self.l.tko_seq_alloc(self.h)
    def seq_free(self, s): return self.l.tko_seq_free(self.h, s)
    def reserve(self, s, n): return self.l.tko_reserve(self.h, s, n)
    def truncate(self, s, n): return self.l.tko_truncate(self.h, s, n)

    def adopt(self, s, pages, seq_len):
        p = _c(pages, np.int32)
        return self.l.tko_adopt(self.h, s, _p(p), len(p), seq_len)

    def enable_cold(self, hot_window, num_cold_pages): return self.l.tko_mgr_enable_cold(self.h, hot_window, num_cold_pages)
    def evict_cold(self, s, stable_len): return self.l.tko_evict_cold(self.h, s, stable_len)
    def num_cold_used(self): return self.l.tko_num_cold_used(self.h)
    def set_tail(self, s, tail): return self.l.tko_set_tail(self.h, s, tail)
    def fork(self, parent):
        """-> (child slot or negative code, copy_src page, copy_dst page)"""
        a, b = C.c_int32(-1), C.c_int32(-1)
        child = self.l.tko_fork(self.h, parent, C.byref(a), C.byref(b))
        return child, a.value, b.value

    def seq_len(self, s): return self.l.tko_seq_len(self.h, s)
    def num_free_pages(self): return self.l.tko_num_free_pages(self.h)
    def slot(self, s, pos): return self.l.tko_slot(self.h, s, pos)
    def digest(self): return self.l.tko_state_digest(self.h)

    def table(self) -> np.ndarray:
        ptr = self.l.tko_page_table(self.h)
        return np.ctypeslib.as_array(ptr, shape=(self.max_seqs, self.mpps)).copy()

    def page_table(self, s) -> np.ndarray:
        n = self.l.tko_seq_num_pages(self.h, s)
        return self.table()[s, :n]


# ---- tier 2: pool ---------------------------------------------------------------------------
class Pool:
    """One layer of a paged pool in host memory, with the oracle's append and decode."""

    def __init__(self, dtype, num_pages, H, Hkv, D, max_seqs, max_pages_per_seq, page_size=16, carrier=None, Dv=None):
        self.dtype, self.carrier = dtype, (carrier or (BF16 if dtype == FP8 else dtype))
        self.num_pages, self.H, self.Hkv, self.D = num_pages, H, Hkv, D
        self.Dv = Dv or D                      # V rows / output width (differs from D for the MLA cache)
        self.max_seqs, self.mpps, self.ps = max_seqs, max_pages_per_seq, page_size
        # tile of (page, kv head): page_size K rows of D, then page_size V rows of Dv
        shape = (num_pages, Hkv, 2, page_size, D) if self.Dv == D else (num_pages, Hkv, page_size * (D + self.Dv))
        if dtype == FP8:
            self.pool = np.zeros(shape, dtype=np.uint8)
            self.scales = np.zeros((num_pages, Hkv, 2), dtype=np.float32)
            self.open_pages = np.zeros((max_seqs, Hkv, 2, page_size, D), dtype=np.uint16)
        else:
            self.pool = np.zeros(shape, dtype=np.uint16)
            self.scales = None
            self.open_pages = None

    def append(self, table: np.ndarray, tok_seq, tok_pos, k16: np.ndarray, v16: np.ndarray) -> np.ndarray:
        table, tok_seq, tok_pos = _c(table, np.int32), _c(tok_seq, np.int32), _c(tok_pos, np.int32)
        k16, v16 = _c(k16, np.uint16), _c(v16, np.uint16)
        n = len(tok_seq)
        slots = np.empty(n, dtype=np.int64)
        if self.dtype == FP8:
            lib().tko_append_fp8(_p(self.pool), _p(self.scales), _p(self.open_pages), self.carrier,
                                 self.Hkv, self.D, self.ps, _p(table), self.mpps, n, _p(tok_seq),
                                 _p(tok_pos), _p(k16), _p(v16), _p(slots))
        else:
            lib().tko_append_16_kv(_p(self.pool), self.Hkv, self.D, self.Dv, self.ps, _p(table), self.mpps, n,
                                   _p(tok_seq), _p(tok_pos), _p(k16), _p(v16), _p(slots))
        return slots

    def view(self, table: np.ndarray) -> View:
        self._table = _c(table, np.int32)
        return View(self.dtype, self.carrier, self.H, self.Hkv, self.D, self.ps, _p(self.pool),
                    _p(self.scales), _p(self.open_pages), _p(self._table), self.mpps, self.Dv)

    def decode(self, table, seq_ids, seq_lens, q16) -> np.ndarray:
        seq_ids, seq_lens, q16 = _c(seq_ids, np.int32), _c(seq_lens, np.int32), _c(q16, np.uint16)
        out = np.empty((len(seq_ids), self.H, self.Dv), dtype=np.float32)
        v = self.view(table)
        lib().tko_decode_paged(C.byref(v), len(seq_ids), _p(seq_ids), _p(seq_lens), _p(q16), _p(out))
        return out

    def decode_partial(self, table, seq, seq_len, t0, t1, q16):
        q16 = _c(q16, np.uint16)
        m = np.empty(self.H, dtype=np.float32)
        l = np.empty(self.H, dtype=np.float32)
        o = np.empty((self.H, self.Dv), dtype=np.float32)
        v = self.view(table)
        lib().tko_decode_partial(C.byref(v), seq, seq_len, t0, t1, _p(q16), _p(m), _p(l), _p(o))
        return m, l, o

    def gather(self, table, seq, seq_len, kvh, t0, t1):
        k = np.empty((t1 - t0, self.D), dtype=np.float32)
        vv = np.empty((t1 - t0, self.Dv), dtype=np.float32)
        v = self.view(table)
        lib().tko_gather_f32(C.byref(v), seq, seq_len, kvh, t0, t1, _p(k), _p(vv))
        return k, vv


def combine(m, l, o) -> np.ndarray:
    m, l, o = _c(m, np.float32), _c(l, np.float32), _c(o, np.float32)
    out = np.empty(o.shape[1], dtype=np.float32)
    lib().tko_combine(len(m), _p(m), _p(l), _p(o), o.shape[1], _p(out))
    return out


def num_threads() -> int:
    return lib().tko_num_threads()


def set_num_threads(n: int) -> None:
    lib().tko_set_num_threads(int(n))


# ---- the compiled reference (GPU only) ---------------------------------------------------------
_ref = None


def ref_lib() -> Optional[C.CDLL]:
    """libtitan_ref.so = the reference's attention.cu + kv_cache.cpp, or None if not built."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        r = C.CDLL(REF_SO)
        vp, i, f = C.c_void_p, C.c_int, C.c_float
        r.tkref_update_and_decode.restype = i
        r.tkref_update_and_decode.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, C.POINTER(C.c_int)]
        r.tkref_attention_decode.restype = i
        r.tkref_attention_decode.argtypes = [vp, vp, vp, vp, i, i, i, i]
        r.tkref_attention_decode_mla.restype = i
        r.tkref_attention_decode_mla.argtypes = [vp, vp, vp, vp, i, i, i, i, i]
        r.tkref_apply_rope.restype = i
        r.tkref_apply_rope.argtypes = [vp, vp, i, i, i, i, f, f]
        r.tkref_apply_rope_mla.restype = i
        r.tkref_apply_rope_mla.argtypes = [vp, vp, i, i, i, i, i, f]
        _ref = r
    return _ref


def ref_attention_decode(q, k, v, H, Hkv, D, seq_len) -> np.ndarray:
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    out = np.empty((H, D), dtype=np.float32)
    st = ref_lib().tkref_attention_decode(_p(q), _p(k), _p(v), _p(out), H, Hkv, D, seq_len)
    if st != 0:
        raise RuntimeError(f"reference attention_decode failed: cudaError {st}")
    return out


def ref_attention_decode_mla(q, k, v, H, Hkv, Dk, Dv, seq_len) -> np.ndarray:
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    out = np.empty((H, Dv), dtype=np.float32)
    st = ref_lib().tkref_attention_decode_mla(_p(q), _p(k), _p(v), _p(out), H, Hkv, Dk, Dv, seq_len)
    if st != 0:
        raise RuntimeError(f"reference attention_decode_mla failed: cudaError {st}")
    return out


def ref_update_and_decode(k, v, q, L, layer, H, Hkv, D, seq_len, max_seq_len):
    k, v, q = _c(k, np.float32), _c(v, np.float32), _c(q, np.float32)
    out = np.empty((H, D), dtype=np.float32)
    n = C.c_int(0)
    st = ref_lib().tkref_update_and_decode(_p(k), _p(v), _p(q), _p(out), L, layer, H, Hkv, D, seq_len,
                                           max_seq_len, C.byref(n))
    if st != 0:
        raise RuntimeError(f"reference update+decode failed: cudaError {st}")
    return out, n.value


def ref_apply_rope_mla(q, k, H, Hkv, nope, rope, position, theta):
    q, k = _c(q, np.float32).copy(), _c(k, np.float32).copy()
    st = ref_lib().tkref_apply_rope_mla(_p(q), _p(k), H, Hkv, nope, rope, position, theta)
    if st != 0:
        raise RuntimeError(f"reference apply_rope_mla failed: cudaError {st}")
    return q, k


def ref_apply_rope(q, k, H, Hkv, D, position, theta, scaling=1.0):
    q, k = _c(q, np.float32).copy(), _c(k, np.float32).copy()
    st = ref_lib().tkref_apply_rope(_p(q), _p(k), H, Hkv, D, position, theta, scaling)
    if st != 0:
        raise RuntimeError(f"reference apply_rope failed: cudaError {st}")
    return q, k
