"""Host-side Python mirror of the paged KV-cache C ABI.

`PagedKVCache` is a thin object over the handle from include/titan_kv.h: the same
calls, torch tensors for device memory and streams.  It stands where the reference
has `titan::KVCache` (src/inference/kv_cache.h:15-81) and
`titan::cuda::attention_decode` (src/compute/dispatch.h:73-75).  All compute runs in
libtitan_kv.so; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib as L

_DTYPES = {"fp16": L.TK_FP16, "bf16": L.TK_BF16, "fp8_e4m3": L.TK_FP8_E4M3, "fp8": L.TK_FP8_E4M3}
_TORCH16 = {L.TK_FP16: torch.float16, L.TK_BF16: torch.bfloat16}
_IMPLS = {"auto": L.TK_DECODE_AUTO, "simt": L.TK_DECODE_SIMT, "mma": L.TK_DECODE_MMA}


class KvError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{L.lib().tk_status_str(status).decode()}] {message}")
        self.status = status


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))


class PagedKVCache:
    """Paged K/V pool + page manager + decode attention for one GPU."""

    live = weakref.WeakSet()        # every open device-backed cache of this process (see check_canaries)

    def __init__(self, num_layers: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 num_pages: int, max_seqs: int, max_pages_per_seq: int, dtype: str = "bf16",
                 io_dtype: Optional[str] = None, page_size: int = 16,
                 max_step_tokens: Optional[int] = None, chunk_tokens: int = 0,
                 decode_impl: str = "auto", device: Optional[int] = None, host_only: bool = False,
                 hot_window: int = 0, cold_pages: int = 0, v_head_dim: int = 0, separate_combine: bool = False,
                 launch_overlap: bool = True, prefill_impl: str = "auto"):
        self._lib = L.lib()
        cfg = L.KvConfig()
        self._lib.tk_kv_config_default(C.byref(cfg))
        cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = num_layers, num_heads, num_kv_heads, head_dim
        cfg.page_size, cfg.dtype = page_size, _DTYPES[dtype]
        cfg.io_dtype = _DTYPES[io_dtype] if io_dtype else (L.TK_BF16 if cfg.dtype == L.TK_FP8_E4M3 else cfg.dtype)
        cfg.num_pages, cfg.max_seqs, cfg.max_pages_per_seq = num_pages, max_seqs, max_pages_per_seq
        cfg.max_step_tokens = max_step_tokens or max_seqs
        cfg.chunk_tokens, cfg.decode_impl = chunk_tokens, _IMPLS[decode_impl]
        cfg.hot_window, cfg.cold_pages, cfg.v_head_dim = hot_window, cold_pages, v_head_dim
        cfg.merge_impl = L.TK_MERGE_SEPARATE if separate_combine else L.TK_MERGE_IN_KERNEL
        cfg.launch_overlap = L.TK_OVERLAP_AUTO if launch_overlap else L.TK_OVERLAP_OFF
        cfg.prefill_impl = {"auto": L.TK_PREFILL_AUTO, "mma_sync": L.TK_PREFILL_MMA_SYNC}[prefill_impl]
        self._h = C.c_void_p()
        self.host_only = host_only
        self._arena = None
        if host_only:
            cfg.device = L.TK_DEVICE_NONE
            st = self._lib.tk_kv_create(C.byref(cfg), C.byref(self._h))
        else:
            if not torch.cuda.is_available():
                raise KvError(L.TK_CUDA_ERROR, "no CUDA device: the paged KV path has no CPU implementation")
            dev = torch.cuda.current_device() if device is None else device
            cfg.device = dev
            self.device = torch.device("cuda", dev)
            nbytes = self._lib.tk_kv_arena_bytes(C.byref(cfg))
            if nbytes == 0:
                raise KvError(L.TK_INVALID_ARG, "invalid configuration")
            guard = 4096                                     # room for the library's guard bytes behind the arena
            self._arena = torch.empty(nbytes + 1024 + guard, dtype=torch.uint8, device=self.device)
            self._arena_off = (-self._arena.data_ptr()) % 1024
            torch.cuda.synchronize(self.device)
            st = self._lib.tk_kv_create_external(C.byref(cfg), self._arena.data_ptr() + self._arena_off,
                                                 nbytes + guard, C.byref(self._h))
        if st != L.TK_OK:
            raise KvError(st, self._lib.tk_kv_last_error(None).decode())
        self.cfg = L.KvConfig()
        self._lib.tk_kv_get_config(self._h, C.byref(self.cfg))
        self.io_torch_dtype = _TORCH16[self.cfg.io_dtype]
        self._n_seqs = 0
        self._n_tokens = 0
        if not host_only:
            PagedKVCache.live.add(self)

    # ---- plumbing ------------------------------------------------------------------
    def _check(self, st: int) -> None:
        if st != L.TK_OK:
            raise KvError(st, self._lib.tk_kv_last_error(self._h).decode())

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            self._lib.tk_kv_destroy(self._h)
            self._h = C.c_void_p()
        self._arena = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- sequences and pages --------------------------------------------------------
    def seq_alloc(self) -> int:
        s = C.c_int32(-1)
        self._check(self._lib.tk_kv_seq_alloc(self._h, C.byref(s)))
        return s.value

    def seq_free(self, seq: int) -> None:
        self._check(self._lib.tk_kv_seq_free(self._h, seq))

    def reserve(self, seq: int, n_tokens: int) -> None:
        self._check(self._lib.tk_kv_reserve(self._h, seq, n_tokens))

    def truncate(self, seq: int, new_len: int) -> None:
        self._check(self._lib.tk_kv_truncate(self._h, seq, new_len))

    def adopt(self, seq: int, pages: Sequence[int], seq_len: int) -> None:
        p = _i32(pages)
        self._check(self._lib.tk_kv_seq_adopt(self._h, seq, _ptr(p), len(p), seq_len))

    def fork(self, parent: int) -> int:
        """New sequence sharing `parent`'s full pages; its partly filled last page is copied."""
        child = C.c_int32(-1)
        stream = None if self.host_only else self._stream()
        self._check(self._lib.tk_kv_seq_fork(self._h, parent, C.byref(child), stream))
        return child.value

    def set_tail(self, seq: int, tail_tokens: int) -> None:
        """Tokens of this logical sequence held by later ranks (moves the hot window)."""
        self._check(self._lib.tk_kv_seq_set_tail(self._h, seq, tail_tokens))

    def seq_len(self, seq: int) -> int:
        return self._lib.tk_kv_seq_len(self._h, seq)

    @property
    def num_free_pages(self) -> int:
        return self._lib.tk_kv_num_free_pages(self._h)

    def page_table(self, seq: int) -> np.ndarray:
        n = C.c_int32(0)
        self._check(self._lib.tk_kv_page_table(self._h, seq, None, 0, C.byref(n)))
        out = np.empty(n.value, dtype=np.int32)
        self._check(self._lib.tk_kv_page_table(self._h, seq, _ptr(out), n.value, C.byref(n)))
        return out

    def slot(self, seq: int, pos: int) -> int:
        return self._lib.tk_kv_slot(self._h, seq, pos)

    def digest(self) -> int:
        return self._lib.tk_kv_state_digest(self._h)

    def state_save(self) -> np.ndarray:
        """Allocator + page-table state as a flat int32 image (see tk_kv_state_save)."""
        n = C.c_int64(0)
        self._check(self._lib.tk_kv_state_save(self._h, None, 0, C.byref(n)))
        image = np.zeros(n.value, dtype=np.int32)
        self._check(self._lib.tk_kv_state_save(self._h, _ptr(image), n.value, C.byref(n)))
        return image

    def state_load(self, image: np.ndarray) -> None:
        image = _i32(image)
        self._check(self._lib.tk_kv_state_load(self._h, _ptr(image), len(image)))

    def stats(self) -> dict:
        s = L.KvStats()
        self._check(self._lib.tk_kv_get_stats(self._h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in L.KvStats._fields_}

    @property
    def launch_count(self) -> int:
        return self._lib.tk_kv_launch_count(self._h)

    @property
    def memory_bytes(self) -> int:
        return self._lib.tk_kv_memory_bytes(self._h)

    # ---- one step -----------------------------------------------------------------------
    def step_begin(self, seq_ids: Sequence[int], n_new: Optional[Sequence[int]] = None) -> None:
        s = _i32(seq_ids)
        n = None if n_new is None else _i32(n_new)
        stream = None if self.host_only else self._stream()
        self._check(self._lib.tk_kv_step_begin(self._h, len(s), _ptr(s), _ptr(n), stream))
        self._n_seqs = len(s)
        self._n_tokens = self._lib.tk_kv_step_num_tokens(self._h)

    @property
    def step_num_tokens(self) -> int:
        return self._lib.tk_kv_step_num_tokens(self._h)

    @property
    def step_num_work_items(self) -> int:
        return self._lib.tk_kv_step_num_work_items(self._h)

    @property
    def step_chunk_tokens(self) -> int:
        return self._lib.tk_kv_step_chunk_tokens(self._h)

    def step_prefill_plan(self):
        """-> (items [n, 4] int32: (sequence index, chunk, kv head, tile), chunk tokens per sequence, decode-kernel items)
        of the prefill attention kernel for the current step; n == 0 when the step does not use it."""
        n, nd = C.c_int32(0), C.c_int32(0)
        self._check(self._lib.tk_kv_step_prefill_plan(self._h, 0, None, C.byref(n), None, C.byref(nd)))
        items = np.zeros((n.value, 4), dtype=np.int32)
        ct = np.zeros(max(self._n_seqs, 1), dtype=np.int32)
        if n.value:
            self._check(self._lib.tk_kv_step_prefill_plan(self._h, n.value, _ptr(items), C.byref(n), _ptr(ct), C.byref(nd)))
        return items, ct[:self._n_seqs], nd.value

    def _check_io(self, t: torch.Tensor, rows: int, heads: int, what: str) -> None:
        dim = self.cfg.v_head_dim if what in ("v", "out") else self.cfg.head_dim
        if t.device != self.device or t.dtype != self.io_torch_dtype or not t.is_contiguous():
            raise KvError(L.TK_INVALID_ARG, f"{what}: need a contiguous {self.io_torch_dtype} tensor on {self.device}")
        if t.numel() != rows * heads * dim:
            raise KvError(L.TK_INVALID_ARG, f"{what}: expected [{rows}, {heads}, {dim}]")

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor,
               slots_out: Optional[torch.Tensor] = None) -> None:
        """k, v: [n_tokens, Hkv, D] on the device, io dtype; the step's tokens in order."""
        self._check_io(k, self._n_tokens, self.cfg.num_kv_heads, "k")
        self._check_io(v, self._n_tokens, self.cfg.num_kv_heads, "v")
        sp = None
        if slots_out is not None:
            assert slots_out.dtype == torch.int64 and slots_out.numel() >= self._n_tokens
            sp = slots_out.data_ptr()
        self._check(self._lib.tk_kv_append(self._h, layer, k.data_ptr(), v.data_ptr(), sp, self._stream()))

    def decode(self, layer: int, q: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """q: [n_seqs, H, D] -> out [n_seqs, H, D], io dtype."""
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(q.shape[0], self.cfg.num_heads, self.cfg.v_head_dim, dtype=q.dtype, device=q.device)
        self._check_io(out, self._n_seqs, self.cfg.num_heads, "out")
        self._check(self._lib.tk_kv_decode(self._h, layer, q.data_ptr(), out.data_ptr(), self._stream()))
        return out

    def decode_f32(self, layer: int, q: torch.Tensor) -> torch.Tensor:
        """decode() with the result left in FP32 (tk_kv_decode_ex): q [n_seqs, H, D] io dtype -> [n_seqs, H, Dv] f32."""
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        out = torch.empty(q.shape[0], self.cfg.num_heads, self.cfg.v_head_dim, dtype=torch.float32, device=q.device)
        self._check(self._lib.tk_kv_decode_ex(self._h, layer, q.data_ptr(), self.cfg.io_dtype, out.data_ptr(),
                                              L.TK_FP32, self._stream()))
        return out

    def decode_multi_f32(self, layer: int, q: torch.Tensor) -> torch.Tensor:
        """decode_multi() with the result left in FP32 (tk_kv_decode_multi_ex)."""
        self._check_io(q, self._n_tokens, self.cfg.num_heads, "q")
        out = torch.empty(self._n_tokens, self.cfg.num_heads, self.cfg.v_head_dim, dtype=torch.float32, device=self.device)
        self._check(self._lib.tk_kv_decode_multi_ex(self._h, layer, q.data_ptr(), out.data_ptr(), L.TK_FP32, self._stream()))
        return out

    def append_decode(self, layer: int, k: torch.Tensor, v: torch.Tensor, q: torch.Tensor,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """append + decode of one layer; a single fused kernel on 16-bit decode steps."""
        self._check_io(k, self._n_tokens, self.cfg.num_kv_heads, "k")
        self._check_io(v, self._n_tokens, self.cfg.num_kv_heads, "v")
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(q.shape[0], self.cfg.num_heads, self.cfg.v_head_dim, dtype=q.dtype, device=q.device)
        self._check(self._lib.tk_kv_append_decode(self._h, layer, k.data_ptr(), v.data_ptr(), q.data_ptr(),
                                                  out.data_ptr(), self._stream()))
        return out

    def rope_append_decode(self, layer: int, k: torch.Tensor, v: torch.Tensor, q: torch.Tensor,
                           theta: float, scaling: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """RoPE(q, k) + append + decode of one layer; q and k are given before rotation."""
        self._check_io(k, self._n_tokens, self.cfg.num_kv_heads, "k")
        self._check_io(v, self._n_tokens, self.cfg.num_kv_heads, "v")
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(q.shape[0], self.cfg.num_heads, self.cfg.v_head_dim, dtype=q.dtype, device=q.device)
        self._check(self._lib.tk_kv_rope_append_decode(self._h, layer, k.data_ptr(), v.data_ptr(), q.data_ptr(),
                                                       out.data_ptr(), theta, scaling, self._stream()))
        return out

    def decode_partial(self, layer: int, q: torch.Tensor, partial: Optional[torch.Tensor] = None) -> torch.Tensor:
        """-> [n_seqs, H, D+2] f32: unnormalised o, then m, then l."""
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        if partial is None:
            partial = torch.empty(self._n_seqs, self.cfg.num_heads, self.cfg.v_head_dim + 2,
                                  dtype=torch.float32, device=self.device)
        self._check(self._lib.tk_kv_decode_partial(self._h, layer, q.data_ptr(), partial.data_ptr(), self._stream()))
        return partial

    def decode_multi(self, layer: int, q: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Causal attention for every token the step appended: q, out [n_tokens, H, D] (rows as in append)."""
        self._check_io(q, self._n_tokens, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(self._n_tokens, self.cfg.num_heads, self.cfg.v_head_dim, dtype=self.io_torch_dtype,
                              device=self.device)
        self._check(self._lib.tk_kv_decode_multi(self._h, layer, q.data_ptr(), out.data_ptr(), self._stream()))
        return out

    def append_decode_multi(self, layer: int, k: torch.Tensor, v: torch.Tensor, q: torch.Tensor,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """append(k, v) of the step's tokens, then decode_multi(q): one library call per layer."""
        self._check_io(k, self._n_tokens, self.cfg.num_kv_heads, "k")
        self._check_io(v, self._n_tokens, self.cfg.num_kv_heads, "v")
        self._check_io(q, self._n_tokens, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(self._n_tokens, self.cfg.num_heads, self.cfg.v_head_dim, dtype=self.io_torch_dtype,
                              device=self.device)
        self._check(self._lib.tk_kv_append_decode_multi(self._h, layer, k.data_ptr(), v.data_ptr(), q.data_ptr(),
                                                        out.data_ptr(), self._stream()))
        return out

    def decode_exchange(self, layer: int, q: torch.Tensor, exchange, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention over the tokens of EVERY rank of `exchange` (a dist.PeerExchange): this rank's
        partial rows, then one kernel that swaps rows with the peers over NVLink and combines."""
        self._check_io(q, self._n_seqs, self.cfg.num_heads, "q")
        if out is None:
            out = torch.empty(self._n_seqs, self.cfg.num_heads, self.cfg.v_head_dim, dtype=self.io_torch_dtype,
                              device=self.device)
        self._check(self._lib.tk_kv_decode_exchange(self._h, layer, q.data_ptr(), exchange._h, out.data_ptr(),
                                                    self._stream()))
        return out

    def append_decode_host(self, layer: int, k: torch.Tensor, v: torch.Tensor, q: torch.Tensor,
                           out: torch.Tensor) -> None:
        """Host (CPU, ideally pinned) tensors in and out; copies are part of the call."""
        for t in (k, v, q, out):
            assert t.device.type == "cpu" and t.is_contiguous() and t.dtype == self.io_torch_dtype
        self._check(self._lib.tk_kv_append_decode_host(self._h, layer, k.data_ptr(), v.data_ptr(),
                                                       q.data_ptr(), out.data_ptr(), self._stream()))

    def append_decode_host_async(self, layer: int, k, v, q, out) -> None:
        """As append_decode_host but returns at once; pinned host tensors, caller syncs the stream."""
        for t in (k, v, q, out):
            assert t.device.type == "cpu" and t.is_contiguous() and t.is_pinned() and t.dtype == self.io_torch_dtype
        self._check(self._lib.tk_kv_append_decode_host_async(self._h, layer, k.data_ptr(), v.data_ptr(),
                                                             q.data_ptr(), out.data_ptr(), self._stream()))

    def host_wait(self) -> None:
        """Current stream waits for the device-to-host copies queued by append_decode_host_async."""
        self._check(self._lib.tk_kv_host_wait(self._h, self._stream()))

    def profile_enable(self, max_launches: int) -> None:
        self._check(self._lib.tk_kv_profile_enable(self._h, max_launches))

    def profile_read(self):
        """-> (summed decode-kernel milliseconds, launches) since profile_enable."""
        ms, n = C.c_double(0.0), C.c_int64(0)
        self._check(self._lib.tk_kv_profile_read(self._h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def profile_read_each(self, cap: int) -> np.ndarray:
        """-> per-launch decode-kernel milliseconds (launch order) since profile_enable."""
        buf = np.zeros(max(cap, 1), dtype=np.float32)
        n = C.c_int32(0)
        self._check(self._lib.tk_kv_profile_read_each(self._h, buf.ctypes.data_as(C.POINTER(C.c_float)), cap,
                                                      C.byref(n)))
        return buf[:min(n.value, cap)].copy()

    def device_status(self) -> None:
        self._check(self._lib.tk_kv_device_status(self._h, self._stream()))

    def check_canaries(self) -> None:
        """Raises when a kernel wrote past the end of the arena, the page table, the split-KV workspace
        or the step metadata (guard bytes behind each are compared)."""
        if getattr(self, "_h", None) and self._h.value and not self.host_only:
            self._check(self._lib.tk_kv_check_canaries(self._h, self._stream()))

    def selftest_set_status(self, value: int) -> None:
        self._check(self._lib.tk_kv_selftest_set_status(self._h, value, self._stream()))

    # ---- views of the pool (parity dumps, synthetic fills) -------------------------------
    def _view(self, ptr: int, nbytes: int) -> torch.Tensor:
        off = ptr - self._arena.data_ptr()
        return self._arena[off:off + nbytes]

    def layer_views(self, layer: int):
        """(pool, scales, open_pages) tensors aliasing layer `layer` of the arena.
        pool: [num_pages, Hkv, 2, page, D] (uint8 codes for FP8); scales: [num_pages, Hkv, 2] f32 or None;
        open_pages: [max_seqs, Hkv, 2, page, D] io dtype or None."""
        p, s, o = C.c_void_p(), C.c_void_p(), C.c_void_p()
        self._check(self._lib.tk_kv_layer_ptrs(self._h, layer, C.byref(p), C.byref(s), C.byref(o)))
        c = self.cfg
        shape = (c.num_pages, c.num_kv_heads, 2, c.page_size, c.head_dim)
        n = int(np.prod(shape))
        if c.dtype == L.TK_FP8_E4M3:
            pool = self._view(p.value, n).view(shape)
            scales = self._view(s.value, c.num_pages * c.num_kv_heads * 2 * 4).view(torch.float32).view(
                c.num_pages, c.num_kv_heads, 2)
            oshape = (c.max_seqs, c.num_kv_heads, 2, c.page_size, c.head_dim)
            open_pages = self._view(o.value, int(np.prod(oshape)) * 2).view(self.io_torch_dtype).view(oshape)
            return pool, scales, open_pages
        if c.v_head_dim != c.head_dim:        # MLA tile: page_size K rows of head_dim, then V rows of v_head_dim
            shape = (c.num_pages, c.num_kv_heads, c.page_size * (c.head_dim + c.v_head_dim))
            n = int(np.prod(shape))
        pool = self._view(p.value, n * 2).view(_TORCH16[c.dtype]).view(shape)
        return pool, None, None
