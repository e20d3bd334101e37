"""Multi-GPU partitioning of the paged KV path: one process per GPU, torch.distributed for the
plumbing.

The reference is single-GPU (GPU 0 only: src/memory/memory_manager.cpp:15); this module defines
how the path shards:

  * batched decode — by sequence (default) or by kv head: independent units, no collective;
  * one very long sequence — contiguous page-aligned token ranges per rank; every rank computes
    the merged, unnormalised (o, m, l) of its range; per layer either ONE kernel stores the rows
    into every peer's memory over NVLink, waits for the peers' rows and combines (PeerExchange),
    or ONE all-gather of [n_seqs][H][D+2] floats exchanges them and the log-sum-exp combine
    kernel consumes the gathered buffer (portable route).

Nothing here computes attention: partials and the combine come from libtitan_kv.so (or, in the
CPU tests of this logic, from the oracle through the same two callables).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_sequences(n_seqs: int, rank: int, world: int) -> range:
    """Contiguous block of sequence indices for `rank`; sizes differ by at most one."""
    base, extra = divmod(n_seqs, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def shard_kv_heads(num_kv_heads: int, num_heads: int, rank: int, world: int) -> Tuple[range, range]:
    """(kv heads, query heads) of `rank` when the batch is smaller than the world: rank r holds
    kv heads [r*Hkv/world, ...) and the query heads that map onto them (kv = h // (H/Hkv))."""
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} kv heads do not split over {world} ranks")
    per = num_kv_heads // world
    g = num_heads // num_kv_heads
    return range(rank * per, (rank + 1) * per), range(rank * per * g, (rank + 1) * per * g)


def token_ranges(n_tokens: int, world: int, page_size: int = 16) -> List[Tuple[int, int]]:
    """Contiguous, page-aligned [start, end) token range of every rank for one long sequence.
    Pages are dealt out as evenly as possible; trailing ranks may be empty for short sequences."""
    n_pages = (n_tokens + page_size - 1) // page_size
    out = []
    for r in range(world):
        pr = shard_sequences(n_pages, r, world)
        out.append((min(pr.start * page_size, n_tokens), min(pr.stop * page_size, n_tokens)))
    return out


def hot_cold_split(rng_tokens: Tuple[int, int], seq_len: int, hot_window: int, page_size: int = 16) -> Tuple[int, int]:
    """(cold tokens, hot tokens) of a rank's range: a page is cold iff its last token index is
    below seq_len - hot_window."""
    lo, hi = rng_tokens
    if hot_window <= 0:
        return 0, hi - lo
    limit = seq_len - hot_window
    cold_end = lo
    p = lo
    while p < hi:
        last = min(p + page_size, hi) - 1
        if last < limit:
            cold_end = min(p + page_size, hi)
        else:
            break
        p += page_size
    return cold_end - lo, hi - cold_end


class LongContextDecoder:
    """Decode attention for sequences whose tokens are spread over the ranks of `group`.

    partial_fn(layer, q) -> tensor [n_seqs, H, D+2] float32 (o unnormalised, m, l) of THIS rank's
    tokens; combine_fn(stacked [world, n_seqs, H, D+2]) -> [n_seqs, H, D].  With the CUDA library
    these are PagedKVCache.decode_partial and combine_partials (below); the collective runs on
    the current stream between them, so there is no host synchronisation in a layer.
    """

    def __init__(self, partial_fn: Callable, combine_fn: Callable, group: Optional[dist.ProcessGroup] = None,
                 exchange: Optional["PeerExchange"] = None, out_dtype: torch.dtype = torch.bfloat16,
                 fused_fn: Optional[Callable] = None):
        """exchange: swap rows over peer memory instead of the all-gather.  fused_fn(layer, q, exchange)
        (PagedKVCache.decode_exchange) does partial + exchange in one library call."""
        self.partial_fn, self.combine_fn, self.group = partial_fn, combine_fn, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.exchange, self.out_dtype, self.fused_fn = exchange, out_dtype, fused_fn
        self._gathered = None

    def decode(self, layer: int, q: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.exchange is not None and self.fused_fn is not None:
            return self.fused_fn(layer, q, self.exchange, out)
        part = self.partial_fn(layer, q)
        if self.exchange is not None:                     # peer stores + combine in one kernel, no collective
            return self.exchange.exchange_combine(part, self.out_dtype)
        if self.world == 1:
            return self.combine_fn(part.unsqueeze(0))
        if self._gathered is None or self._gathered.shape[1:] != part.shape or self._gathered.device != part.device:
            self._gathered = torch.empty((self.world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
        # concatenation along dim 0 is the same memory as the [world, ...] stack
        flat = self._gathered.view((self.world * part.shape[0],) + tuple(part.shape[1:]))
        dist.all_gather_into_tensor(flat, part.contiguous(), group=self.group)
        return self.combine_fn(self._gathered)


def combine_partials(stacked: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """CUDA log-sum-exp merge of stacked per-rank partials [R, n_seqs, H, D+2] -> [n_seqs, H, D]."""
    from . import _lib as L
    assert stacked.is_cuda and stacked.dtype == torch.float32 and stacked.is_contiguous()
    r, n_seqs, h, d2 = stacked.shape
    out = torch.empty(n_seqs, h, d2 - 2, dtype=out_dtype, device=stacked.device)
    code = {torch.float32: L.TK_FP32, torch.float16: L.TK_FP16, torch.bfloat16: L.TK_BF16}[out_dtype]
    st = L.lib().tk_combine_partials(stacked.data_ptr(), r, n_seqs * h, d2 - 2, out.data_ptr(), code,
                                     torch.cuda.current_stream().cuda_stream)
    if st != L.TK_OK:
        raise RuntimeError(f"tk_combine_partials failed with status {st}")
    return out


class PeerExchange:
    """Mailboxes in every rank's device memory, mapped into every other rank through CUDA IPC; the
    handles travel over torch.distributed (any backend).  exchange_combine(partial) is one kernel:
    peer stores of this rank's rows, flags, bounded wait for the peers' rows, log-sum-exp combine."""

    live = None        # weak set of the open exchanges of this process (see check_canaries)

    def __init__(self, max_rows: int, row_floats: int, group: Optional[dist.ProcessGroup] = None,
                 rank: Optional[int] = None, world: Optional[int] = None, connect: bool = True):
        import ctypes as C
        import weakref
        if PeerExchange.live is None:
            PeerExchange.live = weakref.WeakSet()
        from . import _lib as L
        self._L, self._C = L, C
        self._lib = L.lib()
        if rank is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
        if world is None:
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank, self.world, self.group = rank, world, group
        self.row_floats = row_floats
        self._h = C.c_void_p()
        st = self._lib.tk_peer_create(rank, world, max_rows, row_floats, torch.cuda.current_device(), C.byref(self._h))
        if st != L.TK_OK:
            raise RuntimeError(f"tk_peer_create failed with status {st}")
        PeerExchange.live.add(self)
        if connect and world > 1:
            self.connect()

    def _check(self, st: int) -> None:
        if st != self._L.TK_OK:
            msg = self._lib.tk_peer_last_error(self._h)
            raise RuntimeError(f"peer exchange: status {st}: {msg.decode() if msg else ''}")

    def connect(self) -> None:
        """Swap CUDA IPC handles with the other ranks of the group and map their mailboxes."""
        C = self._C
        mine = C.create_string_buffer(self._L.TK_PEER_HANDLE_BYTES)
        self._check(self._lib.tk_peer_export(self._h, mine))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(mine.raw), group=self.group)
        self._check(self._lib.tk_peer_connect(self._h, b"".join(handles)))
        dist.barrier(group=self.group)                    # every rank has mapped every mailbox

    def connect_local(self, others: Sequence["PeerExchange"]) -> None:
        """Ranks living in one process: `others` indexed by rank (this rank's own entry is ignored)."""
        C = self._C
        arr = (C.c_void_p * self.world)()
        for r, o in enumerate(others):
            arr[r] = self._lib.tk_peer_mailbox(o._h)
        self._check(self._lib.tk_peer_connect_ptrs(self._h, arr))

    def set_wait_limit_ms(self, ms: int) -> None:
        self._check(self._lib.tk_peer_set_wait_limit_ms(self._h, ms))

    def _code(self, dtype: torch.dtype) -> int:
        L = self._L
        return {torch.float32: L.TK_FP32, torch.float16: L.TK_FP16, torch.bfloat16: L.TK_BF16}[dtype]

    def _rows(self, partial: torch.Tensor):
        assert partial.is_cuda and partial.dtype == torch.float32 and partial.is_contiguous()
        assert partial.shape[-1] == self.row_floats
        return partial.numel() // self.row_floats, self.row_floats - 2

    def exchange_combine(self, partial: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        n_rows, dv = self._rows(partial)
        out = torch.empty(tuple(partial.shape[:-1]) + (dv,), dtype=out_dtype, device=partial.device)
        self._check(self._lib.tk_peer_exchange_combine(self._h, partial.data_ptr(), n_rows, dv, out.data_ptr(),
                                                       self._code(out_dtype), torch.cuda.current_stream().cuda_stream))
        return out

    def send(self, partial: torch.Tensor) -> None:
        n_rows, dv = self._rows(partial)
        self._check(self._lib.tk_peer_send(self._h, partial.data_ptr(), n_rows, dv,
                                           torch.cuda.current_stream().cuda_stream))

    def recv_combine(self, partial: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        n_rows, dv = self._rows(partial)
        out = torch.empty(tuple(partial.shape[:-1]) + (dv,), dtype=out_dtype, device=partial.device)
        self._check(self._lib.tk_peer_recv_combine(self._h, partial.data_ptr(), n_rows, dv, out.data_ptr(),
                                                   self._code(out_dtype), torch.cuda.current_stream().cuda_stream))
        return out

    def check_canaries(self) -> None:
        """Raises when a kernel wrote past the end of this rank's mailbox."""
        if self._h:
            self._check(self._lib.tk_peer_check_canaries(self._h, torch.cuda.current_stream().cuda_stream))

    def status(self) -> None:
        """Raises if a device-side wait of this exchange gave up (a peer never published its rows)."""
        self._check(self._lib.tk_peer_status(self._h, torch.cuda.current_stream().cuda_stream))

    def close(self) -> None:
        if self._h:
            self._lib.tk_peer_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
