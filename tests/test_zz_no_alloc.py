"""The allocation-free decode entry point, tk_paged_decode_static.

It exists for callers that may not allocate device memory at the point where they need
attention (no handle, no workspace: its split-KV scratch is a fixed array inside the
library).  This test drives it through the C ABI on the pool and page tables of an ordinary
cache and checks it, twice in a row, against the CPU oracle and against the handle-based entry
point tk_kv_decode: the second call reuses the scratch the first one left behind.  It also
checks that oversized requests are refused and that a call takes no device memory: the
driver's count of free bytes (which sees every allocation of the process, the library's own
included) is the same before and after.

Collected last (file name), so a run that stops at the first failure has already run
every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import RTOL, ATOL, assert_close, normal16, rng, to_torch16
from oracle import tk_oracle as O

pytestmark = pytest.mark.gpu


def test_static_decode_matches_handle_decode_twice_in_a_row():
    from titan_engine_b200 import PagedKVCache, _lib as L
    lib = L.lib()
    H, Hkv, D = 32, 8, 128
    lens = [700, 16, 1, 333, 257]
    n_pages = sum((n + 15) // 16 for n in lens) + 4
    mpps = max((n + 15) // 16 for n in lens) + 1
    cache = PagedKVCache(1, H, Hkv, D, n_pages, len(lens), mpps, dtype="bf16", max_step_tokens=sum(lens))
    dev = cache.device
    seqs = [cache.seq_alloc() for _ in lens]
    g = rng(91)
    cache.step_begin(seqs, lens)
    k = normal16(g, (sum(lens), Hkv, D), O.BF16)
    v = normal16(g, (sum(lens), Hkv, D), O.BF16)
    cache.append(0, to_torch16(k, O.BF16, dev), to_torch16(v, O.BF16, dev))

    table = np.full((len(lens), mpps), -1, dtype=np.int32)
    for i, s in enumerate(seqs):
        pt = cache.page_table(s)
        table[i, :len(pt)] = pt
    # the same rows in the CPU oracle's pool
    ref_pool = O.Pool(O.BF16, n_pages, H, Hkv, D, len(lens), mpps, 16)
    tok_seq = np.concatenate([np.full(n, i, np.int32) for i, n in enumerate(lens)])
    tok_pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    ref_pool.append(table, tok_seq, tok_pos, k, v)
    d_table = torch.from_numpy(table).to(dev)
    pool = cache.layer_views(0)[0]
    host_lens = np.asarray(lens, dtype=np.int32)
    stream = torch.cuda.current_stream().cuda_stream

    for call in range(3):                                  # call 0 also warms up (address look-up, module load)
        q16 = normal16(g, (len(lens), H, D), O.BF16)
        q = to_torch16(q16, O.BF16, dev)
        want = ref_pool.decode(table, np.arange(len(lens)), lens, q16)
        handle = cache.decode(0, q).float().cpu().numpy()
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info(dev)[0]
        st = lib.tk_paged_decode_static(pool.data_ptr(), L.TK_BF16, n_pages, d_table.data_ptr(), mpps,
                                        host_lens.ctypes.data_as(C.POINTER(C.c_int32)), len(lens), H, Hkv, D,
                                        q.data_ptr(), out.data_ptr(), stream)
        assert st == L.TK_OK, f"call {call}: status {st}"
        torch.cuda.synchronize()
        if call > 0:
            assert torch.cuda.mem_get_info(dev)[0] == before, "the call changed the device's free memory"
        got = out.float().cpu().numpy()
        assert np.abs(got).max() > 0
        assert_close(got, want, f"static entry point vs the CPU oracle, call {call}", rtol=RTOL, atol=ATOL,
                     out_mantissa_bits=7)
        assert_close(got, handle, f"static entry point vs tk_kv_decode, call {call}", rtol=RTOL, atol=ATOL,
                     out_mantissa_bits=7)

    # beyond the fixed scratch: refused with a status, nothing launched
    big = np.full(8, 16 * mpps, dtype=np.int32)
    too_many = lib.tk_paged_decode_static(pool.data_ptr(), L.TK_BF16, n_pages, d_table.data_ptr(), 1 << 20,
                                          np.full(300, 16, np.int32).ctypes.data_as(C.POINTER(C.c_int32)), 300,
                                          H, Hkv, D, q.data_ptr(), out.data_ptr(), stream)
    assert too_many == L.TK_INVALID_ARG
    huge = np.full(200, 200000, dtype=np.int32)            # 200 x 782 chunks of partial rows > 4 MiB
    st = lib.tk_paged_decode_static(pool.data_ptr(), L.TK_BF16, n_pages, d_table.data_ptr(), 1 << 20,
                                    huge.ctypes.data_as(C.POINTER(C.c_int32)), 200, H, Hkv, D,
                                    q.data_ptr(), out.data_ptr(), stream)
    assert st == L.TK_INVALID_ARG
    del big
    torch.cuda.synchronize()
