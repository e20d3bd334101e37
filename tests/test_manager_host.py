"""Host logic of the page manager through the C ABI, with no device (device = -2:
bookkeeping only).  Page tables, slot indices and the free list must be bit-exact
against the oracle's manager under the same call sequence."""
import re
import os

import numpy as np
import pytest

from helpers import rng
from oracle import tk_oracle as O
from titan_engine_b200 import KvError, PagedKVCache, _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def host_cache(num_pages=64, max_seqs=8, mpps=64, dtype="fp16", **kw):
    return PagedKVCache(2, 8, 2, 64, num_pages, max_seqs, mpps, dtype=dtype, host_only=True,
                        max_step_tokens=kw.pop("max_step_tokens", 4096), **kw)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "titan_kv.h")).read()
    declared = set(re.findall(r"\b(tk_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    lib = L.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in titan_kv.h but not exported"
    assert declared == set(L.SIGNATURES), declared ^ set(L.SIGNATURES)


def test_compute_fails_loudly_without_device():
    c = host_cache()
    s = c.seq_alloc()
    c.step_begin([s], [3])
    with pytest.raises(KvError) as e:
        c._check(c._lib.tk_kv_append(c._h, 0, None, None, None, None))
    assert e.value.status == L.TK_CUDA_ERROR
    with pytest.raises(KvError):
        c._check(c._lib.tk_kv_decode(c._h, 0, None, None, None))


def test_fresh_pool_hands_out_sequential_pages_and_slots():
    c = host_cache()
    s = c.seq_alloc()
    assert s == 0
    c.reserve(s, 512)
    np.testing.assert_array_equal(c.page_table(s), np.arange(32))
    for pos in (0, 15, 16, 511):
        assert c.slot(s, pos) == pos
    assert c.slot(s, 512) == -1
    assert c.num_free_pages == 32
    for _ in range(64):
        c.reserve(s, 1)
    assert c.seq_len(s) == 576 and len(c.page_table(s)) == 36


def test_lifo_reuse_and_lowest_free_slot():
    c = host_cache()
    a, b = c.seq_alloc(), c.seq_alloc()
    c.reserve(a, 40)            # pages 0,1,2
    c.reserve(b, 20)            # pages 3,4
    c.seq_free(a)               # pushes 0,1,2 -> 2 is on top
    assert c.seq_alloc() == 0   # lowest free slot index, like BatchScheduler::allocate_slot
    c.reserve(0, 50)            # needs 4 pages: 2,1,0 then 5
    np.testing.assert_array_equal(c.page_table(0), [2, 1, 0, 5])
    assert c.seq_len(1) == 20 and c.seq_len(5) == -1


def test_out_of_pages_changes_nothing():
    c = host_cache(num_pages=4)
    s = c.seq_alloc()
    c.reserve(s, 40)
    d = c.digest()
    with pytest.raises(KvError) as e:
        c.reserve(s, 100)
    assert e.value.status == L.TK_OUT_OF_PAGES
    assert c.digest() == d and c.seq_len(s) == 40
    t = c.seq_alloc()
    with pytest.raises(KvError) as e:           # step_begin is all-or-nothing across sequences
        c.step_begin([s, t], [8, 17])
    assert e.value.status == L.TK_OUT_OF_PAGES
    assert c.seq_len(s) == 40 and c.seq_len(t) == 0 and c.num_free_pages == 1
    c.step_begin([s, t], [8, 16])
    assert c.num_free_pages == 0


def test_invalid_arguments():
    c = host_cache()
    with pytest.raises(KvError):
        c.reserve(3, 1)                         # not live
    s = c.seq_alloc()
    with pytest.raises(KvError):
        c.reserve(s, 64 * 16 + 1)               # exceeds max_pages_per_seq
    with pytest.raises(KvError):
        c.step_begin([s, s], [1, 1])            # duplicate sequence
    with pytest.raises(KvError):
        c.seq_free(5)
    for _ in range(7):
        c.seq_alloc()
    with pytest.raises(KvError) as e:
        c.seq_alloc()
    assert e.value.status == L.TK_OUT_OF_SEQS
    with pytest.raises(KvError):
        PagedKVCache(2, 8, 3, 64, 8, 2, 4, host_only=True)   # 8 heads / 3 kv heads


def test_adopt_and_truncate():
    c = host_cache(num_pages=32)
    s = c.seq_alloc()
    c.adopt(s, [7, 3, 30], 40)
    np.testing.assert_array_equal(c.page_table(s), [7, 3, 30])
    assert c.slot(s, 17) == 3 * 16 + 1 and c.num_free_pages == 29
    t = c.seq_alloc()
    with pytest.raises(KvError):
        c.adopt(t, [3], 5)                      # page 3 is taken
    c.reserve(t, 16)                            # next free after removing 7,3,30: 0
    np.testing.assert_array_equal(c.page_table(t), [0])
    c.truncate(s, 16)
    np.testing.assert_array_equal(c.page_table(s), [7])
    c.reserve(t, 32)                            # freed 3 then 30 -> 30 on top, then 3
    np.testing.assert_array_equal(c.page_table(t), [0, 30, 3])


def test_step_plan_shapes():
    c = host_cache(num_pages=256, mpps=64, chunk_tokens=128)
    a, b = c.seq_alloc(), c.seq_alloc()
    c.step_begin([a, b], [300, 5])
    assert c.step_num_tokens == 305 and c.step_chunk_tokens == 128
    assert c.step_num_work_items == (3 + 1) * 2      # ceil(300/128)=3 chunks + 1 chunk, x 2 kv heads
    c.step_begin([b, a], None)                       # decode only
    assert c.step_num_tokens == 0 and c.step_num_work_items == 8
    f = host_cache(num_pages=256, mpps=64, chunk_tokens=128, dtype="fp8")
    s = f.seq_alloc()
    f.step_begin([s], [300])                         # 18 sealed pages (288 tokens) + 12 open
    assert f.step_num_work_items == (3 + 1) * 2 and f.stats()["pages_sealed"] == 18
    f.step_begin([s], [4])                           # 304 tokens: 19 sealed, nothing open
    assert f.step_num_work_items == 3 * 2 and f.stats()["pages_sealed"] == 19


@pytest.mark.parametrize("n_seqs,tokens,want_chunk,want_items", [
    (1, 65536, 2048, 256),      # under a wave of items: the largest chunk
    (1, 131072, 1536, 688),     # 512 items would be a little more than one wave of 444: go to 1.5 waves
    (8, 16384, 1536, 704),
    (1, 16384, 1024, 128),      # fewer than 128 items at 2048: shrink until there are 128
    (1, 4096, 256, 128),
    (64, 4600, 2048, 1536),     # a batch: the largest chunk
])
def test_auto_chunk_rule(n_seqs, tokens, want_chunk, want_items):
    """The split-KV chunk the planner picks on its own (8 kv heads, 148 SMs assumed without a device)."""
    pages = (tokens + 15) // 16
    c = PagedKVCache(1, 32, 8, 128, pages * n_seqs + 8, n_seqs, pages + 1, dtype="bf16", host_only=True,
                     max_step_tokens=64)
    seqs = []
    for b in range(n_seqs):
        s = c.seq_alloc()
        c.adopt(s, np.arange(b * pages, (b + 1) * pages, dtype=np.int32), tokens)
        seqs.append(s)
    c.step_begin(seqs, None)
    assert (c.step_chunk_tokens, c.step_num_work_items) == (want_chunk, want_items)


@pytest.mark.parametrize("seed", [3, 4])
def test_churn_matches_oracle_manager_bit_exact(seed):
    """Retire ~5% per step in ascending slot order, admit replacements in ascending slot order,
    every survivor appends one token: page tables, slots and free list equal the oracle's."""
    num_pages, max_seqs, mpps, ps = 3000, 64, 160, 16
    c = host_cache(num_pages, max_seqs, mpps, max_step_tokens=1 << 16)
    o = O.Manager(num_pages, max_seqs, mpps, ps)
    g = rng(seed)
    live = []
    for _ in range(max_seqs):
        s, so = c.seq_alloc(), o.seq_alloc()
        assert s == so
        n = int(min(2048, max(1, round(float(np.exp(g.normal(np.log(300.0), 1.0)))))))
        c.step_begin([s], [n]); assert o.reserve(so, n) == O.OK
        live.append(s)
    assert c.digest() == o.digest()
    for step in range(60):
        retire = sorted(g.choice(live, size=3, replace=False).tolist())
        for s in retire:
            c.seq_free(s); assert o.seq_free(s) == O.OK
            live.remove(s)
        admitted = []
        for _ in retire:
            s, so = c.seq_alloc(), o.seq_alloc()
            assert s == so
            admitted.append(s)
        prefill = [int(g.integers(16, 257)) for _ in admitted]
        ids = sorted(live) + admitted
        n_new = [1] * len(live) + prefill
        need = sum(((c.seq_len(s) + n + ps - 1) // ps) - len(c.page_table(s)) for s, n in zip(ids, n_new))
        if need > c.num_free_pages:
            with pytest.raises(KvError):
                c.step_begin(ids, n_new)
            ids, n_new = sorted(live), [1] * len(live)
            for s in admitted:
                c.seq_free(s); o.seq_free(s)
            admitted = []
        c.step_begin(ids, n_new)
        for s, n in zip(ids, n_new):
            assert o.reserve(s, n) == O.OK
        live = sorted(live) + admitted
        assert c.digest() == o.digest(), f"step {step}"
        s = live[int(g.integers(len(live)))]
        np.testing.assert_array_equal(c.page_table(s), o.page_table(s))
        pos = c.seq_len(s) - 1
        assert c.slot(s, pos) == o.slot(s, pos)
    assert c.stats()["page_frees"] > 0


def test_cold_tier_state_matches_oracle_manager():
    """Window-driven eviction: page ids, cold ids and both free lists equal the oracle's."""
    num_pages, cold_pages, max_seqs, mpps, window = 64, 200, 4, 128, 64
    c = PagedKVCache(2, 8, 2, 64, num_pages, max_seqs, mpps, dtype="fp16", host_only=True,
                     max_step_tokens=4096, hot_window=window, cold_pages=cold_pages)
    o = O.Manager(num_pages, max_seqs, mpps, 16)
    assert o.enable_cold(window, cold_pages) == O.OK
    a, b = c.seq_alloc(), c.seq_alloc()
    assert (o.seq_alloc(), o.seq_alloc()) == (a, b)

    def step(ids, n_new):
        old = [c.seq_len(s) for s in ids]
        c.step_begin(ids, n_new)
        for s, n in zip(ids, n_new):
            assert o.reserve(s, n) == O.OK
        for s, ol in zip(ids, old):
            assert o.evict_cold(s, ol) >= 0
        assert c.digest() == o.digest()

    step([a, b], [300, 50])                      # pages written by this very step stay hot ...
    assert c.stats()["pages_cold"] == 0
    step([a, b], [0, 0])                         # ... a: 300-64=236 -> 14 pages cold; b: none
    assert c.stats()["pages_cold"] == 14 == o.num_cold_used()
    assert c.num_free_pages == num_pages - (19 - 14) - 4
    assert c.slot(a, 0) == -1 and c.slot(a, 299) >= 0          # cold tokens have no device slot
    for _ in range(40):
        step([a, b], [1, 1])
    assert c.stats()["pages_cold"] == (340 - 64) // 16 + (90 - 64) // 16
    c.seq_free(a); assert o.seq_free(a) == O.OK
    assert c.digest() == o.digest() and c.stats()["pages_cold"] == 1
    d = c.seq_alloc(); assert o.seq_alloc() == d
    step([d, b], [700, 1])                       # 44 pages, 39 of them cold from the next step on
    step([d, b], [1, 1])
    assert c.stats()["pages_cold"] == (701 - 64) // 16 + (92 - 64) // 16
    assert c.seq_len(d) == 701 and c.stats()["evictions"] == o.num_cold_used() + 17
    # a rank holding an early part of a long sequence: the tokens after it push its pages out
    c.set_tail(b, 1000); assert o.set_tail(b, 1000) == O.OK
    step([d, b], [0, 0])
    assert c.stats()["pages_cold"] == (701 - 64) // 16 + 92 // 16
    with pytest.raises(KvError):
        PagedKVCache(2, 8, 2, 64, 8, 2, 8, dtype="fp8", host_only=True, hot_window=64, cold_pages=8)


def test_truncate_into_a_cold_page_is_refused():
    """A length that ends inside a page held in the host pool would make the next append write a page
    that has no device row: refused, state untouched; a page-aligned length is fine and the next
    token gets a device slot."""
    c = PagedKVCache(2, 8, 2, 64, 64, 2, 64, dtype="fp16", host_only=True, max_step_tokens=4096,
                     hot_window=64, cold_pages=64)
    o = O.Manager(64, 2, 64, 16); assert o.enable_cold(64, 64) == O.OK
    a = c.seq_alloc(); assert o.seq_alloc() == a
    c.step_begin([a], [300]); assert o.reserve(a, 300) == O.OK and o.evict_cold(a, 0) == 0
    c.step_begin([a], [0]); assert o.evict_cold(a, 300) == 14            # pages 0..13 go cold
    assert c.digest() == o.digest() and c.slot(a, 37) == -1
    d = c.digest()
    with pytest.raises(KvError) as e:
        c.truncate(a, 37)                                                 # inside cold page 2
    assert e.value.status == L.TK_UNSUPPORTED and c.digest() == d and c.seq_len(a) == 300
    assert o.truncate(a, 37) == 6 and o.digest() == d                     # the oracle refuses it too
    c.truncate(a, 32); assert o.truncate(a, 32) == O.OK                   # page-aligned: pages 0, 1 stay cold
    assert c.digest() == o.digest()
    c.step_begin([a], [1]); assert o.reserve(a, 1) == O.OK and o.evict_cold(a, 32) == 0
    assert c.digest() == o.digest() and c.slot(a, 32) >= 0
    # inside a hot page: allowed
    c.step_begin([a], [40]); assert o.reserve(a, 40) == O.OK and o.evict_cold(a, 33) >= 0
    c.truncate(a, 50); assert o.truncate(a, 50) == O.OK
    c.step_begin([a], [1]); assert o.reserve(a, 1) == O.OK and o.evict_cold(a, 50) >= 0
    assert c.digest() == o.digest() and c.slot(a, 50) >= 0


def test_full_cold_pool_is_counted_not_hidden():
    """When the host pool cannot take a sequence's old pages they stay in HBM, the step succeeds and
    the refusal shows in the stats."""
    c = PagedKVCache(2, 8, 2, 64, 64, 2, 64, dtype="fp16", host_only=True, max_step_tokens=4096,
                     hot_window=32, cold_pages=4)
    a = c.seq_alloc()
    c.step_begin([a], [200])
    c.step_begin([a], [0])                                                # 10 pages should go cold, 4 fit: none moves
    st = c.stats()
    assert st["evictions_refused"] == 1 and st["pages_cold"] == 0
    assert "cold" in c._lib.tk_kv_last_error(c._h).decode()


def test_fork_shares_full_pages_and_counts_references():
    c = host_cache(num_pages=16, max_seqs=4, mpps=8)
    o = O.Manager(16, 4, 8, 16)
    a = c.seq_alloc(); assert o.seq_alloc() == a
    c.reserve(a, 40); assert o.reserve(a, 40) == O.OK           # pages 0,1 full-ish: 0,1 full, 2 partial
    b = c.fork(a)
    ob, src, dst = o.fork(a)
    assert (b, ob, src, dst) == (1, 1, 2, 3)
    np.testing.assert_array_equal(c.page_table(b), [0, 1, 3])   # shares 0 and 1, own copy of the partial page
    assert c.seq_len(b) == 40 and c.num_free_pages == 12 and c.digest() == o.digest()
    c.reserve(b, 30); assert o.reserve(b, 30) == O.OK           # both keep growing independently
    c.reserve(a, 10); assert o.reserve(a, 10) == O.OK
    assert c.digest() == o.digest()
    c.seq_free(a); assert o.seq_free(a) == O.OK                 # shared pages stay with b
    assert c.num_free_pages == o.num_free_pages() == 16 - 5 and c.digest() == o.digest()
    np.testing.assert_array_equal(c.page_table(b), [0, 1, 3, 4, 5])
    d = c.fork(b); od, src, dst = o.fork(b)
    assert d == od == 0 and dst >= 0 and c.digest() == o.digest()
    with pytest.raises(KvError) as e:
        c.truncate(d, 20)                                       # would reopen page 1, which b also holds
    assert e.value.status == L.TK_UNSUPPORTED
    c.truncate(d, 32); assert o.truncate(d, 32) == O.OK         # page-aligned is fine
    c.seq_free(b); assert o.seq_free(b) == O.OK
    c.seq_free(d); assert o.seq_free(d) == O.OK
    assert c.num_free_pages == 16 and c.digest() == o.digest()
    # page-aligned parent: nothing to copy, no page taken
    a = c.seq_alloc(); o.seq_alloc(); c.reserve(a, 32); o.reserve(a, 32)
    free0 = c.num_free_pages
    b = c.fork(a); assert o.fork(a) == (b, -1, -1) and c.num_free_pages == free0
    # no slot / no page left: nothing changes
    t = host_cache(num_pages=1, max_seqs=2, mpps=4)
    s = t.seq_alloc(); t.reserve(s, 5)
    dg = t.digest()
    with pytest.raises(KvError) as e:
        t.fork(s)
    assert e.value.status == L.TK_OUT_OF_PAGES and t.digest() == dg


def test_prefill_work_list_order_keeps_a_sequences_pages_together():
    """Launch order of the prefill items: the tiles and chunks of one (sequence, kv head) read the same pages, so
    they go out together - in sets of about 48 MB of K/V (512 B per token and kv head), the biggest (sequence, kv
    head) groups first, and big items first inside a set."""
    H, Hkv, G = 32, 8, 4
    lens0 = [150_000, 60_000, 90_000, 20_000, 0]             # 77, 31, 46, 10 MB of K/V per kv head (+ the new tokens)
    n_new = [512, 512, 512, 512, 512]
    mpps = 9500
    c = PagedKVCache(1, H, Hkv, 128, 21_000, len(lens0), mpps, dtype="bf16", host_only=True, max_step_tokens=4096)
    seqs, at = [], 0
    for n in lens0:
        s = c.seq_alloc()
        pages = (n + 15) // 16
        c.adopt(s, np.arange(at, at + pages, dtype=np.int32), n)
        at += pages
        seqs.append(s)
    c.step_begin(seqs, n_new)
    items, ct, _ = c.step_prefill_plan()
    items = items.tolist()
    tpt = 64 // G
    def weight(it):
        b, chunk, kvh, tile = it
        nq, ln = n_new[b], lens0[b] + n_new[b]
        tok_cnt = min(nq - tile * tpt, tpt)
        p_last = ln - nq + tile * tpt + tok_cnt - 1
        return min(ct[b], p_last + 1 - chunk * ct[b]) * tok_cnt * G
    # replay the rule: groups by total weight (ties: sequence, kv head), cut into sets by bytes
    groups = {}
    for it in items:
        groups.setdefault((it[0], it[2]), 0)
        groups[(it[0], it[2])] += weight(it)
    order = sorted(groups, key=lambda k: (-groups[k], k))
    set_of, cur, bytes_in = {}, 0, 0
    for k in order:
        kv = (lens0[k[0]] + n_new[k[0]]) * 512
        if bytes_in > 0 and bytes_in + kv > 48 << 20:
            cur, bytes_in = cur + 1, 0
        set_of[k] = cur
        bytes_in += kv
    sets = [set_of[(it[0], it[2])] for it in items]
    assert sets == sorted(sets) and sets[-1] >= 3            # the long sequences are alone in their sets
    for a, b in zip(items, items[1:]):                       # big first inside a set
        if set_of[(a[0], a[2])] == set_of[(b[0], b[2])]:
            assert weight(a) >= weight(b)
    first = [it for it, st in zip(items, sets) if st == 0]
    assert {(it[0], it[2]) for it in first} == {(0, 0)}      # the heaviest group: sequence 0, kv head 0, by itself


@pytest.mark.parametrize("shape", [(32, 8), (64, 8), (16, 16), (16, 1), (8, 4)])
def test_prefill_work_list_covers_every_row_once(shape):
    """Index arithmetic of the prefill attention kernel, replayed on the host: the tiles of 64 (token, head)
    rows and their split-KV chunks cover every (query token, head) of the long sequences and every context
    position that token may see exactly once; sequences with one 16-row tile stay with the decode kernel."""
    H, Hkv = shape
    G = H // Hkv
    g = rng(7)
    lens0 = [0, 5000, 33, 0, 40000, 700, 17]
    n_new = [300, 1, 4096, 70, 37, 16 // G, max(2, 128 // G + 1)]
    mpps = 3000
    c = PagedKVCache(1, H, Hkv, 128, 9000, len(lens0), mpps, dtype="bf16", host_only=True, max_step_tokens=8192)
    seqs = []
    at = 0
    for n in lens0:
        s = c.seq_alloc()
        pages = (n + 15) // 16
        c.adopt(s, np.arange(at, at + pages, dtype=np.int32), n)
        at += pages
        seqs.append(s)
    c.step_begin(seqs, n_new)
    items, ct, n_decode = c.step_prefill_plan()
    assert len(items) > 0
    tpt = 64 // G
    small = [i for i, n in enumerate(n_new) if n * G <= 16]
    assert n_decode == sum(-(-(l + n) // c.step_chunk_tokens) * Hkv for i, (l, n) in enumerate(zip(lens0, n_new)) if i in small)
    seen = {}
    for b, chunk, kvh, tile in items.tolist():
        assert b not in small and 0 <= kvh < Hkv
        nq, ln = n_new[b], lens0[b] + n_new[b]
        assert ct[b] % 16 == 0 and ct[b] <= 32768
        tok_first = tile * tpt
        tok_cnt = min(nq - tok_first, tpt)
        assert tok_cnt >= 1
        p_last = ln - nq + tok_first + tok_cnt - 1
        t0, t1 = chunk * ct[b], min(chunk * ct[b] + ct[b], p_last + 1)
        assert t1 > t0 and (t1 - t0 + 15) // 16 <= 2048
        key = (b, kvh, tile)
        seen.setdefault(key, []).append((t0, t1))
    for b, nq in enumerate(n_new):
        if b in small:
            continue
        tiles = -(-nq // tpt)
        for kvh in range(Hkv):
            for tile in range(tiles):
                spans = sorted(seen.pop((b, kvh, tile)))
                p_last = lens0[b] + min(nq, (tile + 1) * tpt) - 1
                assert spans[0][0] == 0 and spans[-1][1] == p_last + 1
                assert all(a[1] == bb[0] for a, bb in zip(spans, spans[1:]))
                assert len(spans) == p_last // ct[b] + 1          # what the kernel takes as the group's item count
    assert not seen
    # a step the decode kernel's token groups can hold does not build the list
    c.step_begin(seqs, [1, 1, 128 // G, 1, 1, 1, 1])
    assert len(c.step_prefill_plan()[0]) == 0


def test_state_image_replays_a_churn_run_from_the_middle():
    """Save the allocator + page-table state in the middle of a churn run, load it into a fresh handle and
    continue both with the same calls: identical digests at every step, and a damaged image is refused."""
    def make():
        return host_cache(num_pages=600, max_seqs=16, mpps=64, max_step_tokens=4096)
    a = make()
    g = rng(12)
    live = []
    def churn(c, g, live, steps):
        for _ in range(steps):
            if live and g.random() < 0.4:
                s = live.pop(int(g.integers(len(live)))); c.seq_free(s)
            if len(live) < 12:
                live.append(c.seq_alloc())
            c.step_begin(sorted(live), [int(g.integers(1, 40)) for _ in live])
            if live and g.random() < 0.3:
                s = live[int(g.integers(len(live)))]
                c.truncate(s, (c.seq_len(s) // 2 // 16) * 16)
    churn(a, g, live, 40)
    image = a.state_save()
    b = make()
    b.state_load(image)
    assert b.digest() == a.digest() and b.num_free_pages == a.num_free_pages
    for s in live:
        np.testing.assert_array_equal(b.page_table(s), a.page_table(s))
    state = g.bit_generator.state
    live_b = list(live)
    churn(a, g, live, 30)
    g2 = rng(0); g2.bit_generator.state = state
    churn(b, g2, live_b, 30)
    assert a.digest() == b.digest() and live == live_b
    bad = image.copy(); bad[0] ^= 1
    with pytest.raises(KvError):
        make().state_load(bad)
    with pytest.raises(KvError):
        make().state_load(image[:-3])
    with pytest.raises(KvError):
        host_cache(num_pages=601, max_seqs=16, mpps=64).state_load(image)
