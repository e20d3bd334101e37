"""Continuous batching over the paged cache, host logic only (bookkeeping handle, no device):
admission order, chunked prefill, retirement, preemption, and bit-exact page state against the
oracle manager replaying the scheduler's decisions."""
import numpy as np
import pytest

from helpers import rng
from oracle import tk_oracle as O
from titan_engine_b200 import KvError, PagedKVCache
from titan_engine_b200.scheduler import BatchScheduler


def make(num_pages=64, max_seqs=4, mpps=32, max_batch=3, prefill=64):
    c = PagedKVCache(2, 8, 2, 64, num_pages, max_seqs, mpps, dtype="fp16", host_only=True,
                     max_step_tokens=prefill + max_batch)
    return c, BatchScheduler(c, max_batch, prefill), O.Manager(num_pages, max_seqs, mpps, 16)


def replay(sched, cache, o, rows):
    """Apply the scheduler's last iteration to the oracle manager; states must stay identical."""
    ev = sched.last_events()
    # order inside next(): retire, admit, then (while short of pages) preempt
    for s in ev["retired"]:
        assert o.seq_free(s) == O.OK
    for s in ev["admitted"]:
        assert o.seq_alloc() == s
    for s in ev["preempted"]:
        assert o.seq_free(s) == O.OK
    for r in rows:
        assert o.reserve(r.seq, r.n_new) == O.OK
    assert cache.digest() == o.digest()


def test_fifo_admission_chunked_prefill_and_retirement():
    c, s, o = make()
    a = s.submit(150, 3); b = s.submit(10, 2); d = s.submit(20, 5); e = s.submit(5, 1)
    rows = s.next(); replay(s, c, o, rows)
    # batch of 3: a, b, d admitted in order (slots 0,1,2); the 64-token budget goes to a first
    assert [(r.req_id, r.seq, r.n_new, r.samples) for r in rows] == [(a, 0, 64, False)]
    assert s.request(e)["state"] == "queued" and s.request(b)["state"] == "prefilling"
    s.commit([False])
    rows = s.next(); replay(s, c, o, rows)
    assert [(r.req_id, r.n_new) for r in rows] == [(a, 64)]
    s.commit([False])
    rows = s.next(); replay(s, c, o, rows)                  # a's last 22 tokens, then b's 10, d's 20
    assert [(r.req_id, r.n_new, r.samples) for r in rows] == [(a, 22, True), (b, 10, True), (d, 20, True)]
    s.commit([False, False, False])
    assert s.request(a) == {"state": "decoding", "seq": 0, "prefill_pos": 150, "output_tokens": 1}
    rows = s.next(); replay(s, c, o, rows)
    assert [(r.req_id, r.n_new) for r in rows] == [(a, 1), (b, 1), (d, 1)]
    s.commit([False, False, True])                           # b reaches max_output 2, d hits EOS
    assert s.request(b)["state"] == "finished" and s.request(d)["state"] == "finished"
    rows = s.next(); replay(s, c, o, rows)                  # b, d retired (slots 1, 2); e admitted into slot 1
    assert s.last_events() == {"retired": [1, 2], "admitted": [1], "preempted": []}
    assert [(r.req_id, r.seq, r.n_new, r.samples) for r in rows] == [(a, 0, 1, True), (e, 1, 5, True)]
    s.commit([False, False])
    assert s.request(a)["state"] == "finished" and s.request(e)["state"] == "finished"
    rows = s.next(); replay(s, c, o, rows)
    assert rows == [] and c.num_free_pages == 64
    st = s.stats()
    assert st["completed_requests"] == 4 and st["total_tokens_generated"] == 3 + 2 + 2 + 1
    assert st["total_prompt_tokens"] == 185 and st["active_requests"] == 0 and st["preemptions"] == 0


def test_cancel_and_rejects():
    c, s, o = make()
    with pytest.raises(KvError):
        s.submit(32 * 16, 1)                                 # prompt + output exceed a sequence's capacity
    with pytest.raises(KvError):
        BatchScheduler(c, 8, 4096)                           # does not fit the cache's max_step_tokens
    a = s.submit(30, 50); b = s.submit(30, 50)
    assert s.cancel(b) and s.request(b)["state"] == "cancelled"
    rows = s.next(); replay(s, c, o, rows); s.commit([False])
    assert s.cancel(a) and not s.cancel(999)
    rows = s.next(); replay(s, c, o, rows)
    assert rows == [] and s.last_events()["retired"] == [0] and c.num_free_pages == 64
    assert s.stats()["cancelled_requests"] == 2


def test_preemption_when_pages_run_out_and_state_parity():
    """A small pool and long generations: the youngest request is preempted, requeued at the head
    and recomputed; every request still completes, and the page state tracks the oracle."""
    c, s, o = make(num_pages=24, max_seqs=4, mpps=24, max_batch=4, prefill=128)
    g = rng(8)
    want = {}
    for _ in range(7):
        p, m = int(g.integers(20, 120)), int(g.integers(20, 150))
        want[s.submit(p, m)] = m
    for it in range(5000):
        rows = s.next(); replay(s, c, o, rows)
        if not rows and s.stats()["queued_requests"] == 0:
            break
        s.commit([False] * len(rows))
    st = s.stats()
    assert st["completed_requests"] == 7 and st["preemptions"] > 0
    assert st["total_tokens_generated"] == sum(want.values())   # a preempted request resumes, it does not restart its count
    assert c.num_free_pages == 24 and 0 < st["batch_utilization"] <= 1


def churn_lengths(g, n=256):
    """The churn configuration's context lengths: lognormal, median 2048, sigma 1, capped at 32768."""
    return [int(min(32768, max(1, round(float(np.exp(g.normal(np.log(2048.0), 1.0))))))) for _ in range(n)]


def test_churn_configuration_full_size_200_steps_direct_calls():
    """The continuous-batching churn configuration at FULL size on the bookkeeping-only handle: 256
    sequences, lognormal lengths, 200 steps; every step retires 13 sequences (ascending slot), admits 13
    with prompts of 256..4096 tokens (ascending slot), every survivor appends one token.  Page tables,
    lengths and the free list equal the oracle manager's after EVERY step."""
    g = rng(3)
    lens = churn_lengths(g)
    num_pages = sum((n + 15) // 16 for n in lens) + 13 * 257 * 8 + 4096
    mpps = (32768 + 4096 + 256) // 16
    c = PagedKVCache(2, 32, 8, 128, num_pages, 256, mpps, dtype="fp16", host_only=True, max_step_tokens=13 * 4096 + 256)
    o = O.Manager(num_pages, 256, mpps, 16)
    live = []
    for n in lens:
        s = c.seq_alloc(); assert o.seq_alloc() == s
        c.reserve(s, n); assert o.reserve(s, n) == O.OK
        live.append(s)
    assert c.digest() == o.digest()
    for step in range(200):
        gone = sorted(g.choice(live, size=13, replace=False).tolist())
        for s in gone:
            c.seq_free(s); assert o.seq_free(s) == O.OK
            live.remove(s)
        new = []
        for _ in gone:
            s = c.seq_alloc(); assert o.seq_alloc() == s
            new.append(s)
        ids = sorted(live) + sorted(new)
        n_new = [1] * len(live) + [int(g.integers(256, 4097)) for _ in new]
        c.step_begin(ids, n_new)
        for s, n in zip(ids, n_new):
            assert o.reserve(s, n) == O.OK
        assert c.digest() == o.digest(), f"churn step {step}: page/slot state diverged"
        live = ids
        # the prompts admitted by this step are prefill chunks for the attention kernel
        items, ct, n_decode = c.step_prefill_plan()
        assert len(items) > 0 and n_decode > 0 and len(set(items[:, 0].tolist())) == 13
    st = c.stats()
    assert st["steps"] == 200 and st["seq_frees"] == 200 * 13 and c.num_free_pages == o.num_free_pages()


def test_churn_configuration_full_size_200_steps_through_the_scheduler():
    """The same configuration driven through tk_sched_*: 256 requests, every step 13 of the decoding ones
    finish and 13 new prompts are queued; the scheduler's retire / admit / step decisions replayed on the
    oracle manager give bit-identical state after every one of the 200 steps."""
    g = rng(33)
    lens = churn_lengths(g)
    budget = 13 * 4096
    num_pages = sum((n + 15) // 16 for n in lens) + 13 * 257 * 8 + 4096
    mpps = (32768 + 4096 + 4096 + 256) // 16
    c = PagedKVCache(2, 32, 8, 128, num_pages, 256, mpps, dtype="fp16", host_only=True, max_step_tokens=budget + 256)
    s = BatchScheduler(c, 256, budget)
    o = O.Manager(num_pages, 256, mpps, 16)
    for n in lens:
        s.submit(n, 4096)
    for _ in range(400):                                     # set-up: chunked prefill of the 256 contexts
        rows = s.next(); replay(s, c, o, rows)
        s.commit([False] * len(rows))
        if len(rows) == 256 and all(r.n_new == 1 for r in rows):
            break
    else:
        raise AssertionError("set-up did not converge")
    admitted = 0
    for step in range(200):
        rows = s.next(); replay(s, c, o, rows)
        admitted += len(s.last_events()["admitted"])
        decoding = [j for j, r in enumerate(rows) if r.n_new == 1]
        gone = set(g.choice(decoding, size=13, replace=False).tolist())
        s.commit([j in gone for j in range(len(rows))])
        for _ in range(13):
            s.submit(int(g.integers(256, 4097)), 4096)
    st = s.stats()
    assert admitted == 199 * 13 and st["preemptions"] == 0 and st["completed_requests"] >= 199 * 13
