"""The five benchmark configurations at their FULL sizes (one layer each), checked through properties
that do not need the oracle to process the whole workload, plus the oracle itself on a seeded
sample of sequences:
  * sampled sequences: attention within 2e-3 rel / 1e-2 abs of the CPU oracle
  * V = 1 everywhere  -> every output element is 1 (softmax weights sum to one)
  * linearity in V    -> out(V1 + V2) = out(V1) + out(V2)
  * split-KV chunk size does not change the result
  * page/slot state digest equals the oracle manager's at full size
"""
import numpy as np
import pytest
import torch

from helpers import RTOL, ATOL, assert_close, from_torch16, rng
from oracle import tk_oracle as O

pytestmark = pytest.mark.gpu


def build(H, Hkv, D, dtype, lens, seed, io=None, extra_pages=64, **kw):
    """Cache with a seeded shuffled pool already holding N(0,1) data for sequences of `lens`."""
    from titan_engine_b200 import PagedKVCache
    ps = 16
    g = rng(seed)
    pages = [(int(n) + ps - 1) // ps for n in lens]
    n_pages = sum(pages) + extra_pages
    mpps = max(pages) + 2
    c = PagedKVCache(1, H, Hkv, D, n_pages, len(lens), mpps, dtype=dtype, io_dtype=io,
                     max_step_tokens=kw.pop("max_step_tokens", len(lens)), **kw)
    mgr = O.Manager(n_pages, len(lens), mpps, ps)
    perm = g.permutation(n_pages).astype(np.int32)
    seqs, at = [], 0
    for n, p in zip(lens, pages):
        s = c.seq_alloc(); assert s == mgr.seq_alloc()
        c.adopt(s, perm[at:at + p], int(n)); assert mgr.adopt(s, perm[at:at + p], int(n)) == O.OK
        at += p
        seqs.append(s)
    assert c.digest() == mgr.digest()
    gen = torch.Generator(device=c.device); gen.manual_seed(seed)
    pool, scales, open_pages = c.layer_views(0)
    if dtype == "fp8":
        # codes of N(0,1) values under a scale of about amax/448 with amax ~ 4, as sealing would leave
        scales.uniform_(0.008, 0.010, generator=gen)
        for p0 in range(0, pool.shape[0], 4096):                   # by slabs: keeps the temporaries small
            sl = slice(p0, min(p0 + 4096, pool.shape[0]))
            x = torch.randn(pool[sl].shape, device=c.device, generator=gen)
            x = (x / scales[sl][..., None, None]).clamp_(-448.0, 448.0)
            pool[sl] = x.to(torch.float8_e4m3fn).view(torch.uint8)
        open_pages.normal_(generator=gen)
    else:
        pool.normal_(generator=gen)
    return c, mgr, seqs, gen


def oracle_sample(c, seqs, lens, sample, q, dtype_name):
    """Oracle attention for the sampled sequences only: their pages are gathered to the host."""
    pool, scales, open_pages = c.layer_views(0)
    cfg = c.cfg
    outs = {}
    for b in sample:
        pt = torch.from_numpy(c.page_table(seqs[b]).astype(np.int64)).to(c.device)
        n_pg = len(pt)
        if dtype_name == "fp8":
            carrier = O.BF16 if c.io_torch_dtype == torch.bfloat16 else O.FP16
            o = O.Pool(O.FP8, n_pg, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, 1, n_pg, 16, carrier)
            o.pool[:] = pool[pt].cpu().numpy()
            o.scales[:] = scales[pt].cpu().numpy()
            o.open_pages[0] = from_torch16(open_pages[seqs[b]])
            dt = carrier
        else:
            dt = O.BF16 if dtype_name == "bf16" else O.FP16
            o = O.Pool(dt, n_pg, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, 1, n_pg, 16)
            o.pool[:] = from_torch16(pool[pt])
        table = np.arange(n_pg, dtype=np.int32)[None]
        outs[b] = o.decode(table, [0], [int(lens[b])], from_torch16(q[b:b + 1]))[0]
    return outs


def properties(c, seqs, lens, gen, dtype_name, sample, fp8=False):
    cfg = c.cfg
    H, D = cfg.num_heads, cfg.head_dim
    bits = 7 if c.io_torch_dtype == torch.bfloat16 else 10
    q = torch.randn(len(seqs), H, D, device=c.device, generator=gen).to(c.io_torch_dtype)
    c.step_begin(seqs, None)
    out = c.decode(0, q)
    c.device_status()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all() and np.abs(got).max() > 0
    for b, want in oracle_sample(c, seqs, lens, sample, q, dtype_name).items():
        assert_close(got[b], want, f"sequence {b} (len {lens[b]}) vs oracle", out_mantissa_bits=bits)
    if fp8:
        return got
    pool = c.layer_views(0)[0]
    # softmax weights sum to one: V := 1
    v_saved = pool[:, :, 1].clone()
    pool[:, :, 1] = 1.0
    ones = c.decode(0, q).float()
    assert torch.allclose(ones, torch.ones_like(ones), rtol=0, atol=6e-3), float((ones - 1).abs().max())
    # linearity in V: out(V) + out(1) = out(V + 1)
    pool[:, :, 1] = v_saved + 1.0
    lin = c.decode(0, q).float().cpu().numpy()
    assert_close(lin, got + 1.0, "linearity in V", rtol=4e-3, atol=2e-2, out_mantissa_bits=bits)
    pool[:, :, 1] = v_saved
    return got


def test_c2_8b_shape_batched_decode_full_size():
    """64 sequences, context U[1024,8192], bf16, shuffled pool: one full layer (1.2 GB)."""
    lens = rng(2).integers(1024, 8193, size=64)
    c, mgr, seqs, gen = build(32, 8, 128, "bf16", lens, seed=2)
    base = properties(c, seqs, lens, gen, "bf16", sample=[0, 17, int(np.argmax(lens)), int(np.argmin(lens))])
    c.close()
    # a different split-KV chunking gives the same answer
    c2, _, seqs2, gen2 = build(32, 8, 128, "bf16", lens, seed=2, chunk_tokens=256)
    q = torch.randn(64, 32, 128, device=c2.device, generator=gen2).to(torch.bfloat16)
    c2.step_begin(seqs2, None)
    other = c2.decode(0, q).float().cpu().numpy()
    assert_close(other, base, "chunk 256 vs default chunking", out_mantissa_bits=7)


def test_c3_churn_full_size_state_and_attention():
    """256 sequences, lognormal lengths (median 2048, sigma 1, cap 32768), fp16; 20 churn steps at
    full size on the page manager (digest vs oracle every step), attention on the final state."""
    g = rng(3)
    draw = lambda: int(min(32768, max(1, round(float(np.exp(g.normal(np.log(2048.0), 1.0)))))))
    lens = np.array([draw() for _ in range(256)])
    c, mgr, seqs, gen = build(32, 8, 128, "fp16", lens, seed=3, extra_pages=16384, max_step_tokens=1 << 16)
    H, Hkv, D = 32, 8, 128
    live = list(seqs)
    kbuf = torch.randn(13 * 4096 + 256, Hkv, D, device=c.device, generator=gen).to(torch.float16)
    for step in range(20):
        for s in sorted(g.choice(live, size=13, replace=False).tolist()):
            c.seq_free(s); assert mgr.seq_free(s) == O.OK
            live.remove(s)
        new = []
        for _ in range(13):
            s = c.seq_alloc(); assert s == mgr.seq_alloc()
            new.append(s)
        ids = sorted(live) + new
        n_new = [1] * len(live) + [int(g.integers(256, 4097)) for _ in new]
        c.step_begin(ids, n_new)
        for s, n in zip(ids, n_new):
            assert mgr.reserve(s, n) == O.OK
        assert c.digest() == mgr.digest(), f"churn step {step}: page/slot state diverged"
        nt = sum(n_new)
        c.append(0, kbuf[:nt], kbuf[:nt])
        live = ids
    final_lens = np.array([c.seq_len(s) for s in live])
    q = torch.randn(len(live), H, D, device=c.device, generator=gen).to(torch.float16)
    c.step_begin(live, None)
    got = c.decode(0, q).float().cpu().numpy()
    c.device_status()
    sample = [0, 100, int(np.argmax(final_lens)), len(live) - 1]
    for b, want in oracle_sample(c, live, final_lens, sample, q, "fp16").items():
        assert_close(got[b], want, f"after churn: sequence {b} (len {final_lens[b]})", out_mantissa_bits=10)


def test_c4_fp8_70b_shape_full_size():
    """32 sequences at 32768 tokens, 64 q heads / 8 kv heads, FP8-E4M3 pool: one full layer (2.1 GB)."""
    lens = np.full(32, 32768)
    c, mgr, seqs, gen = build(64, 8, 128, "fp8", lens, seed=4)
    properties(c, seqs, lens, gen, "fp8", sample=[0, 31], fp8=True)
    # one decode step: append 1 token per sequence (lands in the open page), then attention
    H, Hkv, D = 64, 8, 128
    k = torch.randn(32, Hkv, D, device=c.device, generator=gen).to(torch.bfloat16)
    v = torch.randn(32, Hkv, D, device=c.device, generator=gen).to(torch.bfloat16)
    q = torch.randn(32, H, D, device=c.device, generator=gen).to(torch.bfloat16)
    c.step_begin(seqs, [1] * 32)
    for s in seqs:
        assert mgr.reserve(s, 1) == O.OK
    assert c.digest() == mgr.digest()
    c.append(0, k, v)
    got = c.decode(0, q).float().cpu().numpy()
    c.device_status()
    for b, want in oracle_sample(c, seqs, lens + 1, [5], q, "fp8").items():
        assert_close(got[b], want, "FP8 32769-token sequence vs oracle", out_mantissa_bits=7)


def test_c5_long_context_partials_over_8_emulated_ranks():
    """One 131072-token sequence, 8B head shape, bf16.  Eight 'ranks' each hold 16384 tokens and
    produce (o, m, l); the LSE combine of the eight equals one cache holding everything."""
    from titan_engine_b200 import PagedKVCache, _lib as L
    H, Hkv, D, n, R = 32, 8, 128, 131072, 8
    per = n // R
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev); gen.manual_seed(5)
    q = torch.randn(1, H, D, device=dev, generator=gen).to(torch.bfloat16)
    whole = PagedKVCache(1, H, Hkv, D, n // 16, 1, n // 16, dtype="bf16")
    s = whole.seq_alloc()
    whole.adopt(s, np.arange(n // 16, dtype=np.int32), n)
    wpool = whole.layer_views(0)[0]
    wpool.normal_(generator=gen)
    whole.step_begin([s], None)
    want = whole.decode(0, q).float().cpu().numpy()[0]
    parts = []
    for r in range(R):
        c = PagedKVCache(1, H, Hkv, D, per // 16, 1, per // 16, dtype="bf16")
        sr = c.seq_alloc()
        c.adopt(sr, np.arange(per // 16, dtype=np.int32), per)
        c.layer_views(0)[0].copy_(wpool[r * per // 16:(r + 1) * per // 16])
        c.step_begin([sr], None)
        parts.append(c.decode_partial(0, q).clone())
        c.close()
    stacked = torch.stack(parts).contiguous()
    out = torch.empty(H, D, dtype=torch.bfloat16, device=dev)
    assert L.lib().tk_combine_partials(stacked.data_ptr(), R, H, D, out.data_ptr(), L.TK_BF16,
                                       torch.cuda.current_stream().cuda_stream) == 0
    assert_close(out.float().cpu().numpy(), want, "8-rank LSE combine vs single cache", out_mantissa_bits=7)
    # and the single cache against the oracle for two heads' worth of work (kv head 0)
    o = O.Pool(O.BF16, n // 16, H, Hkv, D, 1, n // 16)
    o.pool[:] = from_torch16(wpool)
    ref = o.decode(np.arange(n // 16, dtype=np.int32)[None], [0], [n], from_torch16(q))[0]
    assert_close(want, ref, "131072-token sequence vs oracle", out_mantissa_bits=7)


def test_c5_cold_window_on_one_rank():
    """The share of one rank of the 131072-token sequence (16384 tokens) with every page outside
    the hot window: all 1024 pages per layer live in pinned host memory, are staged back layer by
    layer, and attention equals the all-in-HBM result bit for bit."""
    from titan_engine_b200 import PagedKVCache
    H, Hkv, D, per, L = 32, 8, 128, 16384, 3
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev); gen.manual_seed(55)
    q = torch.randn(1, H, D, device=dev, generator=gen).to(torch.bfloat16)
    data = torch.randn(L, per // 16, Hkv, 2, 16, D, device=dev, generator=gen).to(torch.bfloat16)
    outs = {}
    for tiered in (False, True):
        c = PagedKVCache(L, H, Hkv, D, per // 16, 1, per // 16, dtype="bf16",
                         hot_window=32768 if tiered else 0, cold_pages=per // 16 if tiered else 0)
        s = c.seq_alloc()
        c.adopt(s, np.arange(per // 16, dtype=np.int32), per)
        for l in range(L):
            c.layer_views(l)[0].copy_(data[l])
        if tiered:
            c.set_tail(s, 131072 - per)                 # rank 0 of 8: 114688 tokens follow
        torch.cuda.synchronize()
        c.step_begin([s], None)
        if tiered:
            st = c.stats()
            assert st["pages_cold"] == per // 16 and c.num_free_pages == per // 16
            for l in range(L):
                c.layer_views(l)[0].zero_()             # the device pool no longer holds the data
        outs[tiered] = [c.decode(l, q).clone() for l in range(L)]
        c.device_status()
        if tiered:
            st = c.stats()
            assert st["prefetch_hits"] == (L - 1) * (per // 16) and st["prefetch_misses"] == per // 16
        c.close()
    for l in range(L):
        assert torch.equal(outs[True][l], outs[False][l]), f"layer {l}: staged pages changed the result"
        assert float(outs[True][l].float().abs().max()) > 0
