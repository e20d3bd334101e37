"""GPU parity tests of the paged KV path through the C ABI, against the CPU oracle.

Bit-exact: page tables, slot indices, pool bytes, FP8 codes and scales.
Attention outputs (fp16/bf16): within 2e-3 relative / 1e-2 absolute of the oracle.
"""
import numpy as np
import pytest
import torch

from helpers import DT, Twin, assert_close, from_torch16, normal16, rng, to_torch16
from oracle import tk_oracle as O

pytestmark = pytest.mark.gpu

IMPLS = ["simt", "mma"]


@pytest.fixture(autouse=True)
def _need_cuda():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------------------------
# append: slots and pool bytes
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_append_scatter_bit_exact(dtype):
    t = Twin(2, 8, 2, 64, 96, 4, 32, dtype=dtype, max_step_tokens=1024, seed=21)
    a, b, c = t.seq_alloc(), t.seq_alloc(), t.seq_alloc()
    t.step([a, b, c], [37, 1, 160], check_pool=True, decode=False)      # ragged prefill
    t.step([a, b, c], [1, 1, 1], check_pool=True, decode=False)
    t.seq_free(b)
    d = t.seq_alloc()
    t.step([c, d, a], [16, 33, 0], check_pool=True, decode=False)       # reuse of freed pages
    t.step([], [], check_pool=True, decode=False)                        # empty step


@pytest.mark.parametrize("io", ["bf16", "fp16"])
def test_append_fp8_codes_and_scales_bit_exact(io):
    t = Twin(2, 16, 2, 128, 64, 3, 24, dtype="fp8", io=io, max_step_tokens=1024, seed=22)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [70, 5], check_pool=True, decode=False, outlier_p=0.01)
    t.step([a, b], [1, 11], check_pool=True, decode=False, outlier_p=0.01)   # b fills its first page exactly
    t.step([a, b], [9, 40], check_pool=True, decode=False, outlier_p=0.01)   # a seals page 4 from open + new rows
    for _ in range(18):
        t.step([a, b], [1, 1], check_pool=True, decode=False, outlier_p=0.01)
    assert t.gpu.stats()["pages_sealed"] > 8


def test_fp8_all_zero_page_uses_clamped_scale():
    t = Twin(1, 8, 1, 128, 8, 1, 8, dtype="fp8", max_step_tokens=64, seed=23)
    s = t.seq_alloc()
    t.gpu.step_begin([s], [16]); assert t.mgr.reserve(s, 16) == O.OK
    z = np.zeros((16, 1, 128), dtype=np.uint16)
    t.pools[0].append(t.mgr.table(), np.zeros(16, np.int32), np.arange(16, dtype=np.int32), z, z)
    t.gpu.append(0, to_torch16(z, O.BF16, t.dev), to_torch16(z, O.BF16, t.dev))
    t.check_pool(0)
    _, scales, _ = t.gpu.layer_views(0)
    assert scales[0, 0, 0].item() == np.float32(1e-10)


# ---------------------------------------------------------------------------------------------
# decode attention
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n", [1, 15, 16, 17, 255, 256, 257])
def test_decode_page_boundaries(impl, n):
    t = Twin(1, 8, 2, 64, 40, 2, 20, dtype="fp16", impl=impl, chunk_tokens=128, max_step_tokens=512, seed=30 + n)
    s = t.seq_alloc()
    t.step([s], [n])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("shape", [
    # H, Hkv, D, dtype
    (8, 2, 64, "fp16"),      # tiny config
    (32, 8, 128, "bf16"),    # 8B head shape
    (32, 8, 128, "fp16"),
    (4, 4, 128, "bf16"),     # MHA, G=1
    (16, 1, 64, "bf16"),     # MQA, G=16
    (16, 8, 64, "bf16"),     # G=2
])
def test_decode_shapes_ragged_batch(impl, shape):
    H, Hkv, D, dtype = shape
    t = Twin(2, H, Hkv, D, 400, 6, 80, dtype=dtype, impl=impl, max_step_tokens=4096, seed=40)
    seqs = [t.seq_alloc() for _ in range(5)]
    t.step(seqs, [1000, 3, 129, 512, 77])
    t.step(seqs, [1, 1, 1, 1, 1])
    t.step(seqs[1:4], None)                               # decode only, subset, no append
    assert t.max_err > 0                                  # outputs are not trivially equal/zero


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("chunk", [16, 64, 0])
def test_decode_split_kv_chunkings_agree(impl, chunk):
    t = Twin(1, 32, 8, 128, 300, 3, 100, dtype="bf16", impl=impl, chunk_tokens=chunk, max_step_tokens=2048, seed=41)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [1500, 260])


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("io", ["bf16", "fp16"])
def test_decode_fp8(impl, io):
    t = Twin(2, 64, 8, 128, 200, 4, 64, dtype="fp8", io=io, impl=impl, max_step_tokens=2048, seed=42)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [700, 16, 5], check_pool=True, outlier_p=0.01)       # sealed + open, exactly one page, open only
    for _ in range(12):
        t.step(seqs, [1, 1, 1], outlier_p=0.01)                       # crosses a seal for two sequences
    t.check_pool(1)


@pytest.mark.parametrize("heads", [(8, 8), (16, 8), (32, 8), (64, 8), (64, 4)])
def test_decode_fp8_group_sizes(heads):
    """FP8 pools with a group of at most 8 query heads run both products transposed (the heads are the MMA's 8
    columns; groups of 1, 2, 4 leave columns empty), larger groups keep the heads as rows.  Long enough for
    several split-KV chunks per sequence; outliers move the reference maximum late in a sequence."""
    H, Hkv = heads
    t = Twin(1, H, Hkv, 128, 260, 3, 200, dtype="fp8", io="bf16", impl="mma", chunk_tokens=512, max_step_tokens=4096, seed=45)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [3000, 300, 17], check_pool=True, outlier_p=0.01)
    for _ in range(3):
        t.step(seqs, [1, 1, 1], outlier_p=0.01, f32_out=True)        # FP32 results: the stated tolerance with no slack
    t.gpu.device_status()


@pytest.mark.parametrize("shape", [(8, 2, 64, "fp16"), (32, 8, 128, "bf16"), (16, 1, 128, "fp16")])
def test_fused_append_decode_single_launch(shape):
    """Decode steps through tk_kv_append_decode: the attention kernel writes the new token's rows
    itself.  Outputs and the pool bytes it leaves behind must match append-then-decode."""
    H, Hkv, D, dtype = shape
    t = Twin(2, H, Hkv, D, 200, 5, 48, dtype=dtype, impl="mma", max_step_tokens=2048, seed=50)
    seqs = [t.seq_alloc() for _ in range(4)]
    t.step(seqs, [14, 16, 250, 1], fused=True, check_pool=True)      # prefill: falls back to two kernels
    n0 = t.gpu.launch_count
    t.step(seqs, [1, 1, 1, 1], fused=True, check_pool=True)          # rows 14, 0 (fresh page), 10, 1
    assert t.gpu.launch_count - n0 <= 1 + 2                           # page-table patch + one kernel per layer
    for i in range(20):
        t.step(seqs, [1, 1, 1, i % 2], fused=True, check_pool=(i % 5 == 0))   # one sequence sometimes idle
    t.step(seqs[:2], [1, 1], fused=True, check_pool=True)
    for layer in range(2):
        t.check_pool(layer)


def test_decode_shuffled_pool_c2_style():
    """Page tables as inputs: a seeded permutation of the pool, batch of ragged contexts."""
    H, Hkv, D = 32, 8, 128
    g = rng(2)
    lens = g.integers(64, 700, size=12)
    n_pages = int(sum((l + 15) // 16 for l in lens)) + 12
    t = Twin(1, H, Hkv, D, n_pages, 12, 64, dtype="bf16", impl="mma", max_step_tokens=8192, seed=43)
    perm = g.permutation(n_pages).astype(np.int32)
    bits = normal16(g, t.pools[0].pool.shape, O.BF16)            # the pool arrives already filled
    t.pools[0].pool[:] = bits
    t.gpu.layer_views(0)[0].copy_(to_torch16(bits, O.BF16, t.dev))
    seqs, at = [], 0
    for l in lens:
        s = t.seq_alloc()
        npg = (int(l) + 15) // 16
        t.adopt(s, perm[at:at + npg], int(l))
        at += npg
        seqs.append(s)
    # one decode step per layer: append 1 token per sequence, then attention over everything
    t.step(seqs, [1] * len(seqs), check_pool=True)
    np.testing.assert_array_equal(t.gpu.page_table(seqs[0])[:3], perm[:3])


def test_tiny_config_prefill_then_64_decode_steps():
    """Tiny workload: 1 sequence, 8 q heads / 2 kv heads, D 64, 2 layers, fp16; 512-token prefill via
    append, then 64 decode steps; pages come off the free list as 0,1,2,..."""
    for impl in IMPLS:
        t = Twin(2, 8, 2, 64, 40, 1, 40, dtype="fp16", impl=impl, max_step_tokens=512, seed=1)
        s = t.seq_alloc()
        t.step([s], [512], check_pool=True)
        for _ in range(64):
            t.step([s], [1])
        np.testing.assert_array_equal(t.gpu.page_table(s), np.arange(36))
        t.check_pool(0); t.check_pool(1)


def test_known_answers_on_gpu():
    """Closed-form cases straight through the CUDA path: equal keys -> mean of V; one token -> V."""
    for impl in IMPLS:
        t = Twin(1, 8, 2, 64, 8, 1, 8, dtype="fp16", impl=impl, max_step_tokens=128, seed=5)
        s = t.seq_alloc()
        n = 40
        t.gpu.step_begin([s], [n])
        g = rng(6)
        k = np.repeat(normal16(g, (1, 2, 64), O.FP16), n, axis=0)
        v = normal16(g, (n, 2, 64), O.FP16)
        q = normal16(g, (1, 8, 64), O.FP16)
        t.gpu.append(0, to_torch16(k, O.FP16, t.dev), to_torch16(v, O.FP16, t.dev))
        out = t.gpu.decode(0, to_torch16(q, O.FP16, t.dev)).float().cpu().numpy()[0]
        vf = O.to_f32(v, O.FP16)
        for h in range(8):
            assert_close(out[h], vf[:, h // 4].mean(0), f"{impl}: uniform weights, head {h}")


def test_host_buffer_entry_point():
    t = Twin(2, 32, 8, 128, 120, 4, 40, dtype="bf16", max_step_tokens=1024, seed=44)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [300, 17, 64], host_api=True)
    t.step(seqs, [1, 1, 1], host_api=True)
    st = t.gpu.stats()
    assert st["bytes_h2d"] > 0 and st["bytes_d2h"] > 0 and t.gpu.launch_count > 0


def test_host_buffer_async_groups_equal_device_path():
    """tk_kv_append_decode_host_async holds its kernel launches back and issues them in groups (1, 1, 2, 2, 4, ...):
    eleven layers per step through it - so that groups of every size and a partly filled last group occur - against a
    second cache driven through the device entry point with the same rows; a device call in the middle of a step and
    the next step_begin both have to issue what is held back first.  Outputs and pools must be identical."""
    from titan_engine_b200 import PagedKVCache
    Lyr, H, Hkv, D, B = 11, 32, 8, 128, 5
    dev = torch.device("cuda")
    mk = lambda: PagedKVCache(Lyr, H, Hkv, D, 64, B, 12, dtype="bf16", max_step_tokens=256)
    a, b = mk(), mk()
    sa = [a.seq_alloc() for _ in range(B)]; sb = [b.seq_alloc() for _ in range(B)]
    gen = torch.Generator(device="cpu"); gen.manual_seed(7)
    for step, n_new in enumerate([[40, 3, 17, 1, 16], [1] * B, [1] * B, [1] * B]):
        n_tok = sum(n_new)
        hk = [torch.randn(n_tok, Hkv, D, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(Lyr)]
        hv = [torch.randn(n_tok, Hkv, D, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(Lyr)]
        hq = [torch.randn(B, H, D, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(Lyr)]
        ho = [torch.zeros(B, H, D, dtype=torch.bfloat16).pin_memory() for _ in range(Lyr)]
        a.step_begin(sa, n_new); b.step_begin(sb, n_new)
        ref = [b.append_decode(l, hk[l].to(dev), hv[l].to(dev), hq[l].to(dev)) for l in range(Lyr)]
        for l in range(Lyr):
            if step == 2 and l == 7:                        # a device call between two held-back host calls
                a.append_decode(l, hk[l].to(dev), hv[l].to(dev), hq[l].to(dev), out=(tmp := torch.empty(B, H, D, dtype=torch.bfloat16, device=dev)))
                ho[l].copy_(tmp)
            else:
                a.append_decode_host_async(l, hk[l], hv[l], hq[l], ho[l])
        if step != 1:                                        # step 1 leaves its last group to the next step_begin
            a.host_wait()
            torch.cuda.synchronize()
            for l in range(Lyr):
                assert torch.equal(ho[l], ref[l].cpu()), f"step {step} layer {l}"
        else:
            keep = (ho, ref)
        if step == 2:                                        # by now step 1's copies have landed too
            for l in range(Lyr):
                assert torch.equal(keep[0][l], keep[1][l].cpu()), f"step 1 layer {l}"
    torch.cuda.synchronize()
    for l in range(Lyr):
        assert torch.equal(a.layer_views(l)[0], b.layer_views(l)[0]), f"pool of layer {l}"
    a.device_status(); b.device_status()


def test_partials_and_cross_rank_combine():
    """Two 'ranks' each hold half of one sequence; merged partials equal single-cache attention."""
    from titan_engine_b200 import _lib as L
    H, Hkv, D, n = 32, 8, 128, 640
    g = rng(45)
    k = normal16(g, (n, Hkv, D), O.BF16); v = normal16(g, (n, Hkv, D), O.BF16); q = normal16(g, (1, H, D), O.BF16)
    dev = torch.device("cuda")
    from titan_engine_b200 import PagedKVCache
    parts = []
    for lo, hi in ((0, 320), (320, n)):
        c = PagedKVCache(1, H, Hkv, D, 64, 1, 64, dtype="bf16", max_step_tokens=1024)
        s = c.seq_alloc()
        c.step_begin([s], [hi - lo])
        c.append(0, to_torch16(k[lo:hi], O.BF16, dev), to_torch16(v[lo:hi], O.BF16, dev))
        parts.append(c.decode_partial(0, to_torch16(q, O.BF16, dev)))
        c.close()
    stacked = torch.stack(parts).contiguous()                  # [2][1][H][D+2]
    out = torch.empty(H, D, dtype=torch.bfloat16, device=dev)
    st = L.lib().tk_combine_partials(stacked.data_ptr(), 2, H, D, out.data_ptr(), L.TK_BF16,
                                     torch.cuda.current_stream().cuda_stream)
    assert st == 0
    want = O.attention_decode_f32(O.to_f32(q[0], O.BF16), O.to_f32(k, O.BF16), O.to_f32(v, O.BF16), H, Hkv, D, n)
    assert_close(out.float().cpu().numpy(), want, "2-rank LSE combine")
    # the partial format itself: (o, m, l) of rank 0 against the oracle's partial
    pool = O.Pool(O.BF16, 64, H, Hkv, D, 1, 64)
    table = np.arange(64, dtype=np.int32)[None]
    pool.append(table, np.zeros(320, np.int32), np.arange(320, dtype=np.int32), k[:320], v[:320])
    m, l, o = pool.decode_partial(table, 0, 320, 0, 320, q[0])
    p0 = parts[0][0].cpu().numpy()
    np.testing.assert_allclose(p0[:, D], m, rtol=1e-3, atol=2e-3)
    scale = np.exp(m - p0[:, D])                               # bring both to the same reference max
    assert_close(p0[:, D + 1], l * scale, "partial l", rtol=5e-3)
    assert_close(p0[:, :D], o * scale[:, None], "partial o", rtol=5e-3, atol=5e-2)


def test_churn_small_bit_exact_and_close():
    """Continuous-batching churn on a small pool: retire / admit / append every step."""
    t = Twin(1, 32, 8, 128, 700, 16, 64, dtype="fp16", impl="mma", max_step_tokens=4096, seed=3)
    g = rng(33)
    live = []
    for _ in range(16):
        s = t.seq_alloc()
        live.append(s)
    t.step(live, [int(min(600, max(1, round(float(np.exp(g.normal(np.log(120.0), 1.0))))))) for _ in live], decode=False)
    for step in range(12):
        for s in sorted(g.choice(live, size=2, replace=False).tolist()):
            t.seq_free(s); live.remove(s)
        new = [t.seq_alloc() for _ in range(2)]
        ids = sorted(live) + new
        t.step(ids, [1] * len(live) + [int(g.integers(16, 200)) for _ in new], check_pool=(step % 4 == 0))
        live = ids


@pytest.mark.parametrize("impl", IMPLS)
def test_cold_tier_eviction_and_prefetch(impl):
    """Pages older than the hot window move to pinned host memory and are staged back one layer
    ahead.  State (page ids, cold ids, free lists) is bit-exact against the oracle's tiering rule;
    attention equals the untiered oracle: where a page lives must not change any result."""
    t = Twin(3, 32, 8, 128, 80, 3, 200, dtype="bf16", impl=impl, max_step_tokens=4096, seed=60,
             hot_window=128, cold_pages=400)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [1000, 100])                  # pages written by this step stay hot for it
    assert t.gpu.stats()["pages_cold"] == 0
    t.step([a, b], [1, 1])                       # a: 54 pages go cold at once; b: entirely hot
    st = t.gpu.stats()
    assert st["pages_cold"] == (1001 - 128) // 16 and st["evictions"] == st["pages_cold"]
    assert t.gpu.num_free_pages == 80 - (63 - 54) - 7
    for i in range(40):                          # decode steps: pages keep falling out of the window
        t.step([a, b], [1, 1], fused=(i % 2 == 0))
    st = t.gpu.stats()
    assert st["pages_cold"] == (1041 - 128) // 16 + (141 - 128) // 16
    assert st["prefetch_hits"] > 0 and st["prefetch_misses"] > 0 and st["bytes_d2h"] > 0
    t.seq_free(a)                                # cold ids go back to their own free list
    c = t.seq_alloc()
    t.step([c, b], [500, 1])
    t.step([c, b], [1, 1], fused=True)           # 23 of c's pages are cold now
    assert t.gpu.seq_len(c) == 501 and t.gpu.stats()["pages_cold"] == (501 - 128) // 16 + (143 - 128) // 16


@pytest.mark.parametrize("shape", [(32, 8, 128, "bf16"), (8, 2, 64, "fp16")])
def test_rope_append_decode_fused(shape):
    """apply_rope -> update -> attention_decode as one call (one kernel on decode steps).  The oracle
    rotates in FP32 exactly as the reference's rope_kernel, rounds to the storage type, appends and
    attends; K rows may differ from it by one unit in the last place of the 16-bit type (device
    powf/sinf/cosf vs libm), V rows not at all."""
    H, Hkv, D, dtype = shape
    dt = DT[dtype]
    theta = 500000.0
    t = Twin(2, H, Hkv, D, 120, 3, 60, dtype=dtype, impl="mma", max_step_tokens=1024, seed=70)
    seqs = [t.seq_alloc() for _ in range(3)]
    g = rng(71)

    def rot(x16, heads, positions):                     # x16: [rows][heads][D] bits; one position per row
        xf = O.to_f32(x16, dt)
        out = np.empty_like(xf)
        for r, pos in enumerate(positions):
            if heads == H:
                out[r], _ = O.rope_f32(xf[r], np.zeros((Hkv, D), np.float32), H, Hkv, D, int(pos), theta)
            else:
                _, out[r] = O.rope_f32(np.zeros((H, D), np.float32), xf[r], H, Hkv, D, int(pos), theta)
        return O.f32_to_16(out, dt)

    def step(n_new):
        old = [t.gpu.seq_len(s) for s in seqs]
        t.gpu.step_begin(seqs, n_new)
        for s, n in zip(seqs, n_new):
            assert t.mgr.reserve(s, n) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
        table = t.mgr.table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seqs, n_new)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)])
        lens = [t.gpu.seq_len(s) for s in seqs]
        n0 = t.gpu.launch_count
        for layer in range(2):
            k16 = normal16(g, (len(tok_seq), Hkv, D), dt); v16 = normal16(g, (len(tok_seq), Hkv, D), dt)
            q16 = normal16(g, (3, H, D), dt)
            got = t.gpu.rope_append_decode(layer, to_torch16(k16, dt, t.dev), to_torch16(v16, dt, t.dev),
                                           to_torch16(q16, dt, t.dev), theta).float().cpu().numpy()
            t.pools[layer].append(table, tok_seq, tok_pos, rot(k16, Hkv, tok_pos), v16)
            want = t.pools[layer].decode(table, seqs, lens, rot(q16, H, [n - 1 for n in lens]))
            assert_close(got, want, f"rope+append+decode layer {layer}", out_mantissa_bits=7 if dt == O.BF16 else 10)
            pool = from_torch16(t.gpu.layer_views(layer)[0])
            np.testing.assert_array_equal(pool[:, :, 1], t.pools[layer].pool[:, :, 1])       # V: plain copy
            kg, kw = O.to_f32(pool[:, :, 0], dt), O.to_f32(t.pools[layer].pool[:, :, 0], dt)
            # one unit in the last place; near zero the angle error (an ulp of freq times the position)
            # dominates, so magnitudes are floored at 0.05 for the purpose of the bound
            ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(kw), 0.05))) - (7 if dt == O.BF16 else 10))
            assert (np.abs(kg - kw) <= ulp).all(), "rotated K rows differ by more than one ulp"
            assert (kg == kw).mean() > 0.98
        return t.gpu.launch_count - n0

    step([300, 17, 1])                                  # prefill: rope kernel + append + decode
    launches = step([1, 1, 1])                          # decode step: one kernel per layer (+ table patch, + cos/sin table)
    assert launches <= 4
    for _ in range(20):
        step([1, 1, 1])
    t.gpu.device_status()


@pytest.mark.parametrize("impl", ["mma", "simt"])
@pytest.mark.parametrize("heads", [(16, 16), (32, 8)])
def test_rope_append_decode_mla_shape(heads, impl):
    """The MLA layer step as one call: apply_rope_mla (only the 64 rope dims at the end of the 192-wide q / K
    rows rotate) -> update -> attention_decode_mla.  Oracle: rope_mla_f32 in FP32, rounded to the storage
    type, appended, attended; K rows may differ by one unit in the last place, V rows not at all."""
    H, Hkv = heads
    D, Dv, nope, rope = 192, 128, 128, 64
    dt, theta = O.BF16, 10000.0
    t = Twin(2, H, Hkv, D, 120, 3, 60, dtype="bf16", impl=impl, max_step_tokens=1024, seed=72, Dv=Dv)
    seqs = [t.seq_alloc() for _ in range(3)]
    g = rng(73)

    def rot(x16, is_q, positions):                      # x16: [rows][heads][192] bits; one position per row
        xf = O.to_f32(x16, dt)
        out = np.empty_like(xf)
        for r, pos in enumerate(positions):
            if is_q:
                out[r], _ = O.rope_mla_f32(xf[r], np.zeros((Hkv, D), np.float32), H, Hkv, nope, rope, int(pos), theta)
            else:
                _, out[r] = O.rope_mla_f32(np.zeros((H, D), np.float32), xf[r], H, Hkv, nope, rope, int(pos), theta)
        return O.f32_to_16(out, dt)

    def step(n_new):
        old = [t.gpu.seq_len(s) for s in seqs]
        t.gpu.step_begin(seqs, n_new)
        for s, n in zip(seqs, n_new):
            assert t.mgr.reserve(s, n) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
        table = t.mgr.table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seqs, n_new)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)])
        lens = [t.gpu.seq_len(s) for s in seqs]
        q_pos = [n - 1 for n in lens]
        n0 = t.gpu.launch_count
        for layer in range(2):
            k16 = normal16(g, (len(tok_seq), Hkv, D), dt); v16 = normal16(g, (len(tok_seq), Hkv, Dv), dt)
            q16 = normal16(g, (3, H, D), dt)
            got = t.gpu.rope_append_decode(layer, to_torch16(k16, dt, t.dev), to_torch16(v16, dt, t.dev),
                                           to_torch16(q16, dt, t.dev), theta).float().cpu().numpy()
            t.pools[layer].append(table, tok_seq, tok_pos, rot(k16, False, tok_pos), v16)
            want = t.pools[layer].decode(table, seqs, lens, rot(q16, True, q_pos))
            assert_close(got, want, f"rope+append+decode (MLA shape) layer {layer}", out_mantissa_bits=7)
            pool = from_torch16(t.gpu.layer_views(layer)[0])                     # [pages][Hkv][16*192 K | 16*128 V]
            np.testing.assert_array_equal(pool[:, :, 16 * D:], t.pools[layer].pool[:, :, 16 * D:])   # V: plain copy
            kg = O.to_f32(pool[:, :, :16 * D], dt).reshape(-1, 16, D)
            kw = O.to_f32(t.pools[layer].pool[:, :, :16 * D], dt).reshape(-1, 16, D)
            np.testing.assert_array_equal(kg[:, :, :nope], kw[:, :, :nope])      # nope dims: plain copy
            ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(kw), 0.05))) - 7)
            assert (np.abs(kg - kw) <= ulp).all(), "rotated K rows differ by more than one ulp"
            assert (kg == kw).mean() > 0.98
        return t.gpu.launch_count - n0

    step([300, 17, 1])                                  # prefill: rope kernel + append + decode
    launches = step([1, 1, 1])
    if impl == "mma":
        assert launches <= 4                            # one kernel per layer (+ table patch, + cos/sin table)
    for _ in range(18):
        step([1, 1, 1])
    t.gpu.device_status()


def test_scheduler_drives_churn_on_gpu():
    """The continuous-batching scheduler as the caller: requests arrive, prefill in chunks, decode,
    finish and get preempted on a small pool; every step's page state is bit-exact against the
    oracle manager and the attention output of EVERY token of every row - each prompt token of a
    prefill chunk included, as the reference's per-token prefill loop computes them
    (src/inference/engine.cpp:182-193) - within tolerance of the oracle."""
    from titan_engine_b200.scheduler import BatchScheduler
    t = Twin(1, 32, 8, 128, 48, 6, 48, dtype="fp16", impl="mma", max_step_tokens=256 + 6, seed=80)
    s = BatchScheduler(t.gpu, max_batch_size=6, max_prefill_tokens=256)
    g = rng(81)
    for _ in range(10):
        s.submit(int(g.integers(30, 300)), int(g.integers(5, 60)))
    steps = multi_steps = 0
    for _ in range(3000):
        rows = s.next()
        ev = s.last_events()
        for q in ev["retired"]:
            assert t.mgr.seq_free(q) == O.OK
        for q in ev["admitted"]:
            assert t.mgr.seq_alloc() == q
        for q in ev["preempted"]:
            assert t.mgr.seq_free(q) == O.OK
        if not rows and s.stats()["queued_requests"] == 0:
            break
        if rows:
            if max(r.n_new for r in rows) > 1:
                t.step([r.seq for r in rows], [r.n_new for r in rows], begun=True, every_token=True)
                multi_steps += 1
            else:
                t.step([r.seq for r in rows], [r.n_new for r in rows], begun=True, fused=(steps % 2 == 0))
            steps += 1
        s.commit([bool(g.random() < 0.02) for _ in rows])
    st = s.stats()
    assert st["completed_requests"] == 10 and st["active_requests"] == 0 and steps > 50 and multi_steps >= 5
    assert t.gpu.num_free_pages == 48 and t.gpu.digest() == t.mgr.digest()


def test_bounded_device_wait_reports_timeout_and_context_survives():
    """Failure detection without a fault: a device wait that nothing satisfies runs out after its
    limit, the kernel returns, the host reads TK_TIMEOUT, and the same handle keeps working."""
    from titan_engine_b200 import KvError, _lib as L
    t = Twin(1, 8, 2, 64, 16, 1, 16, dtype="fp16", impl="mma", max_step_tokens=64, seed=90)
    s = t.seq_alloc()
    t.step([s], [40])
    st = t.gpu._lib.tk_kv_selftest_bounded_wait(t.gpu._h, 50, torch.cuda.current_stream().cuda_stream)
    assert st == L.TK_OK
    with pytest.raises(KvError) as e:
        t.gpu.device_status()
    assert e.value.status == L.TK_TIMEOUT
    t.gpu.device_status()                     # the word was cleared
    t.step([s], [1])                          # and the context is fine


@pytest.mark.parametrize("impl", ["mma", "simt"])
def test_pending_timeout_leaves_the_output_alone(impl):
    """Fail closed.  With the handle's status word saying that a device wait gave up (set from the host
    here; no wait is made to run out), an attention launch writes nothing: `out` keeps its previous
    bytes, tk_kv_device_status reports TK_TIMEOUT and clears the word, and the next launch works."""
    from titan_engine_b200 import KvError, _lib as L
    t = Twin(1, 32, 8, 128, 64, 2, 40, dtype="bf16", impl=impl, max_step_tokens=1024, seed=93)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [600, 33])
    q = to_torch16(normal16(t.g, (2, 32, 128), O.BF16), O.BF16, t.dev)
    t.gpu.step_begin([a, b], None)
    good = t.gpu.decode(0, q).clone()
    sentinel = torch.full_like(good, 7.0)
    out = sentinel.clone()
    t.gpu.selftest_set_status(L.TK_TIMEOUT)
    t.gpu.decode(0, q, out)
    torch.cuda.synchronize()
    assert torch.equal(out, sentinel), "a launch with a pending time-out wrote to `out`"
    with pytest.raises(KvError) as e:
        t.gpu.device_status()
    assert e.value.status == L.TK_TIMEOUT
    t.gpu.device_status()                                  # cleared
    t.gpu.decode(0, q, out)
    assert torch.equal(out, good)


def test_edge_cases_on_gpu():
    """Empty and maximal inputs: a sequence with no tokens attends to nothing (output 0, the
    reference's 0/(0+1e-8)); a sequence filling its whole page-table row; pool exhaustion that must
    leave the device state untouched; FP8 with head_dim 64 (no tensor-core path: generic kernel)."""
    from titan_engine_b200 import KvError, _lib as L
    t = Twin(1, 8, 2, 64, 12, 3, 8, dtype="fp16", impl="mma", max_step_tokens=256, seed=95)
    a, b, c = t.seq_alloc(), t.seq_alloc(), t.seq_alloc()
    outs = t.step([a, b, c], [128, 0, 5])                 # a fills all 8 entries of its row; b is empty
    assert np.all(outs[0][1] == 0.0)
    with pytest.raises(KvError) as e:
        t.gpu.step_begin([a], [1])                        # a 9th page does not fit the row
    assert e.value.status == L.TK_INVALID_ARG
    with pytest.raises(KvError) as e:
        t.gpu.step_begin([b, c], [40, 30])                # 3 + 2 more pages, 3 free
    assert e.value.status == L.TK_OUT_OF_PAGES
    assert t.gpu.digest() == t.mgr.digest()               # nothing changed
    t.step([c, b], [11, 33])                              # exactly the 3 free pages
    assert t.gpu.num_free_pages == 0
    t.step([a, b, c], None, fused=False)                  # decode only on a full pool

    f = Twin(1, 8, 2, 64, 16, 2, 8, dtype="fp8", io="fp16", impl="auto", max_step_tokens=256, seed=96)
    s = f.seq_alloc()
    f.step([s], [50], check_pool=True)
    for _ in range(15):
        f.step([s], [1], check_pool=True, fused=True)


@pytest.mark.parametrize("dtype", ["bf16", "fp8"])
def test_fork_prefix_sharing(dtype):
    """Two sequences share the pages of a common prefix; each then appends its own tokens.  Page
    state is bit-exact against the oracle, attention of both within tolerance, and freeing one of
    them leaves the other intact."""
    t = Twin(2, 32, 8, 128, 64, 4, 32, dtype=dtype, impl="mma", max_step_tokens=1024, seed=97)
    a = t.seq_alloc()
    t.step([a], [200], check_pool=True)                   # 12 full pages + 8 tokens
    b = t.fork(a)
    assert t.gpu.page_table(b)[:12].tolist() == t.gpu.page_table(a)[:12].tolist()
    assert t.gpu.page_table(b)[12] != t.gpu.page_table(a)[12]
    t.step([a, b], [1, 1], check_pool=True, fused=True)   # diverge: different tokens in their own last pages
    for i in range(12):
        t.step([a, b], [1, 3 if i % 2 else 1], check_pool=(i % 4 == 0), fused=(i % 2 == 0))
    c = t.fork(b)
    t.step([a, b, c], [1, 1, 17], check_pool=True)
    t.seq_free(a)
    t.step([b, c], [1, 1], check_pool=True, fused=True)
    t.seq_free(b); t.seq_free(c)
    assert t.gpu.num_free_pages == 64


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
@pytest.mark.parametrize("impl", ["mma", "simt"])
@pytest.mark.parametrize("heads", [(16, 16), (32, 8), (16, 2)])
def test_mla_cache_shape(heads, impl, dtype):
    """K rows of 192, V rows and outputs of 128 (the MLA cache): append, decode, churn, host entry
    point; pool bytes bit-exact, attention within tolerance.  Both kernels: the tensor-core one
    (groups of up to 8 query heads) and the generic one."""
    H, Hkv = heads
    t = Twin(2, H, Hkv, 192, 60, 3, 40, dtype=dtype, impl=impl, max_step_tokens=1024, seed=98, Dv=128)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [300, 17], check_pool=True)
    for i in range(20):
        t.step([a, b], [1, 1], check_pool=(i % 5 == 0), fused=(i % 2 == 0))
    t.seq_free(a)
    c = t.seq_alloc()
    t.step([c, b], [33, 1], check_pool=True, host_api=True)
    assert t.gpu.cfg.v_head_dim == 128


def test_mla_split_kv_long_context_and_chunks():
    """MLA shape on the tensor-core kernel with several split-KV chunks per sequence, ragged lengths
    (partly filled last pages) and fused decode-step appends that cross page boundaries."""
    t = Twin(1, 8, 8, 192, 700, 4, 200, dtype="bf16", impl="mma", max_step_tokens=4096, seed=5, Dv=128,
             chunk_tokens=256)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [2500, 1, 1023], check_pool=True)
    for i in range(36):
        t.step(seqs, [1, 1, 1], check_pool=(i % 12 == 0), fused=True)
    t.step(seqs[:2], [1, 40], check_pool=True)


def test_mla_wide_group_falls_back_to_generic_kernel():
    """Groups of more than 8 query heads are outside the MLA tensor-core kernel: auto picks the generic one,
    an explicit request for it is refused."""
    from titan_engine_b200 import KvError, PagedKVCache
    t = Twin(1, 16, 1, 192, 20, 1, 20, dtype="fp16", impl="auto", max_step_tokens=256, seed=6, Dv=128)
    s = t.seq_alloc()
    t.step([s], [100], check_pool=True)
    t.step([s], [1], check_pool=True, fused=True)
    with pytest.raises(KvError):
        PagedKVCache(1, 16, 1, 192, 20, 1, 20, dtype="fp16", decode_impl="mma", v_head_dim=128)


def test_shard_by_kv_head_outputs_are_head_slices_of_the_whole():
    """The other way to spread a small batch over GPUs: rank r keeps kv heads [r*Hkv/N, ...) and the query
    heads that map onto them.  Two such caches (both on this GPU) fed the matching slices of k, v and q
    must reproduce, head for head, the outputs of one cache holding every head."""
    from titan_engine_b200 import PagedKVCache
    from titan_engine_b200 import dist as D
    H, Hkv, Dh, world = 32, 8, 128, 2
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev); gen.manual_seed(77)
    lens = [700, 33, 1500]
    mk = lambda h, hkv: PagedKVCache(1, h, hkv, Dh, 200, 3, 100, dtype="bf16", max_step_tokens=4096, chunk_tokens=256)
    whole = mk(H, Hkv)
    shards = [mk(H // world, Hkv // world) for _ in range(world)]
    seqs = [whole.seq_alloc() for _ in lens]
    for c in shards:
        assert [c.seq_alloc() for _ in lens] == seqs
    n = sum(lens)
    k = torch.randn(n, Hkv, Dh, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(n, Hkv, Dh, device=dev, generator=gen).to(torch.bfloat16)
    q = torch.randn(len(lens), H, Dh, device=dev, generator=gen).to(torch.bfloat16)
    whole.step_begin(seqs, lens)
    whole.append(0, k, v)
    want = whole.decode(0, q)
    for r, c in enumerate(shards):
        kvr, qr = D.shard_kv_heads(Hkv, H, r, world)
        c.step_begin(seqs, lens)
        c.append(0, k[:, kvr.start:kvr.stop].contiguous(), v[:, kvr.start:kvr.stop].contiguous())
        got = c.decode(0, q[:, qr.start:qr.stop].contiguous())
        assert torch.equal(got, want[:, qr.start:qr.stop]), f"rank {r}"
        c.close()
    whole.close()


@pytest.mark.parametrize("shape", [
    # H, Hkv, D, dtype, tokens per sequence and step
    (32, 8, 128, "bf16", 4),     # 8B head shape: 4 heads x 4 tokens fill the 16 rows of the tile
    (32, 8, 128, "fp16", 3),
    (8, 2, 64, "fp16", 4),
    (16, 16, 128, "bf16", 16),   # MHA: 16 tokens
    (16, 16, 64, "bf16", 5),
    (16, 1, 64, "fp16", 1),      # 16 heads per kv head: one token per pass
    (16, 1, 64, "fp16", 3),      # ... three tokens: three token groups
    (64, 8, 128, "bf16", 5),     # 70B head shape: 2 tokens per pass, 3 groups (the last one half full)
    (32, 8, 128, "bf16", 19),    # 5 groups
])
def test_decode_multi_tokens_causal(shape):
    """Every token a step appended gets its own attention output, causal among the step's tokens, from one
    pass over the pages (the verification of drafted tokens).  Oracle: the single-token decode of the
    oracle, once per token, with the length cut at that token.  Then the rejected tokens are rolled back."""
    H, Hkv, D, dtype, k = shape
    dt = DT[dtype]
    t = Twin(2, H, Hkv, D, 300, 4, 80, dtype=dtype, impl="mma", max_step_tokens=2048, seed=90, chunk_tokens=256)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [700, 13, 250])
    g = rng(91)
    bits = 7 if dt == O.BF16 else 10

    def multi_step(n_new):
        old = [t.gpu.seq_len(s) for s in seqs]
        t.gpu.step_begin(seqs, n_new)
        for s, n in zip(seqs, n_new):
            assert t.mgr.reserve(s, n) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
        table = t.mgr.table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seqs, n_new)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)])
        n0 = t.gpu.launch_count
        for layer in range(2):
            k16 = normal16(g, (len(tok_seq), Hkv, D), dt); v16 = normal16(g, (len(tok_seq), Hkv, D), dt)
            q16 = normal16(g, (len(tok_seq), H, D), dt)
            t.gpu.append(layer, to_torch16(k16, dt, t.dev), to_torch16(v16, dt, t.dev))
            t.pools[layer].append(table, tok_seq, tok_pos, k16, v16)
            got = t.gpu.decode_multi(layer, to_torch16(q16, dt, t.dev)).float().cpu().numpy()
            want = t.pools[layer].decode(table, tok_seq, tok_pos + 1, q16)       # token by token, as the reference would
            assert_close(got, want, f"multi-token attention layer {layer} {n_new}", out_mantissa_bits=bits)
        assert t.gpu.launch_count - n0 == 2 * 2              # (append, attention) per layer
        t.gpu.device_status()

    multi_step([k, k, k])                                    # the second sequence crosses a page boundary (13 -> 13+k)
    multi_step([k, 1, max(1, k // 2)])                       # ragged
    for _ in range(3):
        multi_step([k, k, k])
    # two of the k tokens of the first sequence are rejected: roll back, then decode on as usual
    if k > 2:
        new_len = t.gpu.seq_len(seqs[0]) - 2
        t.gpu.truncate(seqs[0], new_len); assert t.mgr.truncate(seqs[0], new_len) == O.OK
    t.step(seqs, [1, 1, 1], check_pool=True)


@pytest.mark.parametrize("shape", [
    # H, Hkv, D, dtype, prefill kernel
    (32, 8, 128, "bf16", "auto"),      # 8B head shape on tcgen05: 32 tokens per 128-row tile
    (32, 8, 128, "bf16", "mma_sync"),  # ... and on the mma.sync kernel: 16 tokens per 64-row tile
    (64, 8, 128, "fp16", "auto"),      # 70B head shape
    (64, 8, 128, "fp16", "mma_sync"),
    (8, 2, 64, "fp16", "auto"),        # tiny config (head_dim 64: mma.sync kernel)
    (16, 16, 128, "bf16", "auto"),     # MHA: 128 tokens per tile
    (16, 16, 128, "fp16", "mma_sync"),
    (16, 1, 128, "bf16", "auto"),      # 16 heads per kv head: 8 tokens per tile
    (16, 1, 64, "bf16", "auto"),       # ... at head_dim 64: 4 tokens per 64-row tile
])
def test_prefill_chunk_attention_every_token(shape):
    """Prefill chunks through tk_kv_append + tk_kv_decode_multi: a fresh prompt (the chunk is the whole
    context), a chunk on top of a long context (tiles split over the context and merged), short and
    single-token rows in the same step (they stay with the decode kernel), ragged page boundaries.  Both
    prefill kernels: tcgen05 with accumulators in tensor memory (head_dim 128) and mma.sync."""
    H, Hkv, D, dtype, pimpl = shape
    t = Twin(2, H, Hkv, D, 700, 6, 400, dtype=dtype, impl="mma", max_step_tokens=4096, seed=120, prefill_impl=pimpl)
    a, b, c, d = (t.seq_alloc() for _ in range(4))
    t.step([a, b], [3000, 45], decode=False)                       # a long context and a short one
    t.step([a, b, c, d], [333, 1, 777, 2], every_token=True, check_pool=True)
    items, ct, n_decode = t.gpu.step_prefill_plan()
    assert len(items) > 0 and n_decode > 0                         # both kernels had work
    t.step([a, b, c, d], [150, 150, 1, 129], every_token=True)
    t.step([d, c], [1021, 300], every_token=True, f32_out=True)   # FP32 results: the stated tolerance with no slack
    t.step([a, b, c, d], [1, 1, 1, 1], check_pool=True)           # plain decode goes on
    t.gpu.device_status()


@pytest.mark.parametrize("pimpl", ["auto", "mma_sync"])
def test_prefill_chunk_long_context_split_and_merge(pimpl):
    """A 40-token chunk on a 20000-token context at the 8B head shape: few tiles, so every tile is cut
    into split-KV chunks whose partial rows the last CTA merges; and a 2500-token fresh prompt beside it."""
    t = Twin(1, 32, 8, 128, 1600, 2, 1400, dtype="bf16", impl="mma", max_step_tokens=4096, seed=121, prefill_impl=pimpl)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a], [20000 - 4096 * 4], decode=False)
    for _ in range(4):
        t.step([a], [4096], decode=False)
    t.step([a, b], [40, 2500], every_token=True, f32_out=True)
    items, ct, _ = t.gpu.step_prefill_plan()
    assert ct[0] < 20040 and len(set(items[items[:, 0] == 0][:, 1].tolist())) > 1     # sequence a was split
    t.gpu.device_status()


def test_decode_multi_refusals():
    from titan_engine_b200 import KvError
    t = Twin(1, 32, 8, 128, 64, 2, 32, dtype="bf16", impl="mma", max_step_tokens=256, seed=92)
    a, b = t.seq_alloc(), t.seq_alloc()
    t.step([a, b], [40, 40])
    q = torch.zeros(6, 32, 128, device=t.dev, dtype=torch.bfloat16)
    t.gpu.step_begin([a, b], [33, 1]); assert t.mgr.reserve(a, 33) == O.OK and t.mgr.reserve(b, 1) == O.OK
    # 4 heads per kv head x 33 tokens is more than the decode kernel's 8 token groups: the prefill kernel takes it
    t.gpu.decode_multi(0, torch.zeros(34, 32, 128, device=t.dev, dtype=torch.bfloat16))
    assert len(t.gpu.step_prefill_plan()[0]) > 0
    t.gpu.step_begin([a, b], [2, 0]); assert t.mgr.reserve(a, 2) == O.OK
    with pytest.raises(KvError):                             # a sequence without a new token
        t.gpu.decode_multi(0, q[:2].contiguous())
    f = Twin(1, 64, 8, 128, 16, 1, 16, dtype="fp8", impl="mma", max_step_tokens=64, seed=93)
    s = f.seq_alloc()
    f.gpu.step_begin([s], [2])
    with pytest.raises(KvError):                             # FP8 pools are not served
        f.gpu.decode_multi(0, torch.zeros(2, 64, 128, device=f.dev, dtype=torch.bfloat16))


@pytest.mark.parametrize("case", [(1, 32, 8, "bf16"), (2, 64, 8, "fp16"), (3, 16, 16, "bf16")])
def test_prefill_chunks_random_steps(case):
    """Random prefill chunks (1 .. 700 tokens, so tiles that end anywhere in a 128-row tile, blocks that end anywhere in
    a page) on contexts that grow from step to step, sequences leaving and joining, one-token rows in the same
    steps: every token of every step against the oracle's per-token decode, FP32 results at the stated tolerance."""
    seed, H, Hkv, dtype = case
    t = Twin(1, H, Hkv, 128, 700, 4, 260, dtype=dtype, impl="mma", max_step_tokens=2200, seed=300 + seed)
    g = rng(400 + seed)
    live = [t.seq_alloc() for _ in range(3)]
    for it in range(7):
        if it == 3:
            t.seq_free(live.pop(1))
            live.append(t.seq_alloc())
        seqs = sorted(live)
        n_new = []
        for s in seqs:
            room = 260 * 16 - t.gpu.seq_len(s)
            n = int(g.integers(1, 701)) if g.random() < 0.75 else 1
            n_new.append(max(1, min(n, room - 1)))
        t.step(seqs, n_new, every_token=True, f32_out=(it % 2 == 0))
    t.gpu.device_status()


@pytest.mark.parametrize("seed", [1, 2])
def test_decode_multi_random_steps(seed):
    """Random token counts per sequence and step (1 .. 2*16/G + 1), small chunks so that the new tokens keep
    crossing page and chunk boundaries, sequences joining and leaving between steps."""
    H, Hkv, D, dt = 16, 4, 64, O.FP16
    t = Twin(1, H, Hkv, D, 200, 5, 40, dtype="fp16", impl="mma", max_step_tokens=512, seed=95 + seed, chunk_tokens=64)
    g = rng(200 + seed)
    live = [t.seq_alloc() for _ in range(3)]
    t.step(live, [int(x) for x in g.integers(1, 120, size=3)])
    for it in range(25):
        if it % 7 == 3 and len(live) > 1:
            gone = live.pop(int(g.integers(0, len(live))))
            t.seq_free(gone)
        if it % 5 == 4 and len(live) < 5:
            s = t.seq_alloc()
            t.step([s], [int(g.integers(1, 60))])
            live.append(s)
        seqs = sorted(live)
        n_new = [int(x) for x in g.integers(1, 2 * (16 // (H // Hkv)) + 2, size=len(seqs))]     # up to 3 token groups
        old = [t.gpu.seq_len(s) for s in seqs]
        if max(o + n for o, n in zip(old, n_new)) > 40 * 16:
            break
        t.gpu.step_begin(seqs, n_new)
        for s, n in zip(seqs, n_new):
            assert t.mgr.reserve(s, n) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
        table = t.mgr.table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seqs, n_new)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)])
        k16 = normal16(g, (len(tok_seq), Hkv, D), dt); v16 = normal16(g, (len(tok_seq), Hkv, D), dt)
        q16 = normal16(g, (len(tok_seq), H, D), dt)
        got = t.gpu.append_decode_multi(0, to_torch16(k16, dt, t.dev), to_torch16(v16, dt, t.dev),
                                        to_torch16(q16, dt, t.dev)).float().cpu().numpy()
        t.pools[0].append(table, tok_seq, tok_pos, k16, v16)
        want = t.pools[0].decode(table, tok_seq, tok_pos + 1, q16)
        assert_close(got, want, f"step {it}: {n_new} new tokens on lengths {old}", out_mantissa_bits=10)
        # reject a random tail of one sequence's new tokens
        j = int(g.integers(0, len(seqs)))
        keep = int(g.integers(1, n_new[j] + 1))
        new_len = old[j] + keep
        t.gpu.truncate(seqs[j], new_len); assert t.mgr.truncate(seqs[j], new_len) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
    t.gpu.device_status()


@pytest.mark.parametrize("heads,k", [((16, 16), 2), ((16, 16), 8), ((16, 16), 11), ((32, 8), 2), ((32, 8), 5)])
def test_decode_multi_mla_shape(heads, k):
    """Multi-token attention on the MLA cache shape (K rows 192, V rows / outputs 128): 8/G tokens per pass."""
    H, Hkv = heads
    D, Dv, dt = 192, 128, O.BF16
    t = Twin(1, H, Hkv, D, 200, 3, 60, dtype="bf16", impl="mma", max_step_tokens=1024, seed=96, Dv=Dv, chunk_tokens=256)
    seqs = [t.seq_alloc() for _ in range(3)]
    t.step(seqs, [500, 14, 250])
    g = rng(97)
    for n_new in ([k, k, k], [k, 1, max(1, k // 2)], [k, k, k], [k, k, k]):
        old = [t.gpu.seq_len(s) for s in seqs]
        t.gpu.step_begin(seqs, n_new)
        for s, n in zip(seqs, n_new):
            assert t.mgr.reserve(s, n) == O.OK
        assert t.gpu.digest() == t.mgr.digest()
        table = t.mgr.table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seqs, n_new)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)])
        k16 = normal16(g, (len(tok_seq), Hkv, D), dt); v16 = normal16(g, (len(tok_seq), Hkv, Dv), dt)
        q16 = normal16(g, (len(tok_seq), H, D), dt)
        t.gpu.append(0, to_torch16(k16, dt, t.dev), to_torch16(v16, dt, t.dev))
        t.pools[0].append(table, tok_seq, tok_pos, k16, v16)
        got = t.gpu.decode_multi(0, to_torch16(q16, dt, t.dev)).float().cpu().numpy()
        assert got.shape == (len(tok_seq), H, Dv)
        want = t.pools[0].decode(table, tok_seq, tok_pos + 1, q16)
        assert_close(got, want, f"MLA multi-token attention {n_new}", out_mantissa_bits=7)
    t.gpu.device_status()
    t.step(seqs, [1, 1, 1], check_pool=True)
