"""Known-answer tests of the CPU oracle (no GPU).  The oracle is the checker for the CUDA
path, so it is checked first: closed-form attention cases, the reference's E4M3 decode rule
(src/compute/cuda/fp4.cu:173-185), conversions against an independent implementation."""
import numpy as np
import pytest
import torch

from helpers import DT, normal16, rng
from oracle import tk_oracle as O


def test_e4m3_decode_table():
    t = O.e4m3_decode_all()
    assert t[0x00] == 0.0 and t[0x80] == 0.0
    assert t[0x7F] == 0.0 and t[0xFF] == 0.0            # NaN codes decode to 0 (fp4.cu:174)
    assert t[0x7E] == 448.0 and t[0xFE] == -448.0
    assert t[0x01] == 2.0 ** -9 and t[0x07] == 7 * 2.0 ** -9   # subnormals exact
    assert t[0x08] == 2.0 ** -6 and t[0x38] == 1.0
    # independent decoder: torch's float8_e4m3fn, for every non-NaN code
    codes = torch.arange(256, dtype=torch.uint8)
    ref = codes.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    ok = ~np.isnan(ref)
    assert ok.sum() == 254
    np.testing.assert_array_equal(t[ok], ref[ok])


def test_e4m3_encode_identity_and_rounding():
    t = O.e4m3_decode_all()
    finite = [c for c in range(256) if (c & 0x7F) != 0x7F]
    enc = O.e4m3_encode(t[finite])
    for c, e in zip(finite, enc):
        assert e == c or (c == 0x80 and e in (0x00, 0x80)), (c, e)
    # ties go to even; saturation is to +-448, never NaN
    assert O.e4m3_encode(1.0625)[0] == 0x38            # halfway 1.0 / 1.125 -> even mantissa 0
    assert O.e4m3_encode(1.1875)[0] == 0x3A            # halfway 1.125 / 1.25 -> 1.25 (even)
    assert O.e4m3_encode(2.0 ** -10)[0] == 0x00        # halfway 0 / 2^-9 -> 0
    assert O.e4m3_encode(3 * 2.0 ** -10)[0] == 0x02    # halfway 1 / 2 subnormal steps -> 2
    assert O.e4m3_encode(1e9)[0] == 0x7E and O.e4m3_encode(-1e9)[0] == 0xFE
    assert O.e4m3_encode(464.0)[0] == 0x7E
    assert O.e4m3_encode(float("nan"))[0] == 0x7F


def test_e4m3_encode_matches_torch_in_range():
    x = rng(11).standard_normal(20000).astype(np.float32) * 60.0
    x = x[np.abs(x) <= 448.0]
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = O.e4m3_encode(x)
    # -0.0 vs +0.0 code may differ for tiny negatives that round to zero
    same = (got == ref) | (((got | ref) & 0x7F) == 0)
    assert same.all()


@pytest.mark.parametrize("name", ["fp16", "bf16"])
def test_16bit_conversions_match_torch(name):
    x = np.concatenate([rng(5).standard_normal(5000).astype(np.float32) * 3,
                        np.array([0.0, -0.0, 1.0, 65504.0, 1e-8, -1e-8, 3.3895e38], dtype=np.float32)])
    tdt = torch.float16 if name == "fp16" else torch.bfloat16
    ref = torch.from_numpy(x).to(tdt).view(torch.int16).numpy().view(np.uint16)
    got = O.f32_to_16(x, DT[name])
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(O.to_f32(got, DT[name]),
                                  torch.from_numpy(x).to(tdt).to(torch.float32).numpy())


def _contig(seed, H, Hkv, D, n):
    g = rng(seed)
    q = g.standard_normal((H, D), dtype=np.float32)
    k = g.standard_normal((n, Hkv, D), dtype=np.float32)
    v = g.standard_normal((n, Hkv, D), dtype=np.float32)
    return q, k, v


def test_attention_equal_keys_gives_mean_of_values():
    H, Hkv, D, n = 8, 2, 64, 37
    q, k, v = _contig(1, H, Hkv, D, n)
    k[:] = k[0]
    out = O.attention_decode_f32(q, k, v, H, Hkv, D, n)
    for h in range(H):
        np.testing.assert_allclose(out[h], v[:, h // (H // Hkv)].mean(0), rtol=1e-5, atol=1e-6)


def test_attention_single_token_and_normaliser():
    H, Hkv, D = 8, 2, 64
    q, k, v = _contig(2, H, Hkv, D, 1)
    out = O.attention_decode_f32(q, k, v, H, Hkv, D, 1)
    inv = np.float32(1.0) / (np.float32(1.0) + np.float32(1e-8))      # attention.cu:142
    for h in range(H):
        np.testing.assert_array_equal(out[h], (v[0, h // 4] * inv).astype(np.float32))


def test_attention_dominant_key_selects_its_value():
    H, Hkv, D, n = 4, 1, 64, 50
    q, k, v = _contig(3, H, Hkv, D, n)
    k[17, 0] = q[2] * 40.0
    out = O.attention_decode_f32(q, k, v, H, Hkv, D, n)
    np.testing.assert_allclose(out[2], v[17, 0], rtol=1e-4, atol=1e-4)


def test_attention_matches_float64_softmax():
    H, Hkv, D, n = 8, 2, 64, 300
    q, k, v = _contig(4, H, Hkv, D, n)
    out = O.attention_decode_f32(q, k, v, H, Hkv, D, n)
    for h in range(H):
        kv = h // (H // Hkv)
        s = (k[:, kv].astype(np.float64) @ q[h].astype(np.float64)) / np.sqrt(D)
        w = np.exp(s - s.max()); w /= w.sum()
        np.testing.assert_allclose(out[h], w @ v[:, kv].astype(np.float64), rtol=2e-5, atol=2e-6)


def test_kv_update_rules():
    L, S, Hkv, D = 2, 8, 2, 4
    kd = np.zeros((L, S, Hkv, D), dtype=np.float32); vd = np.zeros_like(kd)
    key = np.arange(Hkv * D, dtype=np.float32); val = key + 100
    n = O.kv_update_f32(kd, vd, L, S, Hkv, D, 1, 3, key, val, 0)
    assert n == 4                                               # kv_cache.cpp:148-150
    np.testing.assert_array_equal(kd[1, 3].ravel(), key)
    np.testing.assert_array_equal(vd[1, 3].ravel(), val)
    assert kd.sum() == key.sum()
    for bad_layer, bad_pos in ((2, 0), (0, -1), (0, 8)):        # silent no-op, kv_cache.cpp:124-126
        assert O.kv_update_f32(kd, vd, L, S, Hkv, D, bad_layer, bad_pos, key, val, 4) == 4
    assert kd.sum() == key.sum()
    assert O.kv_update_f32(kd, vd, L, S, Hkv, D, 0, 1, key, val, 4) == 4   # no shrink


@pytest.mark.parametrize("name", ["fp16", "bf16"])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 255, 256, 257])
def test_paged_equals_contiguous(name, n):
    """Paging is a pure re-indexing: gather + reference arithmetic == contiguous reference."""
    H, Hkv, D, ps = 8, 2, 64, 16
    dt = DT[name]
    g = rng(100 + n)
    k16 = normal16(g, (n, Hkv, D), dt); v16 = normal16(g, (n, Hkv, D), dt); q16 = normal16(g, (1, H, D), dt)
    n_pages = (n + ps - 1) // ps
    perm = g.permutation(n_pages + 3).astype(np.int32)
    table = np.full((2, n_pages + 1), -1, dtype=np.int32)
    table[1, :n_pages] = perm[:n_pages]
    pool = O.Pool(dt, n_pages + 3, H, Hkv, D, 2, n_pages + 1, ps)
    slots = pool.append(table, np.ones(n, np.int32), np.arange(n, dtype=np.int32), k16, v16)
    want_slots = table[1, np.arange(n) // ps].astype(np.int64) * ps + np.arange(n) % ps
    np.testing.assert_array_equal(slots, want_slots)
    out = pool.decode(table, [1], [n], q16)[0]
    ref = O.attention_decode_f32(O.to_f32(q16[0], dt), O.to_f32(k16, dt), O.to_f32(v16, dt), H, Hkv, D, n)
    np.testing.assert_array_equal(out, ref)


def test_split_kv_partials_combine_to_full():
    H, Hkv, D, ps, n = 8, 2, 64, 16, 333
    dt = O.FP16
    g = rng(7)
    k16 = normal16(g, (n, Hkv, D), dt); v16 = normal16(g, (n, Hkv, D), dt); q16 = normal16(g, (1, H, D), dt)
    n_pages = (n + ps - 1) // ps
    table = np.arange(n_pages, dtype=np.int32)[None, :].copy()
    pool = O.Pool(dt, n_pages, H, Hkv, D, 1, n_pages, ps)
    pool.append(table, np.zeros(n, np.int32), np.arange(n, dtype=np.int32), k16, v16)
    full = pool.decode(table, [0], [n], q16)[0]
    bounds = [0, 128, 256, n]
    parts = [pool.decode_partial(table, 0, n, a, b, q16[0]) for a, b in zip(bounds[:-1], bounds[1:])]
    for h in range(H):
        out = O.combine([p[0][h] for p in parts], [p[1][h] for p in parts], np.stack([p[2][h] for p in parts]))
        np.testing.assert_allclose(out, full[h], rtol=1e-5, atol=1e-6)


def test_fp8_seal_is_chunking_independent_and_decodes_within_quantisation_error():
    H, Hkv, D, ps, n = 8, 2, 128, 16, 70
    g = rng(9)
    k16 = normal16(g, (n, Hkv, D), O.BF16, 0.01); v16 = normal16(g, (n, Hkv, D), O.BF16, 0.01)
    q16 = normal16(g, (1, H, D), O.BF16)
    n_pages = 5
    table = np.array([[3, 0, 4, 1, 2]], dtype=np.int32)
    pos = np.arange(n, dtype=np.int32); seq = np.zeros(n, np.int32)
    a = O.Pool(O.FP8, n_pages, H, Hkv, D, 1, n_pages, ps)
    a.append(table, seq, pos, k16, v16)                          # one prefill call
    b = O.Pool(O.FP8, n_pages, H, Hkv, D, 1, n_pages, ps)
    for lo, hi in ((0, 5), (5, 16), (16, 17), (17, 49), (49, 70)):   # ragged chunks
        b.append(table, seq[lo:hi], pos[lo:hi], k16[lo:hi], v16[lo:hi])
    np.testing.assert_array_equal(a.pool, b.pool)
    np.testing.assert_array_equal(a.scales, b.scales)
    # sealed pages: 4 full pages; last 6 tokens stay 16-bit in the open page
    np.testing.assert_array_equal(a.open_pages[0, :, 0, :6], k16[64:70].transpose(1, 0, 2))
    kf = O.to_f32(k16, O.BF16)
    amax = np.abs(kf[:16, 0]).max()
    assert a.scales[3, 0, 0] == max(np.float32(amax) / np.float32(448.0), np.float32(1e-10))
    kd, _ = a.gather(table, 0, n, 0, 0, n)
    np.testing.assert_array_equal(kd[64:], kf[64:, 0])           # open page is exact
    assert np.abs(kd[:64] - kf[:64, 0]).max() <= amax * 2 ** -3  # e4m3: 3 mantissa bits, generous bound
    out8 = a.decode(table, [0], [n], q16)[0]
    ref = O.attention_decode_f32(O.to_f32(q16[0], O.BF16), kf, O.to_f32(v16, O.BF16), H, Hkv, D, n)
    vf = O.to_f32(v16, O.BF16)
    assert np.abs(out8 - ref).max() < 0.1 * np.abs(vf).max()     # outliers x20 widen the page scale
    # and it is exactly the reference arithmetic on the dequantised rows
    kd_all = np.stack([a.gather(table, 0, n, h, 0, n)[0] for h in range(Hkv)], axis=1)
    vd_all = np.stack([a.gather(table, 0, n, h, 0, n)[1] for h in range(Hkv)], axis=1)
    np.testing.assert_array_equal(
        out8, O.attention_decode_f32(O.to_f32(q16[0], O.BF16), kd_all, vd_all, H, Hkv, D, n))


def test_rope_pairs_rotate():
    H, Hkv, D = 4, 2, 8
    g = rng(12)
    q = g.standard_normal((H, D), dtype=np.float32); k = g.standard_normal((Hkv, D), dtype=np.float32)
    q2, k2 = O.rope_f32(q, k, H, Hkv, D, 0, 10000.0)
    np.testing.assert_array_equal(q2, q); np.testing.assert_array_equal(k2, k)   # position 0 = identity
    q3, k3 = O.rope_f32(q, k, H, Hkv, D, 5, 10000.0)
    np.testing.assert_allclose(np.hypot(q3[:, 0::2], q3[:, 1::2]), np.hypot(q[:, 0::2], q[:, 1::2]), rtol=1e-5)
    ang = 5.0 * 1.0                                                             # d=0: freq 1
    np.testing.assert_allclose(k3[0, 0], k[0, 0] * np.cos(ang) - k[0, 1] * np.sin(ang), rtol=1e-5)


def test_mla_shape_paged_equals_contiguous_and_float64():
    """K rows of 192 (scores, scale 1/sqrt(192)), V rows and output of 128."""
    H, Hkv, Dk, Dv, n, ps = 8, 2, 192, 128, 131, 16
    g = rng(13)
    k16 = normal16(g, (n, Hkv, Dk), O.BF16); v16 = normal16(g, (n, Hkv, Dv), O.BF16); q16 = normal16(g, (1, H, Dk), O.BF16)
    n_pages = (n + ps - 1) // ps
    table = g.permutation(n_pages).astype(np.int32)[None].copy()
    pool = O.Pool(O.BF16, n_pages, H, Hkv, Dk, 1, n_pages, ps, Dv=Dv)
    pool.append(table, np.zeros(n, np.int32), np.arange(n, dtype=np.int32), k16, v16)
    out = pool.decode(table, [0], [n], q16)[0]
    qf, kf, vf = O.to_f32(q16[0], O.BF16), O.to_f32(k16, O.BF16), O.to_f32(v16, O.BF16)
    np.testing.assert_array_equal(out, O.attention_decode_mla_f32(qf, kf, vf, H, Hkv, Dk, Dv, n))
    for h in range(H):
        s = (kf[:, h // 4].astype(np.float64) @ qf[h].astype(np.float64)) / np.sqrt(Dk)
        w = np.exp(s - s.max()); w /= w.sum()
        np.testing.assert_allclose(out[h], w @ vf[:, h // 4].astype(np.float64), rtol=2e-5, atol=2e-6)
