"""The reference's own kernels (src/compute/cuda/attention.cu, src/inference/kv_cache.cpp,
compiled unmodified into oracle/_ref/libtitan_ref.so) against the CPU oracle and against
this library, on the same seeded inputs.  The reference path is contiguous FP32, one
sequence, seq_len <= 12288 - head_dim."""
import numpy as np
import pytest
import torch

from helpers import assert_close, normal16, rng, to_torch16
from oracle import tk_oracle as O

pytestmark = pytest.mark.gpu

CASES = [  # H, Hkv, D, seq_len
    (8, 2, 64, 576),        # tiny config after 512 prefill + 64 decode steps
    (8, 2, 64, 1),
    (32, 8, 128, 1500),     # one sequence of the 8B-shape batch
    (32, 8, 128, 8193),     # longest context of that batch (+1 appended token)
    (64, 8, 128, 257),
]


@pytest.fixture(scope="module")
def ref():
    lib = O.ref_lib()
    assert lib is not None, "oracle/_ref/libtitan_ref.so missing: run `make -C oracle ref` where the reference is mounted"
    return lib


@pytest.mark.parametrize("case", CASES)
def test_oracle_matches_reference_kernel(ref, case):
    H, Hkv, D, n = case
    g = rng(1000 + n)
    q = g.standard_normal((H, D), dtype=np.float32)
    k = g.standard_normal((n, Hkv, D), dtype=np.float32)
    v = g.standard_normal((n, Hkv, D), dtype=np.float32)
    want = O.ref_attention_decode(q, k, v, H, Hkv, D, n)
    got = O.attention_decode_f32(q, k, v, H, Hkv, D, n)
    # same FP32 arithmetic, different summation order (the kernel reduces over 256 threads)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)


def test_reference_update_path_and_seq_len(ref):
    L, H, Hkv, D, n = 2, 8, 2, 64, 80
    g = rng(7)
    k = g.standard_normal((L, n, Hkv, D), dtype=np.float32)
    v = g.standard_normal((L, n, Hkv, D), dtype=np.float32)
    q = g.standard_normal((H, D), dtype=np.float32)
    for layer in range(L):
        out, seq_len = O.ref_update_and_decode(k, v, q, L, layer, H, Hkv, D, n, 128)
        assert seq_len == n
        np.testing.assert_allclose(out, O.attention_decode_f32(q, k[layer], v[layer], H, Hkv, D, n),
                                   rtol=2e-4, atol=2e-5)


@pytest.mark.parametrize("impl", ["simt", "mma"])
@pytest.mark.parametrize("case", CASES[:4])
def test_library_matches_reference_kernel(ref, impl, case):
    """Same values (exactly representable in the 16-bit storage type) through the reference's
    FP32 kernel and through the paged CUDA path."""
    from titan_engine_b200 import PagedKVCache
    H, Hkv, D, n = case
    dt, name = (O.FP16, "fp16") if D == 64 else (O.BF16, "bf16")
    g = rng(2000 + n)
    k16 = normal16(g, (n, Hkv, D), dt); v16 = normal16(g, (n, Hkv, D), dt); q16 = normal16(g, (1, H, D), dt)
    want = O.ref_attention_decode(O.to_f32(q16[0], dt), O.to_f32(k16, dt), O.to_f32(v16, dt), H, Hkv, D, n)
    n_pages = (n + 15) // 16
    c = PagedKVCache(1, H, Hkv, D, n_pages, 1, n_pages, dtype=name, decode_impl=impl, max_step_tokens=n)
    s = c.seq_alloc()
    c.step_begin([s], [n])
    dev = c.device
    c.append(0, to_torch16(k16, dt, dev), to_torch16(v16, dt, dev))
    got = c.decode(0, to_torch16(q16, dt, dev)).float().cpu().numpy()[0]
    c.device_status()
    assert_close(got, want, f"{impl} vs reference kernel {case}")


def test_rope_oracle_matches_reference_kernel(ref):
    H, Hkv, D = 32, 8, 128
    g = rng(9)
    q = g.standard_normal((H, D), dtype=np.float32); k = g.standard_normal((Hkv, D), dtype=np.float32)
    for pos in (0, 1, 77, 4096):
        rq, rk = O.ref_apply_rope(q, k, H, Hkv, D, pos, 500000.0, 1.0)
        oq, ok = O.rope_f32(q, k, H, Hkv, D, pos, 500000.0, 1.0)
        # powf differs in the last ulp between libm and the device; one ulp of freq is an angle
        # error of ~6e-8 * position radians, so the tolerance grows with the position
        atol = 2e-4 + 2e-6 * pos
        np.testing.assert_allclose(oq, rq, rtol=1e-4, atol=atol)
        np.testing.assert_allclose(ok, rk, rtol=1e-4, atol=atol)


def test_rope_mla_oracle_matches_reference_kernel(ref):
    H, Hkv, nope, rope = 16, 4, 128, 64
    g = rng(10)
    q = g.standard_normal((H, nope + rope), dtype=np.float32); k = g.standard_normal((Hkv, nope + rope), dtype=np.float32)
    for pos in (0, 3, 500, 8191):
        rq, rk = O.ref_apply_rope_mla(q, k, H, Hkv, nope, rope, pos, 10000.0)
        oq, ok = O.rope_mla_f32(q, k, H, Hkv, nope, rope, pos, 10000.0)
        atol = 2e-4 + 2e-6 * pos
        np.testing.assert_allclose(oq, rq, rtol=1e-4, atol=atol)
        np.testing.assert_allclose(ok, rk, rtol=1e-4, atol=atol)


@pytest.mark.parametrize("case", [(16, 16, 192, 128, 77), (16, 4, 192, 128, 1000)])
def test_mla_oracle_and_library_match_reference_kernel(ref, case):
    """attention_decode_mla of the reference vs the oracle (FP32) and vs the paged library (bf16)."""
    from titan_engine_b200 import PagedKVCache
    H, Hkv, Dk, Dv, n = case
    g = rng(3000 + n)
    k16 = normal16(g, (n, Hkv, Dk), O.BF16); v16 = normal16(g, (n, Hkv, Dv), O.BF16); q16 = normal16(g, (1, H, Dk), O.BF16)
    qf, kf, vf = O.to_f32(q16[0], O.BF16), O.to_f32(k16, O.BF16), O.to_f32(v16, O.BF16)
    want = O.ref_attention_decode_mla(qf, kf, vf, H, Hkv, Dk, Dv, n)
    np.testing.assert_allclose(O.attention_decode_mla_f32(qf, kf, vf, H, Hkv, Dk, Dv, n), want, rtol=2e-4, atol=2e-5)
    n_pages = (n + 15) // 16
    c = PagedKVCache(1, H, Hkv, Dk, n_pages, 1, n_pages, dtype="bf16", v_head_dim=Dv, max_step_tokens=n)
    s = c.seq_alloc()
    c.step_begin([s], [n])
    c.append(0, to_torch16(k16, O.BF16, c.device), to_torch16(v16, O.BF16, c.device))
    got = c.decode(0, to_torch16(q16, O.BF16, c.device)).float().cpu().numpy()[0]
    assert got.shape == (H, Dv)
    assert_close(got, want, f"MLA {case} vs reference kernel", out_mantissa_bits=7)
