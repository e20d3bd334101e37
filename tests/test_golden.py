"""Pins the CPU oracle against golden vectors produced by the UNMODIFIED reference kernels
(src/compute/cuda/attention.cu, src/inference/kv_cache.cpp) run on a B200 by
tests/golden/make_golden.py.  Inputs are regenerated from the stored seeds."""
import os
import sys

import numpy as np

from oracle import tk_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import make_golden as G  # noqa: E402


def _load():
    path = os.path.join(GOLDEN, "reference_attention.npz")
    assert os.path.exists(path), "golden vectors missing"
    return np.load(path)


def test_golden_cases_are_the_generator_cases():
    d = _load()
    np.testing.assert_array_equal(d["cases"], np.array(G.CASES, dtype=np.int64))
    np.testing.assert_array_equal(d["rope_cases"], np.array(G.ROPE_CASES, dtype=np.float64))


def test_oracle_attention_matches_reference_golden():
    d = _load()
    for i, (seed, H, Hkv, D, n) in enumerate(G.CASES):
        q, k, v = G.inputs(seed, H, Hkv, D, n)
        got = O.attention_decode_f32(q, k, v, H, Hkv, D, n)
        want = d[f"out_{i}"]
        assert np.abs(want).max() > 0
        # same FP32 formulae; only the summation order differs (256-thread tree vs sequential)
        np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5, err_msg=f"case {i}")


def test_oracle_update_path_matches_reference_golden():
    d = _load()
    q, k, v = G.inputs(107, 8, 2, 64, 40)
    kk, vv = np.stack([k, v]), np.stack([v, k])
    L, S, Hkv, D = 2, 64, 2, 64
    kd = np.zeros((L, S, Hkv, D), dtype=np.float32); vd = np.zeros_like(kd)
    seq_len = 0
    for pos in range(40):
        for layer in range(L):
            seq_len = O.kv_update_f32(kd, vd, L, S, Hkv, D, layer, pos, kk[layer, pos], vv[layer, pos], seq_len)
    assert seq_len == int(d["update_seq_len"]) == 40
    got = O.attention_decode_f32(q, kd[1], vd[1], 8, 2, 64, seq_len)
    np.testing.assert_allclose(got, d["update_out"], rtol=2e-4, atol=2e-5)


def test_oracle_rope_matches_reference_golden():
    d = _load()
    for i, (seed, H, Hkv, D, pos, theta) in enumerate(G.ROPE_CASES):
        H, Hkv, D, pos = int(H), int(Hkv), int(D), int(pos)
        q, k = G.rope_inputs(int(seed), H, Hkv, D)
        oq, ok = O.rope_f32(q, k, H, Hkv, D, pos, float(theta), 1.0)
        atol = 2e-4 + 2e-6 * pos          # one ulp of freq is ~6e-8*pos radians of angle
        np.testing.assert_allclose(oq, d[f"rope_q_{i}"], rtol=1e-4, atol=atol)
        np.testing.assert_allclose(ok, d[f"rope_k_{i}"], rtol=1e-4, atol=atol)


def test_oracle_rope_mla_matches_reference_golden():
    """apply_rope_mla of the reference (rope dims of 128 + 64 rows), run on a B200."""
    d = _load()
    np.testing.assert_array_equal(d["rope_mla_cases"], np.array(G.ROPE_MLA_CASES, dtype=np.float64))
    for i, (seed, H, Hkv, nope, rope, pos, theta) in enumerate(G.ROPE_MLA_CASES):
        H, Hkv, nope, rope, pos = int(H), int(Hkv), int(nope), int(rope), int(pos)
        q, k = G.rope_inputs(int(seed), H, Hkv, nope + rope)
        oq, ok = O.rope_mla_f32(q, k, H, Hkv, nope, rope, pos, float(theta))
        atol = 2e-4 + 2e-6 * pos
        np.testing.assert_allclose(oq, d[f"rope_mla_q_{i}"], rtol=1e-4, atol=atol)
        np.testing.assert_allclose(ok, d[f"rope_mla_k_{i}"], rtol=1e-4, atol=atol)
        np.testing.assert_array_equal(oq[:, :nope], q[:, :nope])          # the nope dims are untouched
        assert np.abs(oq[:, nope:] - q[:, nope:]).max() > (0.1 if pos else -1)


def test_oracle_mla_attention_matches_reference_golden():
    """attention_decode_mla (K rows of 192, V rows of 128) of the reference, run on a B200."""
    d = _load()
    np.testing.assert_array_equal(d["mla_cases"], np.array(G.MLA_CASES, dtype=np.int64))
    for i, (seed, H, Hkv, Dk, Dv, n) in enumerate(G.MLA_CASES):
        q, k, v = G.mla_inputs(seed, H, Hkv, Dk, Dv, n)
        got = O.attention_decode_mla_f32(q, k, v, H, Hkv, Dk, Dv, n)
        np.testing.assert_allclose(got, d[f"mla_out_{i}"], rtol=2e-4, atol=2e-5, err_msg=f"MLA case {i}")
