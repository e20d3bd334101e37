"""Generates tests/golden/reference_attention.npz by running the UNMODIFIED reference
kernels (oracle/_ref/libtitan_ref.so = the reference's src/compute/cuda/attention.cu and
src/inference/kv_cache.cpp, built by `make -C oracle ref`) on a GPU.

Run on a machine with a B200:   python tests/golden/make_golden.py [out_dir]
Inputs are regenerated from the seeds stored in the file, so only seeds, shapes and the
reference outputs are committed."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import tk_oracle as O  # noqa: E402

CASES = [  # seed, H, Hkv, D, seq_len
    (101, 8, 2, 64, 1), (102, 8, 2, 64, 17), (103, 8, 2, 64, 576),
    (104, 32, 8, 128, 300), (105, 32, 8, 128, 2049), (106, 64, 8, 128, 129),
]
MLA_CASES = [  # seed, H, Hkv, k_head_dim, v_head_dim, seq_len
    (301, 16, 16, 192, 128, 77), (302, 16, 4, 192, 128, 513),
]
ROPE_MLA_CASES = [(401, 16, 16, 128, 64, 0, 10000.0), (402, 16, 4, 128, 64, 4321, 10000.0)]   # seed, H, Hkv, nope, rope, pos, theta
ROPE_CASES = [(201, 32, 8, 128, 0, 500000.0), (202, 32, 8, 128, 1234, 500000.0), (203, 8, 2, 64, 77, 10000.0)]


def inputs(seed, H, Hkv, D, n):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.standard_normal((H, D), dtype=np.float32), g.standard_normal((n, Hkv, D), dtype=np.float32),
            g.standard_normal((n, Hkv, D), dtype=np.float32))


def mla_inputs(seed, H, Hkv, Dk, Dv, n):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.standard_normal((H, Dk), dtype=np.float32), g.standard_normal((n, Hkv, Dk), dtype=np.float32),
            g.standard_normal((n, Hkv, Dv), dtype=np.float32))


def rope_inputs(seed, H, Hkv, D):
    g = np.random.Generator(np.random.Philox(seed))
    return g.standard_normal((H, D), dtype=np.float32), g.standard_normal((Hkv, D), dtype=np.float32)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    data = {"cases": np.array(CASES, dtype=np.int64), "rope_cases": np.array(ROPE_CASES, dtype=np.float64)}
    for i, (seed, H, Hkv, D, n) in enumerate(CASES):
        q, k, v = inputs(seed, H, Hkv, D, n)
        data[f"out_{i}"] = O.ref_attention_decode(q, k, v, H, Hkv, D, n)
    # KVCache::update + attention_decode through the reference's own cache object
    q, k, v = inputs(107, 8, 2, 64, 40)
    kk = np.stack([k, v]); vv = np.stack([v, k])          # two layers with different content
    out, seq_len = O.ref_update_and_decode(kk, vv, q, 2, 1, 8, 2, 64, 40, 64)
    data["update_out"], data["update_seq_len"] = out, np.int64(seq_len)
    data["mla_cases"] = np.array(MLA_CASES, dtype=np.int64)
    for i, (seed, H, Hkv, Dk, Dv, n) in enumerate(MLA_CASES):
        q, k, v = mla_inputs(seed, H, Hkv, Dk, Dv, n)
        data[f"mla_out_{i}"] = O.ref_attention_decode_mla(q, k, v, H, Hkv, Dk, Dv, n)
    for i, (seed, H, Hkv, D, pos, theta) in enumerate(ROPE_CASES):
        q, k = rope_inputs(seed, H, Hkv, D)
        rq, rk = O.ref_apply_rope(q, k, H, Hkv, D, pos, theta, 1.0)
        data[f"rope_q_{i}"], data[f"rope_k_{i}"] = rq, rk
    data["rope_mla_cases"] = np.array(ROPE_MLA_CASES, dtype=np.float64)
    for i, (seed, H, Hkv, nope, rope, pos, theta) in enumerate(ROPE_MLA_CASES):
        q, k = rope_inputs(seed, H, Hkv, nope + rope)
        rq, rk = O.ref_apply_rope_mla(q, k, H, Hkv, nope, rope, pos, theta)
        data[f"rope_mla_q_{i}"], data[f"rope_mla_k_{i}"] = rq, rk
    path = os.path.join(out_dir, "reference_attention.npz")
    np.savez_compressed(path, **data)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
