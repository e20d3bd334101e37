"""The N>1 host logic on CPU: two gloo ranks.  Each rank holds half of one long sequence,
computes the (o, m, l) partial of its range with the CPU oracle, the ranks exchange partials with
one all-gather (titan_engine_b200.dist.LongContextDecoder), and the merged result must equal
single-rank attention.  Also the sharding helpers and the max-over-ranks timing reduction."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import normal16, rng
from oracle import tk_oracle as O
from titan_engine_b200 import dist as D


def test_sharding_helpers():
    assert [len(D.shard_sequences(64, r, 8)) for r in range(8)] == [8] * 8
    assert [list(D.shard_sequences(10, r, 4)) for r in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    kv, qh = D.shard_kv_heads(8, 32, 3, 8)
    assert list(kv) == [3] and list(qh) == [12, 13, 14, 15]
    with pytest.raises(ValueError):
        D.shard_kv_heads(8, 32, 0, 3)
    r = D.token_ranges(131072, 8)
    assert r[0] == (0, 16384) and r[7] == (114688, 131072)
    assert D.token_ranges(100, 4) == [(0, 32), (32, 64), (64, 96), (96, 100)]
    assert D.token_ranges(20, 4) == [(0, 16), (16, 20), (20, 20), (20, 20)]
    # hot window 32768 of 131072: ranks 0-5 cold, 6-7 hot
    split = [D.hot_cold_split(x, 131072, 32768) for x in r]
    assert [c for c, _ in split] == [16384] * 6 + [0, 0]
    assert [h for _, h in split] == [0] * 6 + [16384, 16384]
    assert D.hot_cold_split((0, 100), 100, 0) == (0, 100)
    assert D.hot_cold_split((0, 100), 100, 40) == (48, 52)          # pages 0-2 end below token 60


def _worker(rank, world, port, n, H, Hkv, Dh, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = rng(77)                                    # same seed on every rank: same global data
        k = normal16(g, (n, Hkv, Dh), O.BF16); v = normal16(g, (n, Hkv, Dh), O.BF16)
        q = normal16(g, (1, H, Dh), O.BF16)
        lo, hi = D.token_ranges(n, world)[rank]
        n_pg = max((hi - lo + 15) // 16, 1)
        pool = O.Pool(O.BF16, n_pg, H, Hkv, Dh, 1, n_pg)
        table = np.arange(n_pg, dtype=np.int32)[None]
        pool.append(table, np.zeros(hi - lo, np.int32), np.arange(hi - lo, dtype=np.int32), k[lo:hi], v[lo:hi])

        def partial_fn(layer, q_bits):
            m, l, o = pool.decode_partial(table, 0, hi - lo, 0, hi - lo, q_bits[0])
            return torch.from_numpy(np.concatenate([o, m[:, None], l[:, None]], axis=1)[None].astype(np.float32))

        def combine_fn(stacked):
            s = stacked.numpy()                        # [world, 1, H, D+2]
            out = np.stack([O.combine(s[:, 0, h, Dh], s[:, 0, h, Dh + 1], s[:, 0, h, :Dh]) for h in range(H)])
            return torch.from_numpy(out[None])

        dec = D.LongContextDecoder(partial_fn, combine_fn)
        out = dec.decode(0, q).numpy()[0]
        # timing reduction used by the benchmark: max over ranks
        t = torch.tensor([10.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            ret["out"], ret["tmax"] = out, float(t.item())
    finally:
        dist.destroy_process_group()


def test_two_rank_lse_combine_matches_single_rank():
    world, n, H, Hkv, Dh = 2, 333, 8, 2, 64
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as man:
        ret = man.dict()
        mp.spawn(_worker, args=(world, port, n, H, Hkv, Dh, ret), nprocs=world, join=True)
        out, tmax = np.asarray(ret["out"]), ret["tmax"]
    g = rng(77)
    k = normal16(g, (n, Hkv, Dh), O.BF16); v = normal16(g, (n, Hkv, Dh), O.BF16); q = normal16(g, (1, H, Dh), O.BF16)
    want = O.attention_decode_f32(O.to_f32(q[0], O.BF16), O.to_f32(k, O.BF16), O.to_f32(v, O.BF16), H, Hkv, Dh, n)
    np.testing.assert_allclose(out, want, rtol=2e-5, atol=2e-6)
    assert tmax == 11.0
