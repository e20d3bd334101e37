"""One rank of the long-context decode across GPUs (run under torchrun, NCCL).

A single sequence of N tokens (8B head shape, bf16, page 16) is split into contiguous page-aligned
ranges, one per rank.  Per layer each rank computes the merged (o, m, l) of its range, the ranks
all-gather the [1][H][D+2] partials and the LSE combine kernel produces the output.  Rank 0 also
holds the whole sequence and checks the distributed result against single-GPU attention, then
times `--steps` decode steps of `--layers` layers.  Prints one JSON line on rank 0."""
import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from titan_engine_b200 import PagedKVCache  # noqa: E402
from titan_engine_b200 import dist as D  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--hot-window", type=int, default=0,
                    help="most recent tokens kept in HBM; older pages live in pinned host memory (0 = all in HBM)")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer"],
                    help="nccl: all-gather + combine kernel; peer: one kernel storing into the peers' mailboxes over "
                         "NVLink, waiting for theirs and combining")
    ap.add_argument("--mixed", action="store_true",
                    help="odd ranks take the two-launch route (rows, then the exchange kernel) while even ranks let "
                         "the attention kernel carry the exchange: the routes must meet on the same flags")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    H, Hkv, Dh, n, L = 32, 8, 128, args.tokens, args.layers
    lo, hi = D.token_ranges(n, world)[rank]
    gen = torch.Generator(device=dev); gen.manual_seed(5)          # same stream of values on every rank
    q = torch.randn(1, H, Dh, device=dev, generator=gen).to(torch.bfloat16)
    n_pg = n // 16
    full = torch.randn(n_pg, Hkv, 2, 16, Dh, device=dev, generator=gen).to(torch.bfloat16)   # layer-shared data

    my_pages = (hi - lo) // 16
    cache = PagedKVCache(L, H, Hkv, Dh, max(my_pages, 1), 1, max(my_pages, 1), dtype="bf16",
                         hot_window=args.hot_window, cold_pages=max(my_pages, 1) if args.hot_window else 0,
                         separate_combine=args.mixed and rank % 2 == 1)
    s = cache.seq_alloc()
    cache.adopt(s, np.arange(my_pages, dtype=np.int32), hi - lo)
    for l in range(L):
        cache.layer_views(l)[0][:my_pages].copy_(full[lo // 16:hi // 16])
    if args.hot_window:
        cache.set_tail(s, n - hi)                      # tokens held by later ranks push this rank's pages out
    torch.cuda.synchronize()
    cache.step_begin([s], None)                        # evicts what lies outside the window
    ex = D.PeerExchange(H, Dh + 2) if args.exchange == "peer" else None
    dec = D.LongContextDecoder(cache.decode_partial, lambda st: D.combine_partials(st, torch.bfloat16), exchange=ex,
                               fused_fn=cache.decode_exchange)
    out = dec.decode(0, q)
    torch.cuda.synchronize()
    if ex is not None:
        ex.status()
        two_calls = D.LongContextDecoder(cache.decode_partial, None, exchange=ex).decode(0, q)   # partial, then exchange
        torch.cuda.synchronize()
        assert torch.equal(two_calls, out)
        # the all-gather route must give the same bytes: same rows, same arithmetic, same order
        ref = D.LongContextDecoder(cache.decode_partial, lambda st: D.combine_partials(st, torch.bfloat16)).decode(0, q)
        torch.cuda.synchronize()
        same_as_nccl = bool(torch.equal(ref, out))
    else:
        same_as_nccl = True

    ok, err = True, 0.0
    if rank == 0:
        whole = PagedKVCache(1, H, Hkv, Dh, n_pg, 1, n_pg, dtype="bf16")
        ws = whole.seq_alloc()
        whole.adopt(ws, np.arange(n_pg, dtype=np.int32), n)
        whole.layer_views(0)[0].copy_(full)
        whole.step_begin([ws], None)
        want = whole.decode(0, q).float()
        err = float((out.float() - want).abs().max())
        ok = bool(torch.allclose(out.float(), want, rtol=2e-3, atol=1e-2)) and float(want.abs().max()) > 0 and same_as_nccl
        whole.close()
    del full

    out_buf = torch.empty_like(out) if ex is not None else None

    def step():
        for l in range(L):
            if out_buf is not None:
                dec.decode(l, q, out_buf)
            else:
                dec.decode(l, q)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    if ex is not None:
        ex.status()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms_layer = float(t.item()) / args.steps / L
        kv_bytes = n * Hkv * Dh * 2 * 2
        print(json.dumps({"workload": f"one {n}-token sequence over {world} GPUs, 8B head shape, bf16",
                          "ok": ok, "exchange": args.exchange, "same_bytes_as_all_gather_route": same_as_nccl,
                          "max_abs_err_vs_single_gpu": err, "n_gpus": world, "layers": L,
                          "us_per_layer": ms_layer * 1e3, "aggregate_kv_gbs": kv_bytes / (ms_layer * 1e-3) / 1e9,
                          "exchange_bytes_per_rank_per_layer": H * (Dh + 2) * 4,
                          "hot_window": args.hot_window, "rank0_stats": {k: v for k, v in cache.stats().items()
                                                                          if k in ("pages_cold", "evictions", "prefetch_hits",
                                                                                   "prefetch_misses", "bytes_h2d", "bytes_d2h")}}),
              flush=True)
    if ex is not None:
        torch.cuda.synchronize(); dist.barrier()
        ex.close()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
