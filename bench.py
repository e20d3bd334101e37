#!/usr/bin/env python
"""Benchmark of the paged KV-cache hot path on B200.

Workload (default): the Llama-3.1-8B-shape batched decode — 32 query heads, 8 kv heads,
head_dim 128, 32 layers, bf16, 64 sequences with contexts uniform in [1024, 8192],
page size 16, physical pages shuffled across one pool.  One step = for every layer:
append 1 token per sequence, then paged GQA decode attention.  Synthetic data: N(0,1)
values from a fixed seed.

  python bench.py --gpus N --steps K --warmup W            (N>1: launched by torchrun)
  python bench.py --impl reference ...                      CPU oracle port on the host cores
  python bench.py --workload 70b-fp8 | mla-bf16             the FP8 70B shape / the MLA cache shape (extras)
  python bench.py --append-prefill T                        the append kernels alone (prefill step of T tokens)
  python bench.py --multi K                                 multi-token attention (K new tokens per sequence)

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (decode steps/s,
all GPUs); `e2e` goes through the host-buffer C-ABI entry point with the H2D/D2H copies
inside the timed region; `roofline` is the dominant kernel against the measured HBM peak;
`cpu_baseline` is the CPU oracle timed on this box's host cores (a reported number only).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "paged_decode_steps_per_s"
UNIT = "decode steps/s (1 step = 64 seqs x 32 layers: append 1 token + paged GQA attention)"
SHAPE = dict(H=32, Hkv=8, D=128, L=32, B=64, lo=1024, hi=8192, ps=16)
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode launch divided by its algorithmic
# bytes, from the ncu captures summarised under profiles/ (taken on a 4-layer / 2-layer cut of the
# same workload; the traffic is proportional to the tokens read, so it scales to a full launch)
TRAFFIC_OVER_ALGORITHMIC = {"8b-bf16": 1.0085, "70b-fp8": 1.0108, "mla-bf16": 1.0044}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"


def contexts(rank: int, B: int, lo: int, hi: int) -> np.ndarray:
    """Context lengths of one GPU's batch.  Every rank draws the SAME lengths (seed 2), so that the
    per-GPU work is fixed as N grows (weak scaling); page placement and K/V data differ per rank."""
    g = np.random.Generator(np.random.Philox(2))
    return g.integers(lo, hi + 1, size=B).astype(np.int64)


def algorithmic_bytes(ctx: np.ndarray, s=SHAPE):
    """Per layer per step: K+V of every live token read once per kv head (+ FP8 page scales) +
    appended rows + q read and out write + page-table entries; `kernel` is the share the decode
    kernel moves."""
    esize = s.get("esize", 2)
    dv = s.get("Dv", s["D"])
    kv = int(ctx.sum()) * s["Hkv"] * (s["D"] + dv) * esize
    if esize == 1:
        kv += int(((ctx + s["ps"] - 1) // s["ps"]).sum()) * s["Hkv"] * 2 * 4
    app = len(ctx) * s["Hkv"] * (s["D"] + dv) * 2
    q_b = len(ctx) * s["H"] * s["D"] * 2
    o_b = len(ctx) * s["H"] * dv * 2
    pt = int(((ctx + s["ps"] - 1) // s["ps"]).sum()) * 4
    return {"layer": kv + app + q_b + o_b + pt, "kernel": kv + q_b + pt}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons during the timed region (read-only queries)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# -------------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores (the reference has no CPU code for this path)
# -------------------------------------------------------------------------------------------------
class CpuLayer:
    """ONE layer of the workload in host memory, run through the CPU oracle (append 1 token
    per sequence + paged decode attention)."""

    def __init__(self, ctx: np.ndarray):
        from oracle import tk_oracle as O
        s = SHAPE
        B, ps = len(ctx), s["ps"]
        pages = (ctx + 1 + ps - 1) // ps
        n_pages, mpps = int(pages.sum()), int(pages.max())
        self.O, self.ctx = O, ctx
        self.pool = O.Pool(O.BF16, n_pages, s["H"], s["Hkv"], s["D"], B, mpps, ps)
        g = np.random.Generator(np.random.Philox(77))
        tile = O.f32_to_16(g.standard_normal(1 << 22, dtype=np.float32), O.BF16)
        flat = self.pool.pool.reshape(-1)
        for off in range(0, flat.size, tile.size):
            n = min(tile.size, flat.size - off)
            flat[off:off + n] = tile[:n]
        perm = g.permutation(n_pages).astype(np.int32)
        self.table = np.full((B, mpps), -1, dtype=np.int32)
        at = 0
        for b in range(B):
            self.table[b, :pages[b]] = perm[at:at + pages[b]]
            at += int(pages[b])
        self.k = O.f32_to_16(g.standard_normal((B, s["Hkv"], s["D"]), dtype=np.float32), O.BF16)
        self.v = O.f32_to_16(g.standard_normal((B, s["Hkv"], s["D"]), dtype=np.float32), O.BF16)
        self.q = O.f32_to_16(g.standard_normal((B, s["H"], s["D"]), dtype=np.float32), O.BF16)
        self.seqs = np.arange(B, dtype=np.int32)
        # all host cores this process may use, whatever OMP_NUM_THREADS a multi-process launcher exported
        # (torchrun sets it to 1; the other ranks of the reference arm have exited by now)
        try:
            cores = len(os.sched_getaffinity(0))
        except AttributeError:
            cores = os.cpu_count() or 1
        O.set_num_threads(cores)
        self.threads = O.num_threads()

    def run(self) -> float:
        t0 = time.perf_counter()
        self.pool.append(self.table, self.seqs, self.ctx.astype(np.int32), self.k, self.v)
        out = self.pool.decode(self.table, self.seqs, (self.ctx + 1).astype(np.int32), self.q)
        dt = time.perf_counter() - t0
        assert np.isfinite(out).all() and np.abs(out).max() > 0
        return dt


def cpu_layer_time(ctx: np.ndarray, min_seconds: float):
    """(seconds per layer, repetitions, threads) of the CPU oracle on one layer."""
    layer = CpuLayer(ctx)
    layer.run()                                                # warm
    times = []
    while sum(times) < min_seconds and len(times) < 50 or not times:
        times.append(layer.run())
    return float(np.mean(times)), len(times), layer.threads


def run_reference(args):
    """`--impl reference`: the reference has no CPU implementation of this path, so this arm
    times the CPU oracle port (same arithmetic as the reference's kernel, plus paging) with
    all host threads.  Each step is a bounded sample: ONE layer of the 64-sequence batch;
    a full step is 32 such layers."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ctx = contexts(0, SHAPE["B"], SHAPE["lo"], SHAPE["hi"])
    layer = CpuLayer(ctx)
    for _ in range(args.warmup):
        layer.run()
    times = [layer.run() for _ in range(args.steps)]
    threads = layer.threads
    t_layer = float(np.mean(times))
    value = 1.0 / (t_layer * SHAPE["L"])
    ab = algorithmic_bytes(ctx)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * SHAPE["L"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config_dict(ctx, 1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} x one layer of the 64-sequence batch "
                                   f"({int(ctx.sum())} live tokens), extrapolated x32 layers"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "hbm_gbs": ab["layer"] / t_layer / 1e9,
        "note": "the reference has no CPU code for this path; this is the CPU oracle port (OpenMP)",
    }
    print(json.dumps(line), flush=True)


def config_dict(ctx, n_gpus):
    d = _config_dict(ctx, n_gpus)
    if SHAPE.get("modified"):
        d["workload"] += f" [MODIFIED for an experiment: {len(ctx)} sequences, context U[{SHAPE['lo']},{SHAPE['hi']}]]"
    return d


def _config_dict(ctx, n_gpus):
    if "Dv" in SHAPE:
        return {"workload": "MLA-shape decode (K rows 192 = nope 128 + rope 64, V rows 128): 128 q heads / 128 kv heads, "
                            "bf16, 16 sequences/GPU at 4096 tokens, page 16, shuffled pool; resident layer subset",
                "sequences_per_gpu": int(len(ctx)), "live_tokens_per_gpu": int(ctx.sum()),
                "parallelism": f"by sequence x{n_gpus} (no data-path collective)",
                "l2": "inputs larger than L2: each layer reads its own ~5.4 GB of pool per step"}
    if SHAPE.get("esize", 2) == 1:
        return {"workload": "llama-3-70b-shape FP8 decode: 64 q heads / 8 kv heads, head_dim 128, FP8-E4M3 pool with "
                            "per-page per-head scales, 32 sequences/GPU at 32768 tokens, page 16, shuffled pool; "
                            "resident layer subset (80 layers = 172 GB do not fit one GPU)",
                "sequences_per_gpu": int(len(ctx)), "live_tokens_per_gpu": int(ctx.sum()),
                "parallelism": f"by sequence x{n_gpus} (no data-path collective)",
                "l2": "inputs larger than L2: each layer reads its own ~2.1 GB of pool per step"}
    return {"workload": "llama-3.1-8b-shape batched decode: 32 q heads / 8 kv heads, head_dim 128, "
                        "32 layers, bf16, 64 sequences/GPU, context U[1024,8192], page 16, shuffled pool",
            "sequences_per_gpu": int(len(ctx)), "live_tokens_per_gpu": int(ctx.sum()),
            "parallelism": f"by sequence x{n_gpus} (no data-path collective)",
            "l2": "inputs larger than L2: each layer reads its own ~1.2 GB of pool per step"}


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    from titan_engine_b200 import PagedKVCache

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the paged KV path has no CPU implementation "
                         "(use --impl reference for the CPU oracle arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    s = SHAPE
    B, ps, L = s["B"], s["ps"], args.layers
    ctx = contexts(rank, B, s["lo"], s["hi"])
    total_steps = 2 * (args.steps + args.warmup) + 8
    pages0 = (ctx + ps - 1) // ps
    pages_end = (ctx + total_steps + ps - 1) // ps
    num_pages = int(pages_end.sum()) + 64
    mpps = int(pages_end.max()) + 1
    fp8 = s.get("esize", 2) == 1
    dv = s.get("Dv", s["D"])
    cache = PagedKVCache(L, s["H"], s["Hkv"], s["D"], num_pages, B, mpps, dtype="fp8" if fp8 else "bf16",
                         max_step_tokens=B, decode_impl=args.decode_impl, chunk_tokens=args.chunk,
                         v_head_dim=dv if dv != s["D"] else 0)
    g = np.random.Generator(np.random.Philox(2 + 1000 * rank))
    perm = g.permutation(num_pages).astype(np.int32)
    seqs, at = [], 0
    for b in range(B):
        sid = cache.seq_alloc()
        cache.adopt(sid, perm[at:at + pages0[b]], int(ctx[b]))
        at += int(pages0[b])
        seqs.append(sid)
    gen = torch.Generator(device=dev); gen.manual_seed(1234 + rank)
    for l in range(L):                                          # N(0,1) K/V in every page
        pool, scales, open_pages = cache.layer_views(l)
        if not fp8:
            pool.normal_(generator=gen)
            continue
        # sealed pages as appending N(0,1) data would leave them: scale ~ amax/448, E4M3 codes of x/scale
        scales.uniform_(0.008, 0.010, generator=gen)
        for p0 in range(0, pool.shape[0], 8192):
            sl = slice(p0, min(p0 + 8192, pool.shape[0]))
            x = torch.randn(pool[sl].shape, device=dev, generator=gen)
            pool[sl] = (x / scales[sl][..., None, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        open_pages.normal_(generator=gen)
    k = torch.randn(B, s["Hkv"], s["D"], device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, s["Hkv"], dv, device=dev, generator=gen).to(torch.bfloat16)
    q = torch.randn(B, s["H"], s["D"], device=dev, generator=gen).to(torch.bfloat16)
    out = torch.empty(B, s["H"], dv, device=dev, dtype=torch.bfloat16)
    hk, hv, hq = (t.cpu().pin_memory() for t in (k, v, q))
    hout = torch.empty_like(out, device="cpu").pin_memory()
    ones = [1] * B
    lens = ctx.copy()

    def step_device():
        cache.step_begin(seqs, ones)
        for l in range(L):
            if args.separate:
                cache.append(l, k, v)
                cache.decode(l, q, out)
            elif args.rope:
                cache.rope_append_decode(l, k, v, q, 500000.0, 1.0, out)
            else:
                cache.append_decode(l, k, v, q, out)

    def step_host():
        cache.step_begin(seqs, ones)
        for l in range(L):
            cache.append_decode_host_async(l, hk, hv, hq, hout)
        cache.host_wait()
        torch.cuda.current_stream().synchronize()              # the step's result is on the host

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, profile=False):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if profile:
            cache.profile_enable(steps * L)
        barrier()
        n0 = cache.launch_count
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        each = cache.profile_read_each(steps * L) if profile else np.zeros(0, np.float32)
        prof = (float(each.sum()), int(each.size), each)
        if profile:
            cache.profile_enable(0)
        launches = cache.launch_count - n0
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches, prof

    for _ in range(args.warmup):
        step_device()
    lens_mid = lens + args.warmup
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, launches, (kern_ms, kern_n, kern_each) = timed(step_device, args.steps, profile=True)
    clocks = sampler.stop() if rank == 0 else None
    cache.device_status()
    ctx_timed = lens_mid + (args.steps + 1) / 2.0               # mean context over the timed steps

    for _ in range(args.warmup):
        step_host()
    ms_e2e, _, _ = timed(step_host, args.steps)
    cache.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak()
    ab = algorithmic_bytes(ctx_timed)
    ms_per_step = ms / args.steps
    value = world * args.steps / (ms / 1e3)
    kern_avg_ms = kern_ms / max(kern_n, 1)
    achieved = ab["kernel"] / (kern_avg_ms * 1e-3) / 1e9 if kern_n else None
    unit = UNIT
    if fp8 or "Dv" in s:
        unit = (f"decode steps/s (1 step = {B} seqs x {L} layers: append 1 token + paged "
                + ("GQA attention over the FP8 pool)" if fp8 else "MLA-shape attention)"))
    kernel = "decode_simt_kernel" if args.decode_impl == "simt" else ("decode_mma_mla_kernel" if "Dv" in s else "decode_mma_kernel")
    ratio = TRAFFIC_OVER_ALGORITHMIC[args.workload]
    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 storage, fp16 mma, f32 accumulate" if fp8 else "bf16",
        "data": "synthetic", "config": config_dict(ctx, world),
        "hbm_gbs_step": ab["layer"] * L / (ms_per_step * 1e-3) / 1e9,
        "hbm_frac_step": ab["layer"] * L / (ms_per_step * 1e-3) / 1e9 / peak,
        "layers": L, "chunk_tokens": cache.step_chunk_tokens, "work_items_per_layer": cache.step_num_work_items,
        "roofline": {"bound": "hbm", "kernel": kernel,
                     "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": (achieved / peak) if achieved else None,
                     "traffic": int(ab["kernel"] * ratio) if ratio else None,
                     "traffic_source": "ncu dram bytes of a reduced-layer capture (profiles/), scaled by tokens",
                     "algorithmic_bytes_per_launch": ab["kernel"], "avg_launch_ms": kern_avg_ms,
                     "launch_ms_p10_p50_p90": [float(x) for x in np.percentile(kern_each, [10, 50, 90])] if kern_n else None,
                     "launches_timed": kern_n, "peak_source": peak_src},
        "e2e": {"value": world * args.steps / (ms_e2e / 1e3), "unit": unit,
                "h2d_bytes_per_step": int(L * (hk.numel() + hv.numel() + hq.numel()) * 2),
                "d2h_bytes_per_step": int(L * hout.numel() * 2), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        t_layer, reps, threads = cpu_layer_time(ctx, args.cpu_seconds)
        line["cpu_baseline"] = {
            "value": 1.0 / (t_layer * SHAPE["L"]), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{reps} x one layer of the 64-sequence batch ({int(ctx.sum())} live tokens) "
                      f"through the CPU oracle (OpenMP), extrapolated x32 layers"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_append(args):
    """`--append-prefill T`: the append half of the path alone - one prefill step of B sequences x T tokens
    appended to every layer (page-table scatter; FP8 pools seal every completed page).  Prints one JSON line
    with the per-layer time and the read + write bandwidth; not the headline metric."""
    import torch
    from titan_engine_b200 import PagedKVCache
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s, T, L = SHAPE, args.append_prefill, args.layers
    B, Hkv, D = s["B"], s["Hkv"], s["D"]
    fp8 = s.get("esize", 2) == 1
    reps = args.warmup + args.steps
    pages_per_seq = (T * reps + 15) // 16 + 1
    cache = PagedKVCache(L, s["H"], Hkv, D, B * pages_per_seq + 64, B, pages_per_seq, dtype="fp8" if fp8 else "bf16",
                         max_step_tokens=B * T)
    seqs = [cache.seq_alloc() for _ in range(B)]
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    k = torch.randn(B * T, Hkv, D, device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(B * T, Hkv, D, device=dev, generator=gen).to(torch.bfloat16)
    times = []
    for _ in range(reps):
        cache.step_begin(seqs, [T] * B)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for l in range(L):
            cache.append(l, k, v)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / L)
    cache.device_status()
    ms = float(np.median(times[args.warmup:]))
    rd = B * T * Hkv * D * 2 * 2
    wr = B * T * Hkv * D * 2 * (1 if fp8 else 2) + (B * (T // 16) * Hkv * 2 * 4 if fp8 else 0)
    peak, peak_src = measured_peak()
    print(json.dumps({"metric": "prefill_append_gbs", "value": (rd + wr) / (ms * 1e-3) / 1e9, "unit": "GB/s read + written",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "us_per_layer": ms * 1e3,
                      "config": {"workload": f"prefill append: {B} sequences x {T} tokens, {Hkv} kv heads, head_dim {D}, "
                                             f"{'FP8-E4M3' if fp8 else 'bf16'} pool, {L} layers"},
                      "bytes_read_per_layer": rd, "bytes_written_per_layer": wr,
                      "roofline": {"bound": "hbm", "achieved": (rd + wr) / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                   "frac": (rd + wr) / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_src}}), flush=True)


def run_multi(args):
    """`--multi K`: every sequence of the workload appends K tokens per step and gets K causal attention
    outputs (tk_kv_append_decode_multi) - the verification step of a speculative decoder.  Prints one JSON
    line with the time per layer and per token-layer; not the headline metric."""
    import torch
    from titan_engine_b200 import PagedKVCache
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s, K, L = SHAPE, args.multi, args.layers
    B, ps = s["B"], s["ps"]
    ctx = contexts(0, B, s["lo"], s["hi"])
    reps = args.warmup + args.steps
    pages_end = (ctx + reps * K + ps - 1) // ps
    cache = PagedKVCache(L, s["H"], s["Hkv"], s["D"], int(pages_end.sum()) + 64, B, int(pages_end.max()) + 1, dtype="bf16",
                         max_step_tokens=B * K)
    seqs, at = [], 0
    for b in range(B):
        sid = cache.seq_alloc()
        n = int((ctx[b] + ps - 1) // ps)
        cache.adopt(sid, np.arange(at, at + n, dtype=np.int32), int(ctx[b]))
        at += n
        seqs.append(sid)
    gen = torch.Generator(device=dev); gen.manual_seed(11)
    for l in range(L):
        cache.layer_views(l)[0].normal_(generator=gen)
    k = torch.randn(B * K, s["Hkv"], s["D"], device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn(B * K, s["Hkv"], s["D"], device=dev, generator=gen).to(torch.bfloat16)
    q = torch.randn(B * K, s["H"], s["D"], device=dev, generator=gen).to(torch.bfloat16)
    out = torch.empty_like(q)
    times = []
    for _ in range(reps):
        cache.step_begin(seqs, [K] * B)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for l in range(L):
            if K == 1:
                cache.append(l, k, v)
                cache.decode(l, q, out)
            else:
                cache.append_decode_multi(l, k, v, q, out)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / L)
    cache.device_status()
    ms = float(np.median(times[args.warmup:]))
    print(json.dumps({"metric": "multi_token_decode_us_per_layer", "value": ms * 1e3, "unit": "us per layer (append + attention)",
                      "higher_is_better": False, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "tokens_per_sequence": K, "us_per_token_layer": ms * 1e3 / K,
                      "config": {"workload": f"{B} sequences, context U[{s['lo']},{s['hi']}], {s['H']} q / {s['Hkv']} kv heads, "
                                             f"head_dim {s['D']}, bf16, {L} layers, {K} new tokens per sequence and step"}}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="8b-bf16", choices=["8b-bf16", "70b-fp8", "mla-bf16"],
                    help="8b-bf16: the headline batched decode; 70b-fp8: 64 q / 8 kv heads, 32 sequences at 32768 "
                         "tokens, FP8-E4M3 pool, a resident subset of the 80 layers; mla-bf16: K rows 192 / V rows "
                         "128, 128 kv heads, 16 sequences at 4096 tokens (extras, not the headline)")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--decode-impl", default="auto", choices=["auto", "simt", "mma"])
    ap.add_argument("--chunk", type=int, default=0, help="split-KV chunk tokens (0 = library default)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--rope", action="store_true", help="also fuse RoPE of q and the new K rows into each layer's call")
    ap.add_argument("--ctx-range", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="experiment: context lengths uniform in [LO, HI] instead of the workload's (reported in config)")
    ap.add_argument("--seqs", type=int, default=0, help="experiment: sequences per GPU instead of the workload's")
    ap.add_argument("--append-prefill", type=int, default=0, metavar="T",
                    help="measure the append kernels alone: one prefill step of T tokens per sequence and layer")
    ap.add_argument("--multi", type=int, default=0, metavar="K",
                    help="measure multi-token attention: K new tokens per sequence and step (1 = plain decode, separate launches)")
    ap.add_argument("--separate", action="store_true", help="call append and decode separately (two entry points)")
    args = ap.parse_args()
    if args.workload == "70b-fp8":
        SHAPE.update(H=64, Hkv=8, D=128, L=16, B=32, lo=32768, hi=32768, esize=1)
        args.no_cpu = True
    if args.workload == "mla-bf16":
        SHAPE.update(H=128, Hkv=128, D=192, Dv=128, L=8, B=16, lo=4096, hi=4096)
        args.no_cpu = True
    if args.ctx_range:
        SHAPE.update(lo=args.ctx_range[0], hi=args.ctx_range[1], modified=True)
    if args.seqs:
        SHAPE.update(B=args.seqs, modified=True)
    args.layers = args.layers or SHAPE["L"]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.append_prefill > 0:
        run_append(args)
    elif args.multi > 0:
        run_multi(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
