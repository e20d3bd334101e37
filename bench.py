#!/usr/bin/env python
"""Benchmark of the paged KV-cache hot path on B200.

Headline workload: the Llama-3.1-8B-shape batched decode — 32 query heads, 8 kv heads,
head_dim 128, 32 layers, bf16, 64 sequences with contexts uniform in [1024, 8192],
page size 16, physical pages shuffled across one pool.  One step = for every layer:
append 1 token per sequence, then paged GQA decode attention.  Synthetic data: N(0,1)
values from a fixed seed.

  python bench.py --gpus N --steps K --warmup W            (N>1: launched by torchrun)
  python bench.py --impl reference ...                      CPU oracle port on the host cores
  python bench.py --workload 70b-fp8 | mla-bf16             one of the other decode workloads as the line
  python bench.py --append-prefill T                        the append kernels alone (prefill step of T tokens)
  python bench.py --multi K                                 attention for K new tokens per sequence (K >= 256: prefill chunks)

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (decode steps/s,
all GPUs); `e2e` goes through the host-buffer C-ABI entry point with the H2D/D2H copies
inside the timed region; `roofline` is the dominant kernel against the measured HBM peak;
`cpu_baseline` is the CPU oracle timed on this box's host cores (a reported number only).
After the headline legs the same run measures the other configurations as short sub-records
under `workloads`: the FP8 70B shape, the MLA shape, continuous-batching churn through the
scheduler and — on 2 or more GPUs — one 131072-token sequence split over the ranks.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")      # the path has no bandwidth-bound collective; plain NVLink transports

METRIC = "paged_decode_steps_per_s"
WORKLOADS = {
    "8b-bf16": dict(H=32, Hkv=8, D=128, L=32, B=64, lo=1024, hi=8192, ps=16, esize=2,
                    profile="decode_mma_kernel_8b_shape_bf16.md"),
    "70b-fp8": dict(H=64, Hkv=8, D=128, L=16, B=32, lo=32768, hi=32768, ps=16, esize=1,
                    profile="decode_mma_kernel_70b_shape_fp8.md"),
    "mla-bf16": dict(H=128, Hkv=128, D=192, Dv=128, L=8, B=16, lo=4096, hi=4096, ps=16, esize=2,
                     profile="decode_mma_mla_kernel_mla_shape_bf16.md"),
}
FALLBACK_HBM_GBS = 6650.0


def unit_of(s, L):
    kind = ("GQA attention over the FP8 pool" if s["esize"] == 1 else
            "MLA-shape attention" if "Dv" in s else "GQA attention")
    return f"decode steps/s (1 step = {s['B']} seqs x {L} layers: append 1 token + paged {kind})"


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"


def traffic_ratio(s):
    """dram bytes (read + written) of one decode launch over its algorithmic bytes, as the ncu capture
    summarised under profiles/ measured it on a reduced-layer cut of the same workload (traffic grows in
    proportion to the tokens read, so the ratio carries over to a full launch).  None if the summary is gone."""
    try:
        text = open(os.path.join(ROOT, "profiles", s["profile"])).read()
        m = re.search(r"traffic / algorithmic = ([0-9.]+)", text)
        return float(m.group(1)) if m else None
    except OSError:
        return None


def contexts(B: int, lo: int, hi: int) -> np.ndarray:
    """Context lengths of one GPU's batch.  Every rank draws the SAME lengths (seed 2), so that the
    per-GPU work is fixed as N grows (weak scaling); page placement and K/V data differ per rank."""
    g = np.random.Generator(np.random.Philox(2))
    return g.integers(lo, hi + 1, size=B).astype(np.int64)


def algorithmic_bytes(ctx: np.ndarray, s):
    """Per layer per step: K+V of every live token read once per kv head (+ FP8 page scales) +
    appended rows + q read and out write + page-table entries; `kernel` is the share the decode
    kernel moves."""
    esize = s["esize"]
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
        return self

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
    """ONE layer of the headline workload in host memory, run through the CPU oracle (append 1 token
    per sequence + paged decode attention)."""

    def __init__(self, ctx: np.ndarray, s):
        from oracle import tk_oracle as O
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


def cpu_layer_time(ctx: np.ndarray, s, min_seconds: float):
    """(seconds per layer, repetitions, threads) of the CPU oracle on one layer."""
    layer = CpuLayer(ctx, s)
    layer.run()                                                # warm
    times = []
    while sum(times) < min_seconds and len(times) < 50 or not times:
        times.append(layer.run())
    return float(np.mean(times)), len(times), layer.threads


def run_reference(args):
    """`--impl reference`: the reference has no CPU implementation of this path, so this arm times the
    CPU oracle port (same arithmetic as the reference's kernel, plus paging) with all host threads.
    A step is what it is in the other arm - all 32 layers of the 64-sequence batch (the one layer held in
    host memory is run 32 times: 1.2 GB per pass, nothing stays in cache) - so `steps` x `ms_per_step` is
    the time this arm really ran; the number of steps is capped so that the run ends within about a minute."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = WORKLOADS["8b-bf16"]
    ctx = contexts(s["B"], s["lo"], s["hi"])
    layer = CpuLayer(ctx, s)
    t_probe = layer.run()                                      # also warms the pages
    step_s = t_probe * s["L"]
    steps = max(1, min(args.steps, int(60.0 / max(step_s, 1e-3))))
    warmup = 1 if args.warmup > 0 and step_s < 20.0 else 0
    for _ in range(warmup):
        for _ in range(s["L"]):
            layer.run()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        for _ in range(s["L"]):
            layer.run()
        times.append(time.perf_counter() - t0)
    t_step = float(np.mean(times))
    value = 1.0 / t_step
    unit = unit_of(s, s["L"])
    ab = algorithmic_bytes(ctx, s)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config_dict("8b-bf16", s, ctx, args.gpus),
        "cpu_baseline": {"value": value, "unit": unit, "cores": layer.threads, "kind": "port",
                         "sample": f"{steps} step(s) of 32 layers of the 64-sequence batch ({int(ctx.sum())} live "
                                   f"tokens per layer) through the CPU oracle (OpenMP); steps capped to about a minute"},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "hbm_gbs": ab["layer"] * s["L"] / t_step / 1e9,
        "host_note": "the host arm runs ONE GPU's share (one 64-sequence batch) whatever --gpus says",
        "note": "the reference has no CPU code for this path; this is the CPU oracle port (OpenMP)",
    }
    print(json.dumps(line), flush=True)


def config_dict(name, s, ctx, n_gpus):
    par = f"by sequence x{n_gpus} (no data-path collective)"
    base = {"sequences_per_gpu": int(len(ctx)), "live_tokens_per_gpu": int(ctx.sum()), "parallelism": par}
    if name == "mla-bf16":
        base.update(workload="MLA-shape decode (K rows 192 = nope 128 + rope 64, V rows 128): 128 q heads / 128 kv heads, "
                             "bf16, 16 sequences/GPU at 4096 tokens, page 16, shuffled pool; resident layer subset",
                    l2="inputs larger than L2: each layer reads its own ~5.4 GB of pool per step")
    elif name == "70b-fp8":
        base.update(workload="llama-3-70b-shape FP8 decode: 64 q heads / 8 kv heads, head_dim 128, FP8-E4M3 pool with "
                             "per-page per-head scales, 32 sequences/GPU at 32768 tokens, page 16, shuffled pool; "
                             "resident layer subset (80 layers = 172 GB do not fit one GPU)",
                    l2="inputs larger than L2: each layer reads its own ~2.1 GB of pool per step")
    else:
        base.update(workload="llama-3.1-8b-shape batched decode: 32 q heads / 8 kv heads, head_dim 128, "
                             "32 layers, bf16, 64 sequences/GPU, context U[1024,8192], page 16, shuffled pool",
                    l2="inputs larger than L2: each layer reads its own ~1.2 GB of pool per step")
    if s.get("modified"):
        base["workload"] += f" [MODIFIED: {len(ctx)} sequences per GPU]"
    return base


# -------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------
class Env:
    """Process-wide state of a GPU run: rank, device, barrier and max-over-ranks timing."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the paged KV path has no CPU implementation "
                             "(use --impl reference for the CPU oracle arm)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_ms(self, ms: float) -> float:
        if self.world == 1:
            return ms
        t = self.torch.tensor([ms], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        t = self.torch.tensor([1 if ok else 0], device=self.dev, dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def release(self):
        gc.collect()
        self.torch.cuda.empty_cache()

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def decode_workload(env: Env, name: str, s, L: int, steps: int, warmup: int, *, e2e: bool, clocks: bool,
                    decode_impl="auto", chunk=0, rope=False):
    """One decode workload (append 1 token + attention for every sequence and layer): device-resident
    timing with one CUDA-event bracket per decode launch, optionally the host-buffer leg.  Returns the
    record the JSON line (or a `workloads` sub-record) is made from."""
    torch = env.torch
    from titan_engine_b200 import PagedKVCache
    dev, rank, world = env.dev, env.rank, env.world
    B, ps = s["B"], s["ps"]
    ctx = contexts(B, s["lo"], s["hi"])
    total_steps = 3 * steps + 2 * warmup + 8
    pages0 = (ctx + ps - 1) // ps
    pages_end = (ctx + total_steps + ps - 1) // ps
    num_pages = int(pages_end.sum()) + 64
    mpps = int(pages_end.max()) + 1
    fp8 = s["esize"] == 1
    dv = s.get("Dv", s["D"])
    cache = PagedKVCache(L, s["H"], s["Hkv"], s["D"], num_pages, B, mpps, dtype="fp8" if fp8 else "bf16",
                         max_step_tokens=B, decode_impl=decode_impl, chunk_tokens=chunk,
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

    def step_device():
        cache.step_begin(seqs, ones)
        for l in range(L):
            if rope:
                cache.rope_append_decode(l, k, v, q, 500000.0, 1.0, out)
            else:
                cache.append_decode(l, k, v, q, out)

    def step_host():
        cache.step_begin(seqs, ones)
        for l in range(L):
            cache.append_decode_host_async(l, hk, hv, hq, hout)
        cache.host_wait()
        torch.cuda.current_stream().synchronize()              # the step's result is on the host

    def timed(fn, n, profile=False):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if profile:
            cache.profile_enable(n * L)
        env.barrier()
        n0 = cache.launch_count
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        env.barrier()
        ms = e0.elapsed_time(e1)
        each = cache.profile_read_each(n * L) if profile else np.zeros(0, np.float32)
        if profile:
            cache.profile_enable(0)
        return env.max_ms(ms), cache.launch_count - n0, each

    for _ in range(warmup):
        step_device()
    sampler = ClockSampler(env.local).start() if (clocks and rank == 0) else None
    # the timed region: the steps as a caller runs them (a layer's launch may start while the previous layer's
    # drains: programmatic dependent launch)
    ms, launches, _ = timed(step_device, steps)
    # the same steps once more with one CUDA-event bracket per decode launch, for the kernel's own duration
    # (a bracket between two launches keeps them from overlapping, so these steps run a little slower)
    ms_bracketed, _, kern_each = timed(step_device, steps, profile=True)
    clock_rec = sampler.stop() if sampler else None
    cache.device_status()
    ctx_timed = ctx + warmup + (steps + 1) / 2.0                # mean context over the timed steps
    ctx_bracketed = ctx_timed + steps                           # ... and over the bracketed ones
    rec = {"name": name, "ctx": ctx, "L": L, "ms": ms, "steps": steps, "warmup": warmup, "launches": int(launches),
           "kern_each": kern_each, "clocks": clock_rec, "ab": algorithmic_bytes(ctx_timed, s),
           "ab_bracketed": algorithmic_bytes(ctx_bracketed, s), "ms_bracketed": ms_bracketed,
           "chunk_tokens": cache.step_chunk_tokens, "work_items": cache.step_num_work_items, "fp8": fp8,
           "kernel": "decode_simt_kernel" if decode_impl == "simt" else
                     ("decode_mma_mla_kernel" if "Dv" in s else "decode_mma_kernel")}
    if e2e:
        for _ in range(warmup):
            step_host()
        ms_e2e, _, _ = timed(step_host, steps)
        cache.device_status()
        rec.update(ms_e2e=ms_e2e, h2d=int(L * (hk.numel() + hv.numel() + hq.numel()) * 2), d2h=int(L * hout.numel() * 2))
    cache.close()
    del cache, k, v, q, out
    env.release()
    return rec


def roofline_of(rec, s):
    peak, peak_src = measured_peak()
    each = rec["kern_each"]
    n = int(each.size)
    avg_ms = float(each.sum()) / max(n, 1)
    ab = rec["ab_bracketed"]["kernel"]
    achieved = ab / (avg_ms * 1e-3) / 1e9 if n else None
    ratio = traffic_ratio(s)
    return {"bound": "hbm", "kernel": rec["kernel"], "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": (achieved / peak) if achieved else None,
            "traffic": int(ab * ratio) if ratio else None,
            "traffic_source": f"algorithmic bytes x the ncu dram-bytes ratio recorded in profiles/{s['profile']}"
                              " (reduced-layer capture of the same workload)",
            "algorithmic_bytes_per_launch": ab, "avg_launch_ms": avg_ms,
            "ms_per_step_while_bracketed": rec["ms_bracketed"] / rec["steps"],
            "timing": "one CUDA-event bracket per decode launch, in a second pass over the same number of steps right after "
                      "the timed region; a bracket between two launches keeps the later one from starting while the earlier "
                      "drains, so layers x avg_launch_ms is the bracketed pass's step time, not the timed region's",
            "launch_ms_p10_p50_p90": [float(x) for x in np.percentile(each, [10, 50, 90])] if n else None,
            "launches_timed": n, "peak_source": peak_src}


def sub_record(env, rec, s):
    """Short form of a decode workload for the `workloads` key."""
    peak, _ = measured_peak()
    ms_per_step = rec["ms"] / rec["steps"]
    return {"ok": True, "value": env.world * rec["steps"] / (rec["ms"] / 1e3), "unit": unit_of(s, rec["L"]),
            "ms_per_step": ms_per_step, "steps": rec["steps"], "warmup": rec["warmup"], "layers": rec["L"],
            "config": config_dict(rec["name"], s, rec["ctx"], env.world),
            "hbm_frac_step": rec["ab"]["layer"] * rec["L"] / (ms_per_step * 1e-3) / 1e9 / peak,
            "roofline": roofline_of(rec, s), "clocks": rec["clocks"], "gpu_launches": rec["launches"]}


def churn_workload(env: Env, steps: int, warmup: int, L: int = 8):
    """Continuous-batching churn (the 8B head shape in fp16) driven through the tk_sched_* scheduler:
    256 concurrent requests with context lengths lognormal (median 2048, sigma 1, cap 32768); every step 13
    requests finish and 13 new ones are admitted with prompts of 256..4096 tokens, appended in that step;
    every other request appends one token.  Per layer: tk_kv_append of the step's rows, then attention for
    EVERY appended token (tk_kv_decode_multi: the decode kernel for the one-token rows, the prefill kernel
    for the prompts).  A resident subset of the 32 layers."""
    torch = env.torch
    from titan_engine_b200 import PagedKVCache
    from titan_engine_b200.scheduler import BatchScheduler
    H, Hkv, D, ps, n_req, churn = 32, 8, 128, 16, 256, 13
    g = np.random.Generator(np.random.Philox(3 + 1000 * env.rank))
    g0 = np.random.Generator(np.random.Philox(3))                 # the same lengths on every rank
    lens = np.minimum(32768, np.maximum(1, np.round(np.exp(g0.normal(np.log(2048.0), 1.0, size=n_req))))).astype(np.int64)
    prompts = g0.integers(256, 4097, size=(steps + warmup + 2, churn))
    max_prefill = churn * 4096
    total_steps = steps + warmup + 2
    num_pages = int(((lens + ps - 1) // ps).sum()) + total_steps * (churn * 4096 // ps + n_req) + 1024
    mpps = (32768 + 4096 + total_steps + 64) // ps
    cache = PagedKVCache(L, H, Hkv, D, num_pages, n_req, mpps, dtype="fp16", max_step_tokens=max_prefill + n_req)
    sched = BatchScheduler(cache, max_batch_size=n_req, max_prefill_tokens=max_prefill)
    dev = env.dev
    gen = torch.Generator(device=dev); gen.manual_seed(33 + env.rank)
    cap_tok = max_prefill + n_req
    k = torch.randn(cap_tok, Hkv, D, device=dev, generator=gen).to(torch.float16)
    v = torch.randn(cap_tok, Hkv, D, device=dev, generator=gen).to(torch.float16)
    q = torch.randn(cap_tok, H, D, device=dev, generator=gen).to(torch.float16)
    out = torch.empty_like(q)
    for n in lens:
        sched.submit(int(n), 1 << 12)
    # set-up: prefill the 256 contexts through the scheduler (append only; attention is not needed to fill the pool)
    fill_steps = 0
    while True:
        rows = sched.next()
        nt = cache.step_num_tokens
        for l in range(L):
            cache.append(l, k[:nt], v[:nt])
        sched.commit([False] * len(rows))
        fill_steps += 1
        if all(r.n_new == 1 for r in rows) and len(rows) == n_req:
            break
        if fill_steps > 400:
            raise RuntimeError("churn set-up did not converge")
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(L)]
    t_append = t_attn = 0.0
    admitted_tokens = 0

    def step(i, timed):
        nonlocal t_append, t_attn, admitted_tokens
        rows = sched.next()                                    # retires last step's 13, admits the 13 queued, begins the step
        nt = cache.step_num_tokens
        for l in range(L):
            ev[l][0].record()
            cache.append(l, k[:nt], v[:nt])
            ev[l][1].record()
            cache.decode_multi(l, q[:nt], out[:nt])
            ev[l][2].record()
        decoding = [j for j, r in enumerate(rows) if r.n_new == 1]
        gone = set(g.choice(decoding, size=churn, replace=False).tolist())
        sched.commit([j in gone for j in range(len(rows))])
        for n in prompts[i]:
            sched.submit(int(n), 1 << 12)
        if timed:
            torch.cuda.synchronize()
            t_append += sum(ev[l][0].elapsed_time(ev[l][1]) for l in range(L))
            t_attn += sum(ev[l][1].elapsed_time(ev[l][2]) for l in range(L))
            admitted_tokens += nt - sum(1 for r in rows if r.n_new == 1)
        return len(rows), nt

    # the first warm-up step is plain decode (nothing has finished yet); from the second on, every step
    # retires 13 requests and admits 13 prompts
    for i in range(warmup):
        step(i, False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    n0 = cache.launch_count
    e0.record()
    rows_seen = tok_seen = 0
    for i in range(steps):
        r, nt = step(warmup + i, True)
        rows_seen += r; tok_seen += nt
    e1.record()
    env.barrier()
    ms = env.max_ms(e0.elapsed_time(e1))
    cache.device_status()
    st = sched.stats()
    live = int(sum(cache.seq_len(sid) for sid in range(n_req) if cache.seq_len(sid) > 0))
    rec = {"ok": True, "value": env.world * steps / (ms / 1e3),
           "unit": f"churn steps/s (1 step = {n_req} requests x {L} layers: retire {churn}, admit {churn} prompts of "
                   f"256..4096 tokens, append, attention for every appended token)",
           "ms_per_step": ms / steps, "steps": steps, "warmup": warmup, "layers": L,
           "config": {"workload": "continuous-batching churn, 8B head shape (32 q / 8 kv heads, head_dim 128), fp16, 256 "
                                  "requests/GPU, contexts lognormal (median 2048, sigma 1, cap 32768), 13 retire + 13 admit "
                                  "per step, page 16, pages freed and reallocated through the free list; resident layer subset",
                      "driver": "tk_sched_submit / tk_sched_next / tk_sched_commit", "parallelism": f"by sequence x{env.world}",
                      "live_tokens_per_gpu": live, "rows_per_step": rows_seen / steps, "tokens_appended_per_step": tok_seen / steps,
                      "prompt_tokens_admitted_per_step": admitted_tokens / steps},
           "attention": "every appended token (tk_kv_decode_multi)",
           "append_ms_per_layer": t_append / (steps * L), "attention_ms_per_layer": t_attn / (steps * L),
           "append_share": t_append / max(t_append + t_attn, 1e-9), "attention_share": t_attn / max(t_append + t_attn, 1e-9),
           "note": "the per-layer event brackets synchronise the host once per step (inside the timed region)",
           "scheduler": {k_: st[k_] for k_ in ("iterations", "preemptions", "completed_requests", "active_requests")},
           "gpu_launches": int(cache.launch_count - n0)}
    sched.close(); cache.close()
    del cache, k, v, q, out
    env.release()
    return rec


def long_context_workload(env: Env, steps: int, warmup: int, L: int = 4, n: int = 131072, hot_window: int = 32768):
    """One 131072-token sequence (8B head shape, bf16) split contiguously over the ranks.  Per layer every
    rank attends over its own tokens and the ranks exchange their merged (o, m, l) rows: inside the attention
    kernel over NVLink peer memory (tk_kv_decode_exchange), or with an NCCL all-gather + tk_combine_partials.
    Rank 0 also holds the whole sequence and checks the result.  Then the same with a hot window: ranks whose
    tokens lie outside the most recent `hot_window` keep them in pinned host memory and stage them back."""
    torch, dist = env.torch, env.dist
    from titan_engine_b200 import PagedKVCache
    from titan_engine_b200 import dist as D
    H, Hkv, Dh = 32, 8, 128
    rank, world, dev = env.rank, env.world, env.dev
    lo, hi = D.token_ranges(n, world)[rank]
    gen = torch.Generator(device=dev); gen.manual_seed(5)          # the same values on every rank
    q = torch.randn(1, H, Dh, device=dev, generator=gen).to(torch.bfloat16)
    n_pg = n // 16
    full = torch.randn(n_pg, Hkv, 2, 16, Dh, device=dev, generator=gen).to(torch.bfloat16)   # one layer's data, shared by all layers
    my_pages = (hi - lo) // 16
    rec = {"ok": True, "tokens": n, "layers": L, "steps": steps, "warmup": warmup, "n_gpus": world,
           "config": {"workload": f"one {n}-token sequence, 8B head shape, bf16, page 16, tokens split contiguously over "
                                  f"{world} GPUs ({hi - lo} per rank)", "parallelism": f"by token range x{world}"},
           "exchange_bytes_per_rank_per_layer": H * (Dh + 2) * 4}

    def make(window):
        c = PagedKVCache(L, H, Hkv, Dh, max(my_pages, 1), 1, max(my_pages, 1), dtype="bf16",
                         hot_window=window, cold_pages=max(my_pages, 1) if window else 0)
        sid = c.seq_alloc()
        c.adopt(sid, np.arange(my_pages, dtype=np.int32), hi - lo)
        for l in range(L):
            c.layer_views(l)[0][:my_pages].copy_(full[lo // 16:hi // 16])
        if window:
            c.set_tail(sid, n - hi)
        torch.cuda.synchronize()
        c.step_begin([sid], None)
        return c

    def time_route(fn):
        for _ in range(warmup):
            for l in range(L):
                fn(l)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        e0.record()
        for _ in range(steps):
            for l in range(L):
                fn(l)
        e1.record()
        env.barrier()
        return env.max_ms(e0.elapsed_time(e1)) / steps / L * 1e3

    cache = make(0)
    ex = D.PeerExchange(H, Dh + 2)
    out_x = torch.empty(1, H, Dh, device=dev, dtype=torch.bfloat16)
    gather = D.LongContextDecoder(cache.decode_partial, lambda st_: D.combine_partials(st_, torch.bfloat16))
    cache.decode_exchange(0, q, ex, out_x)
    torch.cuda.synchronize()
    ex.status()
    ref = gather.decode(0, q)
    torch.cuda.synchronize()
    same = env.all_ok(bool(torch.equal(ref, out_x)))
    err, ok = 0.0, True
    if rank == 0:
        whole = PagedKVCache(1, H, Hkv, Dh, n_pg, 1, n_pg, dtype="bf16")
        ws = whole.seq_alloc()
        whole.adopt(ws, np.arange(n_pg, dtype=np.int32), n)
        whole.layer_views(0)[0].copy_(full)
        whole.step_begin([ws], None)
        want = whole.decode(0, q).float()
        err = float((out_x.float() - want).abs().max())
        ok = bool(torch.allclose(out_x.float(), want, rtol=2e-3, atol=1e-2)) and float(want.abs().max()) > 0
        whole.close()
        del whole
    ok = env.all_ok(ok and same)
    rec.update(ok=ok, same_bytes_as_all_gather_route=same, max_abs_err_vs_single_gpu=err)
    rec["us_per_layer"] = time_route(lambda l: cache.decode_exchange(l, q, ex, out_x))
    ex.status()
    rec["us_per_layer_all_gather_route"] = time_route(lambda l: gather.decode(l, q))
    rec["aggregate_kv_gbs"] = n * Hkv * Dh * 2 * 2 / (rec["us_per_layer"] * 1e-6) / 1e9
    cache.device_status()
    cache.close()
    del cache, gather
    env.release()

    # cold-window variant: ranks outside the hot window stream their pages host -> device per layer
    try:
        cold = make(hot_window)
        st0 = cold.stats()
        out_c = torch.empty(1, H, Dh, device=dev, dtype=torch.bfloat16)
        cold.decode_exchange(0, q, ex, out_c)
        torch.cuda.synchronize()
        ex.status()
        same_cold = env.all_ok(bool(torch.equal(out_c, out_x)))
        us = time_route(lambda l: cold.decode_exchange(l, q, ex, out_c))
        ex.status()
        st1 = cold.stats()
        layers_run = (warmup + steps) * L
        h2d_layer = (st1["bytes_h2d"] - st0["bytes_h2d"]) / max(layers_run + 1, 1)
        t = torch.tensor([float(st1["pages_cold"]), h2d_layer], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rec["cold_window"] = {"ok": same_cold, "hot_window": hot_window, "us_per_layer": us,
                              "cold_pages_on_the_coldest_rank": int(t[0].item()),
                              "h2d_bytes_per_layer_on_the_coldest_rank": float(t[1].item()),
                              "h2d_gbs": float(t[1].item()) / (us * 1e-6) / 1e9,
                              "same_bytes_as_all_in_hbm": same_cold}
        rec["ok"] = rec["ok"] and same_cold
        cold.close()
        del cold
    except Exception as e:                                      # the cold variant must not cost the all-in-HBM numbers
        rec["cold_window"] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:300]}
    env.barrier()
    ex.close()
    del full
    env.release()
    return rec


def run_ours(args):
    env = Env()
    s = WORKLOADS[args.workload]
    L = args.layers or s["L"]
    rec = decode_workload(env, args.workload, s, L, args.steps, args.warmup, e2e=True, clocks=True,
                          decode_impl=args.decode_impl, chunk=args.chunk, rope=args.rope)
    peak, _ = measured_peak()
    unit = unit_of(s, L)
    ms_per_step = rec["ms"] / args.steps
    line = {
        "metric": METRIC, "value": env.world * args.steps / (rec["ms"] / 1e3), "unit": unit, "n_gpus": env.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 storage, fp16 mma, f32 accumulate" if rec["fp8"] else "bf16",
        "data": "synthetic", "config": config_dict(args.workload, s, rec["ctx"], env.world),
        "hbm_gbs_step": rec["ab"]["layer"] * L / (ms_per_step * 1e-3) / 1e9,
        "hbm_frac_step": rec["ab"]["layer"] * L / (ms_per_step * 1e-3) / 1e9 / peak,
        "layers": L, "chunk_tokens": rec["chunk_tokens"], "work_items_per_layer": rec["work_items"],
        "roofline": roofline_of(rec, s),
        "e2e": {"value": env.world * args.steps / (rec["ms_e2e"] / 1e3), "unit": unit,
                "h2d_bytes_per_step": rec["h2d"], "d2h_bytes_per_step": rec["d2h"], "ms_per_step": rec["ms_e2e"] / args.steps},
        "gpu_launches": rec["launches"], "clocks": rec["clocks"],
        "launch_overlap": "programmatic dependent launch: the attention launch of layer l+1 starts while that of layer l "
                          "drains (its pool is another layer's; it waits before it touches split-KV rows or out), so "
                          "ms_per_step is below layers x roofline.avg_launch_ms",
    }
    if env.rank == 0 and env.world == 1 and not args.no_cpu and args.workload == "8b-bf16":
        t_layer, reps, threads = cpu_layer_time(rec["ctx"], s, args.cpu_seconds)
        line["cpu_baseline"] = {
            "value": 1.0 / (t_layer * s["L"]), "unit": unit_of(s, s["L"]), "cores": threads, "kind": "port",
            "sample": f"{reps} x one layer of the 64-sequence batch ({int(rec['ctx'].sum())} live tokens) "
                      f"through the CPU oracle (OpenMP), extrapolated x32 layers"}

    # ---- the other configurations, as short sub-records; a failing extra never costs the headline line ----
    if args.workload == "8b-bf16" and not args.no_extras and not s.get("modified") and not args.layers:
        extras = {}
        xs, xw = max(3, min(args.steps, args.extra_steps)), 3

        def leg(name, fn):
            try:
                r = fn()
                if env.rank == 0:
                    extras[name] = r
            except Exception as e:
                extras[name] = {"ok": False, "error": f"{type(e).__name__}: {e}"[:400]}
                try:
                    env.release()
                except Exception:
                    pass

        def decode_leg(name):
            ws = WORKLOADS[name]
            r = decode_workload(env, name, ws, ws["L"], xs, xw, e2e=False, clocks=True)
            return sub_record(env, r, ws)

        leg("70b-fp8", lambda: decode_leg("70b-fp8"))
        leg("mla-bf16", lambda: decode_leg("mla-bf16"))
        leg("churn", lambda: churn_workload(env, xs, xw))
        if env.world >= 2:
            leg("long_context", lambda: long_context_workload(env, max(xs, 10), xw))
        line["workloads"] = extras
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    env.close()


def run_append(args):
    """`--append-prefill T`: the append half of the path alone - one prefill step of B sequences x T tokens
    appended to every layer (page-table scatter; FP8 pools seal every completed page).  Prints one JSON line
    with the per-layer time and the read + write bandwidth; not the headline metric."""
    import torch
    from titan_engine_b200 import PagedKVCache
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s = WORKLOADS[args.workload]
    T, L = args.append_prefill, args.layers or s["L"]
    B, Hkv, D = s["B"], s["Hkv"], s["D"]
    fp8 = s["esize"] == 1
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
    """`--multi K`: K new tokens per sequence and step, each with its own causal attention output
    (tk_kv_append_decode_multi).  Small K on the workload's 64 long contexts is the verification step of a
    speculative decoder; K >= 256 is a prefill chunk: 16 fresh sequences that append K tokens per step (the
    chunk attends to everything before it), which is where the 128-row tiles of the prefill kernel make the
    work a contraction.  Prints one JSON line with the time per layer and per token-layer and, for prefill
    chunks, the achieved tensor throughput; not the headline metric."""
    import torch
    from titan_engine_b200 import PagedKVCache
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    s = WORKLOADS[args.workload]
    K, L = args.multi, args.layers or 8
    prefill = K >= 256
    B, ps = (16 if prefill else s["B"]), s["ps"]
    ctx = np.zeros(B, dtype=np.int64) if prefill else contexts(B, s["lo"], s["hi"])
    reps = args.warmup + args.steps
    pages_end = (ctx + reps * K + ps - 1) // ps
    cache = PagedKVCache(L, s["H"], s["Hkv"], s["D"], int(pages_end.sum()) + 64, B, int(pages_end.max()) + 1, dtype="bf16",
                         max_step_tokens=B * K, prefill_impl=args.prefill_impl)
    seqs, at = [], 0
    for b in range(B):
        sid = cache.seq_alloc()
        n = int((ctx[b] + ps - 1) // ps)
        if n:
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
    times, attn_times, lens_at = [], [], []
    for _ in range(reps):
        cache.step_begin(seqs, [K] * B)
        lens_at.append(int(cache.seq_len(seqs[0])))
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        for l in range(L):
            if K == 1:
                cache.append(l, k, v)
                cache.decode(l, q, out)
            else:
                cache.append_decode_multi(l, k, v, q, out)
        e1.record()
        for l in range(L):                                     # the attention alone (the rows are in the pool)
            if K > 1:
                cache.decode_multi(l, q, out)
        e2.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / L)
        attn_times.append(e1.elapsed_time(e2) / L)
    cache.device_status()
    ms = float(np.median(times[args.warmup:]))
    line = {"metric": "multi_token_decode_us_per_layer", "value": ms * 1e3, "unit": "us per layer (append + attention)",
            "higher_is_better": False, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "tokens_per_sequence": K, "us_per_token_layer": ms * 1e3 / K,
            "config": {"workload": f"{B} sequences, " + ("fresh, growing by K tokens per step" if prefill else
                                                         f"context U[{s['lo']},{s['hi']}]") +
                                   f", {s['H']} q / {s['Hkv']} kv heads, head_dim {s['D']}, bf16, {L} layers, {K} new tokens per "
                                   f"sequence and step"}}
    if prefill:
        # flops of the attention of one layer: 4 * D * H * sum over query tokens of the positions they see
        per_step = []
        for i in range(args.warmup, reps):
            ln = lens_at[i]
            seen = K * (ln - K) + K * (K + 1) // 2
            fl = 4.0 * s["D"] * s["H"] * seen * B
            per_step.append(fl / (attn_times[i] * 1e-3) / 1e12)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        tf_peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        line["prefill"] = {"context_after_each_timed_step": lens_at[args.warmup:],
                           "attention_us_per_layer_each_step": [t * 1e3 for t in attn_times[args.warmup:]],
                           "attention_tflops_each_step": per_step,
                           "roofline": {"bound": "tensor", "achieved": float(np.median(per_step)), "peak": tf_peak,
                                        "unit": "TFLOP/s", "frac": float(np.median(per_step)) / tf_peak,
                                        "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (cuBLAS)" if peaks else
                                                       "fallback 1.4 PFLOP/s",
                                        "kernel": "prefill_mma_kernel (mma.sync m16n8k16, 64-row tiles)" if args.prefill_impl == "mma_sync"
                                                  else "prefill_tc_kernel (tcgen05.mma, accumulators in tensor memory, 128-row tiles)",
                                        "note": "flops count the causal half only"}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="8b-bf16", choices=sorted(WORKLOADS),
                    help="8b-bf16: the headline batched decode; 70b-fp8: 64 q / 8 kv heads, 32 sequences at 32768 "
                         "tokens, FP8-E4M3 pool, a resident subset of the 80 layers; mla-bf16: K rows 192 / V rows "
                         "128, 128 kv heads, 16 sequences at 4096 tokens")
    ap.add_argument("--layers", type=int, default=0, help="resident layers (0 = the workload's own)")
    ap.add_argument("--decode-impl", default="auto", choices=["auto", "simt", "mma"])
    ap.add_argument("--chunk", type=int, default=0, help="split-KV chunk tokens (the handle's chunk_tokens; 0 = chosen per step)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the `workloads` sub-records")
    ap.add_argument("--extra-steps", type=int, default=8, help="timed steps of each `workloads` sub-record")
    ap.add_argument("--rope", action="store_true", help="also fuse RoPE of q and the new K rows into each layer's call")
    ap.add_argument("--seqs", type=int, default=0, help="sequences per GPU instead of the workload's (reported in config)")
    ap.add_argument("--append-prefill", type=int, default=0, metavar="T",
                    help="measure the append kernels alone: one prefill step of T tokens per sequence and layer")
    ap.add_argument("--prefill-impl", default="auto", choices=["auto", "mma_sync"],
                    help="--multi: the prefill kernel (auto: tcgen05 at head_dim 128; mma_sync: the warp-level kernel)")
    ap.add_argument("--multi", type=int, default=0, metavar="K",
                    help="measure multi-token attention: K new tokens per sequence and step")
    args = ap.parse_args()
    if args.seqs:
        WORKLOADS[args.workload] = dict(WORKLOADS[args.workload], B=args.seqs, modified=True)
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
