"""Seeded synthetic inputs and small utilities shared by the tests."""
from __future__ import annotations

import numpy as np

from oracle import tk_oracle as O

RTOL, ATOL = 2e-3, 1e-2          # attention-output tolerance (fp16/bf16 outputs)

DT = {"fp16": O.FP16, "bf16": O.BF16, "fp8": O.FP8}


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def normal16(g: np.random.Generator, shape, dtype: int, outlier_p: float = 0.0, outlier_x: float = 20.0):
    """N(0,1) drawn in FP32, optional outliers, rounded to the 16-bit storage type (uint16 bits)."""
    x = g.standard_normal(shape, dtype=np.float32)
    if outlier_p > 0:
        x = np.where(g.random(shape) < outlier_p, x * np.float32(outlier_x), x).astype(np.float32)
    return O.f32_to_16(x, dtype)


def to_torch16(bits: np.ndarray, dtype: int, device=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(
        torch.bfloat16 if dtype == O.BF16 else torch.float16)
    return t.to(device) if device is not None else t


def from_torch16(t) -> np.ndarray:
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", rtol: float = RTOL, atol: float = ATOL,
                 out_mantissa_bits: int = 0):
    """|got - want| <= atol + rtol*|want|, plus (when the result was stored in a 16-bit type) the
    half-ulp of that type at |want|: the rounding of the output format itself, which at bf16
    (7 mantissa bits) exceeds 2e-3 relative for |x| > 5."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values in result"
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    if out_mantissa_bits:
        tol = tol + 2.0 ** (np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - out_mantissa_bits - 1)
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} outside rtol={rtol} atol={atol}; "
                             f"worst at {i}: got {got[i]:.6f} want {want[i]:.6f}; max abs err {err.max():.3e}")
    assert np.abs(got).max() > 0 or np.abs(want).max() == 0, f"{what}: result is all zero"


class Twin:
    """A GPU cache and the CPU oracle driven by the same calls, compared after every step.

    Page tables / slot indices / pool bytes / FP8 codes and scales: bit-exact.
    Attention outputs: within RTOL/ATOL of the oracle's FP32 result.
    """

    def __init__(self, L, H, Hkv, D, num_pages, max_seqs, mpps, dtype="bf16", impl="auto",
                 chunk_tokens=0, max_step_tokens=4096, io=None, seed=0, hot_window=0, cold_pages=0, Dv=None,
                 prefill_impl="auto"):
        import torch
        from titan_engine_b200 import PagedKVCache
        self.torch = torch
        self.L, self.H, self.Hkv, self.D, self.ps = L, H, Hkv, D, 16
        self.Dv = Dv or D
        self.dt = DT[dtype]
        self.carrier = DT[io] if io else (O.BF16 if self.dt == O.FP8 else self.dt)
        self.gpu = PagedKVCache(L, H, Hkv, D, num_pages, max_seqs, mpps, dtype=dtype, io_dtype=io,
                                decode_impl=impl, chunk_tokens=chunk_tokens, max_step_tokens=max_step_tokens,
                                hot_window=hot_window, cold_pages=cold_pages, v_head_dim=self.Dv if self.Dv != D else 0,
                                prefill_impl=prefill_impl)
        self.mgr = O.Manager(num_pages, max_seqs, mpps, 16)
        # With a cold tier the oracle keeps two managers: `mgr` follows the tiering rule (page/slot
        # state parity), `flat` holds the same logical data in one untiered pool (attention parity:
        # where a page lives must not change any result).
        self.tiered = hot_window > 0
        self.flat = None
        if self.tiered:
            assert self.mgr.enable_cold(hot_window, cold_pages) == O.OK
            self.flat = O.Manager(num_pages + cold_pages, max_seqs, mpps, 16)
        data_pages = num_pages + cold_pages
        self.pools = [O.Pool(self.dt, data_pages, H, Hkv, D, max_seqs, mpps, 16, self.carrier, Dv=self.Dv) for _ in range(L)]
        self.g = rng(seed)
        self.dev = self.gpu.device
        self.max_err = 0.0

    def seq_alloc(self):
        a, b = self.gpu.seq_alloc(), self.mgr.seq_alloc()
        assert a == b
        if self.flat:
            assert self.flat.seq_alloc() == a
        return a

    def seq_free(self, s):
        self.gpu.seq_free(s)
        assert self.mgr.seq_free(s) == O.OK
        if self.flat:
            assert self.flat.seq_free(s) == O.OK

    def fork(self, parent):
        """Prefix sharing on both sides: shared full pages, private copy of a partly filled last page."""
        child = self.gpu.fork(parent)
        o_child, src, dst = self.mgr.fork(parent)
        assert child == o_child
        if dst >= 0:
            for p in self.pools:
                if self.dt == O.FP8:
                    p.open_pages[child] = p.open_pages[parent]
                else:
                    p.pool[dst] = p.pool[src]
        assert self.gpu.digest() == self.mgr.digest()
        return child

    def adopt(self, s, pages, seq_len):
        """Install a caller-chosen page list (a shuffled pool) on both sides."""
        self.gpu.adopt(s, pages, seq_len)
        assert self.mgr.adopt(s, pages, seq_len) == O.OK

    def step(self, seq_ids, n_new, check_pool=False, decode=True, outlier_p=0.0, host_api=False, fused=False, begun=False,
             every_token=False, f32_out=False):
        """begun=True: the step was already begun on the GPU cache (e.g. by the scheduler).
        every_token=True: attention for EVERY token the step appends (tk_kv_decode_multi), each against the
        oracle's single-token decode with the length cut at that token - what the reference's per-token
        prefill loop computes."""
        torch = self.torch
        n_new = [0] * len(seq_ids) if n_new is None else list(n_new)
        if begun:
            old = [self.gpu.seq_len(s) - n for s, n in zip(seq_ids, n_new)]
        else:
            old = [self.gpu.seq_len(s) for s in seq_ids]
            self.gpu.step_begin(seq_ids, n_new)
        for s, n in zip(seq_ids, n_new):
            assert self.mgr.reserve(s, n) == O.OK
            if self.flat:
                assert self.flat.reserve(s, n) == O.OK
        if self.tiered:                                   # after every reservation of the step, in call order
            for s, o in zip(seq_ids, old):               # never a page the step itself is still writing
                assert self.mgr.evict_cold(s, o) >= 0
        assert self.gpu.digest() == self.mgr.digest(), "page/slot state diverged from the oracle"
        table = (self.flat or self.mgr).table()
        tok_seq = np.concatenate([np.full(n, s, np.int32) for s, n in zip(seq_ids, n_new)] or [np.zeros(0, np.int32)])
        tok_pos = np.concatenate([np.arange(o, o + n, dtype=np.int32) for o, n in zip(old, n_new)] or [np.zeros(0, np.int32)])
        nt = len(tok_seq)
        lens = [self.gpu.seq_len(s) for s in seq_ids]
        outs = []
        for layer in range(self.L):
            k16 = normal16(self.g, (nt, self.Hkv, self.D), self.carrier, outlier_p)
            v16 = normal16(self.g, (nt, self.Hkv, self.Dv), self.carrier, outlier_p)
            q16 = normal16(self.g, (nt if every_token else len(seq_ids), self.H, self.D), self.carrier)
            want_slots = self.pools[layer].append(table, tok_seq, tok_pos, k16, v16)
            if every_token:
                self.gpu.append(layer, to_torch16(k16, self.carrier, self.dev), to_torch16(v16, self.carrier, self.dev))
                qt = to_torch16(q16, self.carrier, self.dev)
                got = (self.gpu.decode_multi_f32(layer, qt) if f32_out else self.gpu.decode_multi(layer, qt).to(torch.float32)).cpu().numpy()
                if check_pool:
                    self.check_pool(layer)
                want = self.pools[layer].decode(table, tok_seq, tok_pos + 1, q16)
                assert_close(got, want, f"layer {layer} attention of every appended token ({n_new[:6]}...)",
                             out_mantissa_bits=0 if f32_out else (7 if self.carrier == O.BF16 else 10))
                self.max_err = max(self.max_err, float(np.abs(got - want).max()))
                outs.append(got)
                continue
            if host_api:
                kt, vt, qt = (to_torch16(x, self.carrier).pin_memory() for x in (k16, v16, q16))
                out_h = torch.empty(len(seq_ids), self.H, self.Dv, dtype=qt.dtype).pin_memory()
                self.gpu.append_decode_host(layer, kt, vt, qt, out_h)
                got = out_h.to(torch.float32).numpy()
            elif fused:
                got = self.gpu.append_decode(layer, to_torch16(k16, self.carrier, self.dev),
                                             to_torch16(v16, self.carrier, self.dev),
                                             to_torch16(q16, self.carrier, self.dev)).to(torch.float32).cpu().numpy()
            else:
                slots = torch.full((max(nt, 1),), -7, dtype=torch.int64, device=self.dev)
                if nt:
                    self.gpu.append(layer, to_torch16(k16, self.carrier, self.dev), to_torch16(v16, self.carrier, self.dev), slots)
                    if self.tiered:                       # device slots follow the tiered manager
                        want_slots = np.array([self.mgr.slot(int(a), int(b)) for a, b in zip(tok_seq, tok_pos)], dtype=np.int64)
                    np.testing.assert_array_equal(slots[:nt].cpu().numpy(), want_slots)
                got = None
                if decode:
                    got = self.gpu.decode(layer, to_torch16(q16, self.carrier, self.dev)).to(torch.float32).cpu().numpy()
            if check_pool:
                self.check_pool(layer)
            if decode or host_api or fused:
                want = self.pools[layer].decode(table, seq_ids, lens, q16)
                assert_close(got, want, f"layer {layer} attention ({len(seq_ids)} seqs, lens {lens[:4]}...)",
                             out_mantissa_bits=7 if self.carrier == O.BF16 else 10)
                self.max_err = max(self.max_err, float(np.abs(got - want).max()))
                outs.append(got)
        self.gpu.device_status()
        return outs

    def check_pool(self, layer):
        pool, scales, open_pages = self.gpu.layer_views(layer)
        o = self.pools[layer]
        if self.dt == O.FP8:
            np.testing.assert_array_equal(pool.cpu().numpy(), o.pool, err_msg="FP8 codes differ")
            np.testing.assert_array_equal(scales.cpu().numpy().view(np.uint32), o.scales.view(np.uint32),
                                          err_msg="FP8 scales differ")
            # open pages: only rows below each live sequence's length are defined
            got_open = from_torch16(open_pages)
            for s in range(o.max_seqs):
                n = self.mgr.seq_len(s)
                if n > 0 and n % 16:
                    np.testing.assert_array_equal(got_open[s, :, :, :n % 16], o.open_pages[s, :, :, :n % 16])
        else:
            np.testing.assert_array_equal(from_torch16(pool), o.pool, err_msg="pool bytes differ")
