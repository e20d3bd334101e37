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


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", rtol: float = RTOL, atol: float = ATOL):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values in result"
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    if bad.any():
        i = np.unravel_index(np.argmax(err - (atol + rtol * np.abs(want))), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} outside rtol={rtol} atol={atol}; "
                             f"worst at {i}: got {got[i]:.6f} want {want[i]:.6f}; max abs err {err.max():.3e}")
    assert np.abs(got).max() > 0 or np.abs(want).max() == 0, f"{what}: result is all zero"
