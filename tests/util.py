"""Shared helpers for the test-suite: golden vectors, seeded inputs, error metrics."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz")


class Golden:
    def __init__(self):
        self._z = np.load(GOLDEN)

    def __call__(self, name: str) -> torch.Tensor:
        if name + "_bf16" in self._z:
            bits = self._z[name + "_bf16"]
            return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
        return torch.from_numpy(self._z[name].copy())

    def has(self, name: str) -> bool:
        return name in self._z or name + "_bf16" in self._z


def rel_err(a: torch.Tensor, b: torch.Tensor, floor_frac: float = 1e-2) -> float:
    """max |a-b| / max(|b|, floor) with floor = floor_frac * rms(b): the relative error used for
    the norm / RoPE / GLU tolerance (1e-2 in bf16); the floor keeps near-zero outputs, where
    an elementwise relative test is ill-conditioned, from dominating."""
    a, b = a.detach().double().flatten(), b.detach().double().flatten()
    floor = floor_frac * float(b.pow(2).mean().sqrt()) + 1e-30
    return float(((a - b).abs() / b.abs().clamp_min(floor)).max())


def bf16_ulps(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 ulps between two bf16 tensors (monotone integer mapping of the bits)."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()


def assert_norm_close(y: torch.Tensor, ref: torch.Tensor) -> None:
    """Parity of a norm output with the oracle. fp32: 1e-5 relative. 16-bit: the kernels follow
    the oracle's rounding order round(w * round(x * rstd)), but rstd itself can differ in its
    last fp32 bits (summation order), which now and then flips the inner rounding by one ulp and,
    more rarely still, lands the product two ulps away. So: never more than 2 ulps, more than
    1 ulp (the only way past 1e-2 relative) in at most 1e-5 of the elements, any difference at
    all in fewer than 0.2 %."""
    assert y.dtype == ref.dtype and y.shape == ref.shape
    if y.dtype == torch.float32:
        assert rel_err(y, ref) <= 1e-5
        return
    if y.dtype == torch.bfloat16:
        d = bf16_ulps(y, ref)
    else:  # fp16: same monotone integer mapping of the bits
        d = bf16_ulps(y.view(torch.bfloat16), ref.view(torch.bfloat16))
    assert int(d.max()) <= 2, int(d.max())
    assert float((d > 1).float().mean()) <= 1e-5
    assert float((d > 0).float().mean()) < 2e-3
    bad = ((y.double() - ref.double()).abs() >
           1e-2 * ref.double().abs().clamp_min(1e-2 * float(ref.double().pow(2).mean().sqrt())))
    assert float(bad.float().mean()) <= 1e-5


def outlier_matrix(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    """N(0,1) with 0.1% of the entries scaled x20, as in the int8 benchmark configuration."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    mask = torch.rand(rows, cols, generator=g) < 0.001
    return torch.where(mask, 20 * x, x)


def reference_path():
    """Where an unmodified copy of the reference package (a directory holding `trinix/`) can be
    imported from: $TRINIX_REFERENCE, else the untracked install under baseline/_ref of this
    checkout. None when neither exists."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("TRINIX_REFERENCE"), os.path.join(root, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "trinix")):
            return cand
    return None
