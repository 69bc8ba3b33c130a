"""numpy restatement of the per-row symmetric int8 path (test infrastructure only).

The reference has no int8 code, so parity for these functions is unpinned by it; the
contract is the formula in this project's baseline configuration: scale = rowwise
absmax / 127 in fp32 (IEEE division), codes = round-half-to-even(x / scale) clamped to
[-127, 127]. numpy's float32 `/` is the IEEE division and `np.rint` rounds half to even,
which makes this an arithmetic cross-check of the torch restatement in reference_port.py.
"""
from __future__ import annotations

import numpy as np


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 values (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round-to-nearest-even (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))
    return (rounded >> 16).astype(np.uint16)


def quantize_rowwise_np(x: np.ndarray):
    """x float32 [R, C] (already holding the exact input values) -> (int8 codes, f32 scales)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    am = np.abs(x).max(axis=-1, keepdims=True).astype(np.float32)
    s = am / np.float32(127.0)
    safe = np.where(s > 0, s, np.float32(1.0)).astype(np.float32)
    q = np.rint(x / safe)
    q = np.clip(q, -127.0, 127.0)
    q = np.where(s > 0, q, 0.0)
    return q.astype(np.int8), s[..., 0].astype(np.float32)


def dequantize_rowwise_np(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """-> float32 products float(code) * scale (round to the target dtype separately)."""
    return codes.astype(np.float32) * scales.astype(np.float32)[..., None]
