"""Functional attention entry points with the reference's names and argument meaning."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .kernels import TritonAttentionKernel


def triton_attn_func(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    attn_mask: Optional[torch.Tensor] = None,
    dropout_p: float = 0.0,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    window_size: Optional[Tuple[int, int]] = None,
    alibi_slopes: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Drop-in for trinix/layers/attention/functional.py:8-140.

    q (B, Sq, H, D); k, v (B, Sk, Hkv, D). Same checks and error types as the reference
    (ValueError for CPU or non-4-D tensors and shape mismatches, RuntimeError when the
    backend is unavailable), except that Hkv may divide H instead of having to equal it.
    """
    if not q.is_cuda:
        raise ValueError("triton_attn_func only supports CUDA tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(
            f"Expected 4D tensors (batch, seqlen, nheads, headdim), "
            f"got q: {q.shape}, k: {k.shape}, v: {v.shape}"
        )
    batch, _, nheads, headdim = q.shape
    _, seqlen_k, nheads_k, _ = k.shape
    if k.shape[0] != batch or k.shape[3] != headdim or nheads_k == 0 or nheads % nheads_k:
        raise ValueError(f"k shape {k.shape} doesn't match expected shape")
    if v.shape != k.shape:
        raise ValueError(f"v shape {v.shape} doesn't match expected shape")
    if not TritonAttentionKernel.is_available():
        raise RuntimeError(
            "trinix_b200 attention kernel not available: CUDA device or libtrinix_b200.so missing"
        )
    if softmax_scale is None:
        softmax_scale = headdim ** -0.5
    return TritonAttentionKernel.apply(
        q, k, v, attn_mask=attn_mask, causal=causal, scale=softmax_scale, dropout_p=dropout_p,
        window_size=window_size, alibi_slopes=alibi_slopes,
    )


def flash_attn_func(q, k, v, dropout_p: float = 0.0, softmax_scale: Optional[float] = None,
                    causal: bool = False, window_size: Tuple[int, int] = (-1, -1),
                    alibi_slopes: Optional[torch.Tensor] = None, **unsupported) -> torch.Tensor:
    """Stand-in for the third-party symbol the reference binds at
    trinix/layers/attention/base.py:10-16 and calls at :338-344 (q, k, v, dropout_p, causal).
    It runs the same sm_100a kernel, so kernel_type='flash' needs no flash-attn dispatch.

    It keeps the conventions of the symbol it replaces where they differ from
    triton_attn_func: with causal=True and Sq != Sk the mask is aligned to the BOTTOM-RIGHT
    corner (query i sees keys j <= i + Sk - Sq), which is what decoding against a KV cache
    needs; window_size uses -1 for "unbounded" on either side; alibi_slopes is (H,) or (B, H)
    with B == 1. Any other keyword of the original (softcap, deterministic, return_attn_probs,
    ...) raises instead of being dropped silently."""
    if unsupported:
        live = {n: val for n, val in unsupported.items()
                if not (val is None or val is False or (n == "softcap" and val == 0.0))}
        if live:
            raise TypeError(f"flash_attn_func stand-in does not support {sorted(live)}")
    Sq, Sk = q.shape[1], k.shape[1]
    wl, wr = (int(window_size[0]), int(window_size[1])) if window_size is not None else (-1, -1)
    slopes = alibi_slopes
    if slopes is not None and slopes.dim() == 2:
        if slopes.shape[0] != 1:
            raise NotImplementedError("per-batch alibi_slopes are not supported")
        slopes = slopes[0]
    if slopes is not None and Sq != Sk:
        # the original measures ALiBi distances from the bottom-right aligned diagonal
        raise NotImplementedError("flash_attn_func stand-in: alibi_slopes need Sq == Sk")
    window = None
    has_window = wl >= 0 or wr >= 0
    if Sq != Sk and (causal or has_window):
        # The original aligns the causal diagonal and the window to the bottom-right corner:
        # query i sees keys j <= i + (Sk - Sq). Expressed through the kernel's window predicate
        # -left <= j - i <= right with right = Sk - Sq, which needs Sk > Sq and no second window.
        if has_window or Sk < Sq:
            raise NotImplementedError(
                "flash_attn_func stand-in: Sq != Sk is supported with causal=True, Sk > Sq and "
                "no window_size only")
        window = (1 << 29, Sk - Sq)
        causal = False
    elif has_window:
        window = (wl if wl >= 0 else 1 << 29, wr if wr >= 0 else 1 << 29)
    return triton_attn_func(q, k, v, dropout_p=dropout_p, softmax_scale=softmax_scale,
                            causal=causal, window_size=window, alibi_slopes=slopes)
