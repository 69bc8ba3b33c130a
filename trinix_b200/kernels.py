"""Kernel classes with the names and call signatures of the reference's `trinix.kernels`.

The reference's layer modules look up `<KernelClass>.is_available()` and
`<KernelClass>.apply(...)` at call time (e.g. trinix/layers/norm/rmsnorm.py:47-68), so an
object with the same two static methods is a drop-in. Here `apply` runs the sm_100a
kernel through the C ABI. The classes keep the reference's `Triton*` names because that
is the interface being replaced; nothing in this package uses Triton.

Forward only: outputs are attached to the autograd graph so that a later `.backward()`
fails with a clear error instead of silently producing no gradient.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops


def _available() -> bool:
    return torch.cuda.is_available() and _lib.lib_exists()


class _ForwardOnly(torch.autograd.Function):
    """Runs `fn(*args)` outside autograd; backward raises."""

    @staticmethod
    def forward(ctx, fn, *args):
        return fn(*args)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError(
            "trinix_b200 implements the forward path only; run under torch.no_grad() "
            "or use the reference's PyTorch backend for training"
        )


def _run(fn, *args):
    needs_graph = torch.is_grad_enabled() and any(
        isinstance(a, torch.Tensor) and a.requires_grad for a in args
    )
    if needs_graph:
        return _ForwardOnly.apply(fn, *args)
    return fn(*args)


class TritonRMSNormKernel:
    """Same interface as trinix/kernels/rmsnorm_kernel.py:324-389."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: torch.Tensor, eps: float) -> torch.Tensor:
        return _run(lambda x, w: ops.rmsnorm(x, w, eps), X, W)


class TritonLayerNormKernel:
    """Same interface as trinix/kernels/layernorm_kernel.py:356-422; W and b may be None."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: Optional[torch.Tensor], b: Optional[torch.Tensor],
              eps: float) -> torch.Tensor:
        return _run(lambda x, w, bb: ops.layernorm(x, w, bb, eps), X, W, b)


class TritonFusedResidualRMSNormKernel:
    """Same interface as trinix/kernels/fused/residual_rmsnorm_kernel.py:
    apply(X, Residual, W, eps) -> RMSNorm(X + Residual)."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, Residual: torch.Tensor, W: torch.Tensor, eps: float) -> torch.Tensor:
        return _run(lambda x, r, w: ops.residual_rmsnorm(x, r, w, eps), X, Residual, W)


class TritonFusedResidualLayerNormKernel:
    """Same interface as trinix/kernels/fused/residual_layernorm_kernel.py:338-380:
    apply(X, Residual, W, b, eps) -> LayerNorm(X + Residual); W and b may be None."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, Residual: torch.Tensor, W: Optional[torch.Tensor],
              b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
        return _run(lambda x, r, w, bb: ops.residual_layernorm(x, r, w, bb, eps), X, Residual, W, b)


class TritonFusedRMSNormActivationKernel:
    """Same interface as trinix/kernels/fused/rmsnorm_activation_kernel.py:
    apply(X, W, eps, activation) -> activation(RMSNorm(X))."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: torch.Tensor, eps: float, activation: str = "mish") -> torch.Tensor:
        return _run(lambda x, w: ops.rmsnorm_activation(x, w, eps, activation), X, W)


class TritonRoPEKernel:
    """Same interface as trinix/kernels/rope_kernel.py:180-222: (q, k, cos, sin) -> (q', k')."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor,
              sin: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        return _run(lambda a, b, c, s: ops.rope(a, b, c, s), q, k, cos, sin)


class TritonSwiGLUKernel:
    """Same interface as trinix/kernels/swigelu_kernel.py:183-255."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        return _run(lambda x: ops.glu(x, "swiglu"), X)


class TritonGeGLUKernel:
    """Same interface as trinix/kernels/geglu_kernel.py:174-214."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        return _run(lambda x: ops.glu(x, "geglu"), X)


class TritonReGLUKernel:
    """Same interface as trinix/kernels/reglu_kernel.py:177-212."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        return _run(lambda x: ops.glu(x, "reglu"), X)


class TritonAttentionKernel:
    """Same interface as trinix/kernels/attention_kernel.py:436-664.

    Differences, all widening: k/v may have fewer heads than q (grouped / multi-query
    attention without tiling copies) and a different sequence length. `attn_mask` follows
    `_prepare_mask` (attention_kernel.py:479-495): 2-D (Sq, Sk), 3-D (B, Sq, Sk) or 4-D
    (B, 1 | H, Sq, Sk), additive, read through its broadcast strides. `dropout_p > 0` is not
    implemented and raises instead of silently taking another path.
    """

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              attn_mask: Optional[torch.Tensor] = None, causal: bool = False,
              scale: Optional[float] = None, dropout_p: float = 0.0,
              window_size: Optional[tuple] = None,
              alibi_slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
        if dropout_p and dropout_p > 0.0:
            raise NotImplementedError("trinix_b200 attention: dropout is not implemented")
        return _run(
            lambda a, b, c: ops.attention(a, b, c, causal=causal, scale=scale,
                                          window=window_size, alibi_slopes=alibi_slopes,
                                          attn_mask=attn_mask),
            q, k, v)


class RowwiseInt8Kernel:
    """Per-row symmetric int8 ops. The reference has no such class; the naming follows its
    kernel-class convention so the ops are reachable the same way."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def quantize(X: torch.Tensor):
        return ops.quantize_rowwise(X.detach())

    @staticmethod
    def dequantize(codes: torch.Tensor, scales: torch.Tensor,
                   dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return ops.dequantize_rowwise(codes, scales, dtype)

    @staticmethod
    def rmsnorm_quantize(X: torch.Tensor, W: torch.Tensor, eps: float):
        return ops.rmsnorm_quantize(X.detach(), W.detach(), eps)

    @staticmethod
    def residual_rmsnorm_quantize(X: torch.Tensor, Residual: torch.Tensor, W: torch.Tensor,
                                  eps: float, return_sum: bool = False):
        return ops.residual_rmsnorm_quantize(X.detach(), Residual.detach(), W.detach(), eps,
                                             return_sum)


KERNEL_CLASSES = {
    "TritonRMSNormKernel": TritonRMSNormKernel,
    "TritonLayerNormKernel": TritonLayerNormKernel,
    "TritonFusedResidualRMSNormKernel": TritonFusedResidualRMSNormKernel,
    "TritonFusedResidualLayerNormKernel": TritonFusedResidualLayerNormKernel,
    "TritonFusedRMSNormActivationKernel": TritonFusedRMSNormActivationKernel,
    "TritonRoPEKernel": TritonRoPEKernel,
    "TritonSwiGLUKernel": TritonSwiGLUKernel,
    "TritonGeGLUKernel": TritonGeGLUKernel,
    "TritonReGLUKernel": TritonReGLUKernel,
    "TritonAttentionKernel": TritonAttentionKernel,
}
