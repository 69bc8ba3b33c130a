"""Kernel classes with the names and call signatures of the reference's `trinix.kernels`.

The reference's layer modules look up `<KernelClass>.is_available()` and
`<KernelClass>.apply(...)` at call time (e.g. trinix/layers/norm/rmsnorm.py:47-68), so an
object with the same two static methods is a drop-in. Here `apply` runs the sm_100a
kernel through the C ABI. The classes keep the reference's `Triton*` names because that
is the interface being replaced; nothing in this package uses Triton.

RMSNorm, LayerNorm, their residual and activation forms, RoPE and the GLUs are differentiable:
their autograd functions run the backward kernels of the same library (the reference's
Triton*Function.backward methods, e.g. trinix/kernels/rmsnorm_kernel.py:270-321). Attention and
the int8 ops are forward only, as attention is in the reference (TritonAttentionKernel has no
backward): their outputs are attached to the autograd graph so that a later `.backward()` fails
with a clear error instead of silently producing no gradient.
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


def _needs_graph(*args) -> bool:
    return torch.is_grad_enabled() and any(
        isinstance(a, torch.Tensor) and a.requires_grad for a in args
    )


def _run(fn, *args):
    if _needs_graph(*args):
        return _ForwardOnly.apply(fn, *args)
    return fn(*args)


class _RMSNormFn(torch.autograd.Function):
    """Counterpart of TritonRMSNormFunction (trinix/kernels/rmsnorm_kernel.py:197-321). Saves x and
    w only: the backward kernel recomputes the row statistics."""

    @staticmethod
    def forward(ctx, X, W, eps):
        ctx.save_for_backward(X, W)
        ctx.eps = eps
        return ops.rmsnorm(X, W, eps)

    @staticmethod
    def backward(ctx, dY):
        X, W = ctx.saved_tensors
        dx, dw = ops.rmsnorm_backward(dY, X, W, ctx.eps, need_dw=ctx.needs_input_grad[1])
        return dx, dw, None


class _LayerNormFn(torch.autograd.Function):
    """Counterpart of TritonLayerNormFunction (trinix/kernels/layernorm_kernel.py:224-353)."""

    @staticmethod
    def forward(ctx, X, W, b, eps):
        ctx.save_for_backward(X, W)
        ctx.eps = eps
        ctx.bias_dtype = b.dtype if b is not None else None
        return ops.layernorm(X, W, b, eps)

    @staticmethod
    def backward(ctx, dY):
        X, W = ctx.saved_tensors
        need_db = ctx.bias_dtype is not None and ctx.needs_input_grad[2]
        dx, dw, db = ops.layernorm_backward(dY, X, W, ctx.eps, need_dw=ctx.needs_input_grad[1],
                                            need_db=need_db)
        if db is not None and db.dtype != ctx.bias_dtype:
            db = db.to(ctx.bias_dtype)
        return dx, dw, db, None


class _ResidualRMSNormFn(torch.autograd.Function):
    """Counterpart of TritonFusedResidualRMSNormFunction
    (trinix/kernels/fused/residual_rmsnorm_kernel.py:209-303): x and the residual share one
    gradient, the RMSNorm gradient at the fp32 sum."""

    @staticmethod
    def forward(ctx, X, Residual, W, eps):
        ctx.save_for_backward(X, Residual, W)
        ctx.eps = eps
        return ops.residual_rmsnorm(X, Residual, W, eps)

    @staticmethod
    def backward(ctx, dY):
        X, Residual, W = ctx.saved_tensors
        dx, dw = ops.rmsnorm_backward(dY, X, W, ctx.eps, need_dw=ctx.needs_input_grad[2],
                                      residual=Residual)
        return dx, dx, dw, None


class _ResidualLayerNormFn(torch.autograd.Function):
    """Counterpart of TritonFusedResidualLayerNormFunction
    (trinix/kernels/fused/residual_layernorm_kernel.py:228-335)."""

    @staticmethod
    def forward(ctx, X, Residual, W, b, eps):
        ctx.save_for_backward(X, Residual, W)
        ctx.eps = eps
        ctx.bias_dtype = b.dtype if b is not None else None
        return ops.residual_layernorm(X, Residual, W, b, eps)

    @staticmethod
    def backward(ctx, dY):
        X, Residual, W = ctx.saved_tensors
        need_db = ctx.bias_dtype is not None and ctx.needs_input_grad[3]
        dx, dw, db = ops.layernorm_backward(dY, X, W, ctx.eps, need_dw=ctx.needs_input_grad[2],
                                            need_db=need_db, residual=Residual)
        if db is not None and db.dtype != ctx.bias_dtype:
            db = db.to(ctx.bias_dtype)
        return dx, dx, dw, db, None


class _RMSNormActivationFn(torch.autograd.Function):
    """Counterpart of TritonFusedRMSNormActivationFunction
    (trinix/kernels/fused/rmsnorm_activation_kernel.py:236-330)."""

    @staticmethod
    def forward(ctx, X, W, eps, activation):
        ctx.save_for_backward(X, W)
        ctx.eps, ctx.activation = eps, activation
        return ops.rmsnorm_activation(X, W, eps, activation)

    @staticmethod
    def backward(ctx, dY):
        X, W = ctx.saved_tensors
        dx, dw = ops.rmsnorm_backward(dY, X, W, ctx.eps, need_dw=ctx.needs_input_grad[1],
                                      activation=ctx.activation)
        return dx, dw, None, None


class _GLUFn(torch.autograd.Function):
    """Counterpart of Triton{SwiGLU,GeGLU,ReGLU}Function (e.g.
    trinix/kernels/swigelu_kernel.py:94-180): saves the input, one backward kernel."""

    @staticmethod
    def forward(ctx, X, act):
        ctx.save_for_backward(X)
        ctx.act = act
        return ops.glu(X, act)

    @staticmethod
    def backward(ctx, dY):
        (X,) = ctx.saved_tensors
        return ops.glu_backward(dY, X, ctx.act), None


class _RoPEFn(torch.autograd.Function):
    """Counterpart of TritonRoPEFunction (trinix/kernels/rope_kernel.py:133-177): the backward is
    the rotation by the negated angle, applied to both gradients in one launch."""

    @staticmethod
    def forward(ctx, q, k, cos, sin):
        ctx.save_for_backward(cos, sin)
        return ops.rope(q, k, cos, sin)

    @staticmethod
    def backward(ctx, grad_q, grad_k):
        cos, sin = ctx.saved_tensors
        dq, dk = ops.rope(grad_q, grad_k, cos, sin, inverse=True)
        return dq, dk, None, None


class TritonRMSNormKernel:
    """Same interface as trinix/kernels/rmsnorm_kernel.py:324-389."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: torch.Tensor, eps: float) -> torch.Tensor:
        if _needs_graph(X, W):
            return _RMSNormFn.apply(X, W, eps)
        return ops.rmsnorm(X, W, eps)


class TritonLayerNormKernel:
    """Same interface as trinix/kernels/layernorm_kernel.py:356-422; W and b may be None."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: Optional[torch.Tensor], b: Optional[torch.Tensor],
              eps: float) -> torch.Tensor:
        if _needs_graph(X, W, b):
            return _LayerNormFn.apply(X, W, b, eps)
        return ops.layernorm(X, W, b, eps)


class TritonFusedResidualRMSNormKernel:
    """Same interface as trinix/kernels/fused/residual_rmsnorm_kernel.py:
    apply(X, Residual, W, eps) -> RMSNorm(X + Residual)."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, Residual: torch.Tensor, W: torch.Tensor, eps: float) -> torch.Tensor:
        if _needs_graph(X, Residual, W):
            return _ResidualRMSNormFn.apply(X, Residual, W, eps)
        return ops.residual_rmsnorm(X, Residual, W, eps)


class TritonFusedResidualLayerNormKernel:
    """Same interface as trinix/kernels/fused/residual_layernorm_kernel.py:338-380:
    apply(X, Residual, W, b, eps) -> LayerNorm(X + Residual); W and b may be None."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, Residual: torch.Tensor, W: Optional[torch.Tensor],
              b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
        if _needs_graph(X, Residual, W, b):
            return _ResidualLayerNormFn.apply(X, Residual, W, b, eps)
        return ops.residual_layernorm(X, Residual, W, b, eps)


class TritonFusedRMSNormActivationKernel:
    """Same interface as trinix/kernels/fused/rmsnorm_activation_kernel.py:
    apply(X, W, eps, activation) -> activation(RMSNorm(X))."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor, W: torch.Tensor, eps: float, activation: str = "mish") -> torch.Tensor:
        if _needs_graph(X, W):
            return _RMSNormActivationFn.apply(X, W, eps, activation)
        return ops.rmsnorm_activation(X, W, eps, activation)


class TritonRoPEKernel:
    """Same interface as trinix/kernels/rope_kernel.py:180-222: (q, k, cos, sin) -> (q', k')."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor,
              sin: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        if _needs_graph(q, k):
            return _RoPEFn.apply(q, k, cos, sin)
        return ops.rope(q, k, cos, sin)


class TritonSwiGLUKernel:
    """Same interface as trinix/kernels/swigelu_kernel.py:183-255."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        if _needs_graph(X):
            return _GLUFn.apply(X, "swiglu")
        return ops.glu(X, "swiglu")


class TritonGeGLUKernel:
    """Same interface as trinix/kernels/geglu_kernel.py:174-214."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        if _needs_graph(X):
            return _GLUFn.apply(X, "geglu")
        return ops.glu(X, "geglu")


class TritonReGLUKernel:
    """Same interface as trinix/kernels/reglu_kernel.py:177-212."""

    @staticmethod
    def is_available() -> bool:
        return _available()

    @staticmethod
    def apply(X: torch.Tensor) -> torch.Tensor:
        if _needs_graph(X):
            return _GLUFn.apply(X, "reglu")
        return ops.glu(X, "reglu")


class TritonAttentionKernel:
    """Same interface as trinix/kernels/attention_kernel.py:436-664.

    Differences, all widening: k/v may have fewer heads than q (grouped / multi-query
    attention without tiling copies) and a different sequence length. `attn_mask` follows
    `_prepare_mask` (attention_kernel.py:479-495): 2-D (Sq, Sk), 3-D (B, Sq, Sk) or 4-D
    (B, 1 | H, Sq, Sk), additive, read through its broadcast strides. `dropout_p > 0` drops
    normalised probabilities (the order of the reference's PyTorch backend, base.py:394-397; its
    Triton kernel lets dropped probabilities count in the normaliser, attention_kernel.py:395-406)
    with a Philox stream whose seed comes from torch's CPU generator.
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
        return _run(
            lambda a, b, c: ops.attention(a, b, c, causal=causal, scale=scale,
                                          window=window_size, alibi_slopes=alibi_slopes,
                                          attn_mask=attn_mask,
                                          dropout_p=float(dropout_p or 0.0)),
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
