"""Module-level fusion for the int8 path, in the shape of the reference's registry
(trinix/fusion.py:10-77, patterns in trinix/layers/fused/__init__.py:14-54): `fuse(norm, quant)`
returns one module that runs the fused RMSNorm -> int8 kernel instead of two launches and an
activation round trip through HBM. The reference has no int8 modules; `RowwiseInt8Quant` is the
second half of the pattern, `FastFusedRMSNormInt8` the product."""
from __future__ import annotations

import warnings
from typing import Callable, Dict, List, Tuple

import torch
import torch.nn as nn

from . import ops
from .layers import FastRMSNorm

_FUSION_REGISTRY: Dict[Tuple[type, ...], Callable[[List[nn.Module]], nn.Module]] = {}


class RowwiseInt8Quant(nn.Module):
    """x -> (int8 codes, fp32 per-row scales), scale = absmax / 127, round half to even."""

    def forward(self, x: torch.Tensor):
        return ops.quantize_rowwise(x)


class FastFusedRMSNormInt8(nn.Module):
    """RMSNorm followed by per-row int8 quantisation as one kernel: equals
    RowwiseInt8Quant()(FastRMSNorm(...)(x)) bit for bit, without writing the normalised row.
    Shares the weight parameter of the norm it was built from."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, weight: nn.Parameter = None):
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps
        self.weight = weight if weight is not None else nn.Parameter(torch.ones(hidden_size))

    def forward(self, hidden_states: torch.Tensor):
        if hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                f"Expected hidden_states with last dimension {self.hidden_size}, "
                f"but got shape {hidden_states.shape}")
        return ops.rmsnorm_quantize(hidden_states, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"hidden_size={self.hidden_size}, eps={self.eps}"


def register_fusion(pattern_key: Tuple[type, ...], factory_fn) -> None:
    """Same contract as trinix/fusion.py:10-18: factory_fn(list of modules) -> fused module."""
    _FUSION_REGISTRY[tuple(pattern_key)] = factory_fn


def _rmsnorm_int8(modules: List[nn.Module]) -> nn.Module:
    norm = modules[0]
    return FastFusedRMSNormInt8(norm.hidden_size, norm.eps, norm.weight)


register_fusion((FastRMSNorm, RowwiseInt8Quant), _rmsnorm_int8)


def fuse(*modules: nn.Module) -> nn.Module:
    """Fused module for a registered chain of module types; an unregistered chain runs as
    nn.Sequential with the reference's warning (trinix/fusion.py:31-77) — without its
    torch.compile wrapper: this backend has no tracing-compiler path."""
    if len(modules) < 2:
        raise ValueError("fuse() requires at least 2 modules")
    key = tuple(type(m) for m in modules)
    if key in _FUSION_REGISTRY:
        return _FUSION_REGISTRY[key](list(modules))
    warnings.warn(f"No fused kernel available for pattern {key}, falling back to sequential "
                  f"execution.", UserWarning, stacklevel=2)
    return nn.Sequential(*modules)


def register_with_trinix(trinix_fusion_module, trinix_rmsnorm_type) -> None:
    """Add (trinix.FastRMSNorm, RowwiseInt8Quant) to an installed Trinix's own registry, so that
    trinix.fuse(norm, RowwiseInt8Quant()) finds the fused kernel."""
    trinix_fusion_module.register_fusion((trinix_rmsnorm_type, RowwiseInt8Quant), _rmsnorm_int8)
