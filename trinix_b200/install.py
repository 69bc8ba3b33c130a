"""Plug the sm_100a backend into an installed Trinix without touching its layer modules.

The reference's modules import the kernel classes by name once
(`from ...kernels import TritonRMSNormKernel`, trinix/layers/norm/rmsnorm.py:4) but call
`.is_available()` / `.apply()` on the class object every forward. `install()` therefore
rebinds those two static methods on the reference's own class objects (so every module
that already imported them follows), rebinds `TritonAttentionKernel.apply`, replaces the
`flash_attn_func` symbol and availability flags in `trinix.layers.attention.base`
(base.py:10-24) and, in strict mode, turns the reference's silent
"kernel failed, falling back to PyTorch" path (base.py:435-439) into an error.
"""
from __future__ import annotations

import importlib
import warnings
from typing import Dict, Tuple

from . import functional
from .kernels import KERNEL_CLASSES

_saved: Dict[Tuple[object, str], object] = {}
_saved_patterns: list = []  # (registry dict, pattern key, previous factory or None)
_FALLBACK_WARNING = "Triton attention kernel failed"


def _rebind(obj, name, value):
    key = (obj, name)
    if key not in _saved:
        _saved[key] = obj.__dict__.get(name, getattr(obj, name, None))
    setattr(obj, name, value)


def install(strict: bool = True):
    """Route the reference's kernel classes to this package. Returns the `trinix` module.

    strict=True additionally registers a warnings filter that raises on the reference's
    attention fallback warning, so a failing kernel can never be masked by the torch path.
    Raises ImportError if Trinix is not importable.
    """
    trinix = importlib.import_module("trinix")
    kernels = importlib.import_module("trinix.kernels")
    try:  # the fused kernel classes live one package down (trinix/kernels/fused/__init__.py)
        fused_kernels = importlib.import_module("trinix.kernels.fused")
    except ImportError:
        fused_kernels = None
    for name, ours in KERNEL_CLASSES.items():
        theirs = getattr(kernels, name, None)
        if theirs is None and fused_kernels is not None:
            theirs = getattr(fused_kernels, name, None)
        if theirs is None:
            setattr(kernels, name, ours)
            continue
        _rebind(theirs, "is_available", staticmethod(ours.is_available))
        _rebind(theirs, "apply", staticmethod(ours.apply))
    base = importlib.import_module("trinix.layers.attention.base")
    _rebind(base, "flash_attn_func", functional.flash_attn_func)
    _rebind(base, "FLASH_ATTN_AVAILABLE", True)
    _rebind(base, "TRITON_AVAILABLE", True)
    fn_mod = importlib.import_module("trinix.layers.attention.functional")
    _rebind(fn_mod, "triton_attn_func", functional.triton_attn_func)
    attn_pkg = importlib.import_module("trinix.layers.attention")
    if hasattr(attn_pkg, "triton_attn_func"):
        _rebind(attn_pkg, "triton_attn_func", functional.triton_attn_func)
    if hasattr(trinix, "triton_attn_func"):
        _rebind(trinix, "triton_attn_func", functional.triton_attn_func)
    # trinix.fuse(FastRMSNorm(...), RowwiseInt8Quant()) -> the fused RMSNorm -> int8 kernel
    try:
        fusion_mod = importlib.import_module("trinix.fusion")
        from . import fusion as ours_fusion
        key = (trinix.FastRMSNorm, ours_fusion.RowwiseInt8Quant)
        _saved_patterns.append((fusion_mod._FUSION_REGISTRY, key,
                                fusion_mod._FUSION_REGISTRY.get(key)))
        ours_fusion.register_with_trinix(fusion_mod, trinix.FastRMSNorm)
    except (ImportError, AttributeError):
        pass  # a Trinix without the fusion registry: nothing to add
    if strict:
        warnings.filterwarnings("error", message=f".*{_FALLBACK_WARNING}.*")
    return trinix


def uninstall() -> None:
    """Undo install(): restore every rebound attribute."""
    for (obj, name), old in list(_saved.items()):
        if old is None:
            try:
                delattr(obj, name)
            except AttributeError:
                pass
        else:
            setattr(obj, name, old)
    _saved.clear()
    for registry, key, old in _saved_patterns:
        if old is None:
            registry.pop(key, None)
        else:
            registry[key] = old
    _saved_patterns.clear()
    warnings.filterwarnings("default", message=f".*{_FALLBACK_WARNING}.*")
