"""ctypes binding of libtrinix_b200.so (the C ABI declared in include/trinix_b200.h).

The library is the only compute path of this package: if it is missing, loading fails
loudly; there is no fallback of any kind.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libtrinix_b200.so")

TRX_F32, TRX_F16, TRX_BF16 = 0, 1, 2
GLU_SWIGLU, GLU_GEGLU_TANH, GLU_REGLU = 0, 1, 2
TRX_ERR_DEVICE_STATUS = -8

I64x3 = c_int64 * 3

# name -> (restype, argtypes); mirrors include/trinix_b200.h one to one.
SIGNATURES = {
    "trx_version": (c_int, []),
    "trx_status_string": (c_char_p, [c_int]),
    "trx_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                c_int64, c_float, c_int, c_int, c_void_p]),
    "trx_rmsnorm_act_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                    c_float, c_int, c_int, c_int, c_void_p]),
    "trx_layernorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int,
                                  c_void_p]),
    "trx_quant_rowwise_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                     c_int64, c_int, c_void_p]),
    "trx_dequant_rowwise_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                       c_int64, c_int, c_void_p]),
    "trx_rmsnorm_quant_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                     c_int64, c_int64, c_float, c_int, c_int, c_void_p]),
    "trx_residual_rmsnorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_float, c_int, c_int, c_void_p]),
    "trx_residual_layernorm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_float, c_int, c_int, c_void_p]),
    "trx_residual_rmsnorm_quant_i8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_int64, c_int64, c_int64, c_int64,
                                              c_int64, c_int64, c_float, c_int, c_int, c_void_p]),
    "trx_rope_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                             c_int64, c_int64, c_int64, c_int64, I64x3, I64x3, I64x3, I64x3,
                             c_int64, c_int, c_int, c_int, c_void_p]),
    "trx_glu_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                            c_int64, c_int, c_int, c_void_p]),
    "trx_glu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                            c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "trx_norm_bwd_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "trx_rmsnorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                c_int64, c_int64, c_int64, c_float, c_int, c_int, c_void_p,
                                c_size_t, c_void_p]),
    "trx_layernorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int,
                                  c_int, c_void_p, c_size_t, c_void_p]),
    "trx_residual_rmsnorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                         c_float, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "trx_residual_layernorm_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_float, c_int, c_int, c_void_p,
                                           c_size_t, c_void_p]),
    "trx_rmsnorm_act_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                    c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_int,
                                    c_void_p, c_size_t, c_void_p]),
    "trx_attn_workspace_bytes": (c_size_t, []),
    "trx_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                             c_int64, c_int64, c_int64, c_int64, c_int64, I64x3, I64x3, I64x3,
                             I64x3, c_float, c_int, c_int64, c_int64, c_int, c_void_p, c_size_t,
                             c_void_p]),
    "trx_attn_fwd_mask": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, I64x3, c_int64, c_int64, c_int64, c_int64,
                                  c_int64, c_int64, I64x3, I64x3, I64x3, I64x3, c_float, c_int,
                                  c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p]),
    "trx_attn_fwd_dropout": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_int, I64x3, c_int64, c_int64, c_int64, c_int64,
                                     c_int64, c_int64, I64x3, I64x3, I64x3, I64x3, c_float, c_int,
                                     c_int64, c_int64, c_int, c_float, c_uint64, c_uint32, c_void_p,
                                     c_size_t, c_void_p]),
    "trx_attn_status": (c_int, [c_void_p, c_void_p, c_void_p]),
    "trx_attn_fwd_static_scratch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                            c_int64, I64x3, I64x3, I64x3, I64x3, c_float, c_int,
                                            c_int64, c_int64, c_int, c_void_p, c_void_p]),
}

_lib = None
_lock = threading.Lock()


class TrinixB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with status {code}: {text}")
        self.code = code


def lib_exists() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing. Build it with `python -m trinix_b200.build`; "
                    "trinix_b200 has no fallback path."
                )
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
                fn.restype = res
                fn.argtypes = args
            if lib.trx_version() != 1:
                raise RuntimeError("libtrinix_b200.so ABI version mismatch")
            _lib = lib
    return _lib


def check(fn: str, code: int) -> None:
    if code != 0:
        text = load().trx_status_string(code).decode()
        raise TrinixB200Error(fn, code, text)
