"""Tensor-level entry points: torch tensors in, torch tensors out, C ABI in between.

PyTorch is plumbing here (device memory, current stream, device guard); every
computation is a kernel of libtrinix_b200.so. All functions require CUDA tensors and
raise otherwise — there is no CPU path and no fallback.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import I64x3

_DTYPE_CODE = {torch.float32: _lib.TRX_F32, torch.float16: _lib.TRX_F16,
               torch.bfloat16: _lib.TRX_BF16}

GLU_ACTS = {"swiglu": _lib.GLU_SWIGLU, "geglu": _lib.GLU_GEGLU_TANH, "reglu": _lib.GLU_REGLU}

# Number of kernels launched through this module (the benchmark reports it).
launch_count = 0


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"trinix_b200 supports float32/float16/bfloat16, got {t.dtype}") from None


def _need_cuda(*ts: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("trinix_b200 kernels require CUDA tensors (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def _stream(dev: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _rows(x: torch.Tensor) -> torch.Tensor:
    """View (or, if unavoidable, copy) x as 2-D (rows, C) with a unit column stride."""
    c = x.shape[-1]
    x2 = x.reshape(-1, c)
    # expanded tensors (a broadcast gradient, say) have rows that overlap: materialise them
    if x2.numel() and (x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < c)):
        x2 = x2.contiguous()
    return x2


def _row_stride(x2: torch.Tensor) -> int:
    return x2.stride(0) if x2.shape[0] > 1 else x2.shape[1]


# ----------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
            return_rstd: bool = False):
    """RMSNorm over the last dim; output has x's dtype and shape."""
    dev = _need_cuda(x, weight)
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2 = _rows(x)
    w = weight.detach().contiguous()
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=dev) if return_rstd else None
    with torch.cuda.device(dev):
        rc = _lib.load().trx_rmsnorm_fwd(_ptr(x2), _ptr(w), _ptr(y), _ptr(rstd), x2.shape[0],
                                         x2.shape[1], _row_stride(x2), x2.shape[1], float(eps),
                                         _code(x2), _code(w), _stream(dev))
    _lib.check("trx_rmsnorm_fwd", rc)
    _count()
    y = y.view(x.shape)
    return (y, rstd) if return_rstd else y


def layernorm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
              eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm over the last dim; weight/bias may be None."""
    dev = _need_cuda(x, weight, bias)
    x2 = _rows(x)
    wb_dtype = weight.dtype if weight is not None else (bias.dtype if bias is not None else x.dtype)
    w = weight.detach().contiguous() if weight is not None else None
    b = bias.detach().to(wb_dtype).contiguous() if bias is not None else None
    for t in (w, b):
        if t is not None and t.numel() != x.shape[-1]:
            raise ValueError("weight/bias size does not match the normalised dim")
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_layernorm_fwd(_ptr(x2), _ptr(w), _ptr(b), _ptr(y), None, None,
                                           x2.shape[0], x2.shape[1], _row_stride(x2), x2.shape[1],
                                           float(eps), _code(x2), _DTYPE_CODE[wb_dtype],
                                           _stream(dev))
    _lib.check("trx_layernorm_fwd", rc)
    _count()
    return y.view(x.shape)


# ----------------------------------------------------------------------------- int8
def quantize_rowwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric int8: returns (codes int8 of x's shape, scales fp32 of shape[:-1])."""
    dev = _need_cuda(x)
    x2 = _rows(x)
    codes = torch.empty((x2.shape[0], x2.shape[1]), dtype=torch.int8, device=dev)
    scales = torch.empty(x2.shape[0], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_quant_rowwise_i8(_ptr(x2), _ptr(codes), _ptr(scales), x2.shape[0],
                                              x2.shape[1], _row_stride(x2), x2.shape[1], _code(x2),
                                              _stream(dev))
    _lib.check("trx_quant_rowwise_i8", rc)
    _count()
    return codes.view(x.shape), scales.view(x.shape[:-1])


def dequantize_rowwise(codes: torch.Tensor, scales: torch.Tensor,
                       dtype: torch.dtype = torch.bfloat16,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of quantize_rowwise: round_dtype(float(code) * scale[row])."""
    dev = _need_cuda(codes, scales)
    if codes.dtype != torch.int8 or scales.dtype != torch.float32:
        raise TypeError("codes must be int8 and scales float32")
    c2 = _rows(codes)
    s = scales.reshape(-1).contiguous()
    if s.numel() != c2.shape[0]:
        raise ValueError("one scale per row expected")
    if out is None:
        out = torch.empty((c2.shape[0], c2.shape[1]), dtype=dtype, device=dev)
    elif out.dtype != dtype or out.numel() != c2.numel() or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of the requested dtype and size")
    with torch.cuda.device(dev):
        rc = _lib.load().trx_dequant_rowwise_i8(_ptr(c2), _ptr(s), _ptr(out), c2.shape[0],
                                                c2.shape[1], _row_stride(c2), c2.shape[1],
                                                _DTYPE_CODE[dtype], _stream(dev))
    _lib.check("trx_dequant_rowwise_i8", rc)
    _count()
    return out.view(codes.shape)


def rmsnorm_quantize(x: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused RMSNorm -> int8; equals quantize_rowwise(rmsnorm(x, weight, eps)) bit for bit."""
    dev = _need_cuda(x, weight)
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2 = _rows(x)
    w = weight.detach().contiguous()
    codes = torch.empty((x2.shape[0], x2.shape[1]), dtype=torch.int8, device=dev)
    scales = torch.empty(x2.shape[0], dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_rmsnorm_quant_i8(_ptr(x2), _ptr(w), _ptr(codes), _ptr(scales),
                                              x2.shape[0], x2.shape[1], _row_stride(x2),
                                              x2.shape[1], float(eps), _code(x2), _code(w),
                                              _stream(dev))
    _lib.check("trx_rmsnorm_quant_i8", rc)
    _count()
    return codes.view(x.shape), scales.view(x.shape[:-1])


ROW_ACTIVATIONS = {"mish": 0, "quickgelu": 1, "squared_relu": 2}


def rmsnorm_activation(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                       activation: str = "mish") -> torch.Tensor:
    """activation(RMSNorm(x)) in one pass; activation in {"mish", "quickgelu", "squared_relu"}."""
    if activation not in ROW_ACTIVATIONS:
        raise ValueError(f"Unsupported activation '{activation}'. "
                         f"Supported: {sorted(ROW_ACTIVATIONS)}")
    dev = _need_cuda(x, weight)
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2 = _rows(x)
    w = weight.detach().contiguous()
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_rmsnorm_act_fwd(_ptr(x2), _ptr(w), _ptr(y), x2.shape[0], x2.shape[1],
                                             _row_stride(x2), x2.shape[1], float(eps),
                                             ROW_ACTIVATIONS[activation], _code(x2), _code(w),
                                             _stream(dev))
    _lib.check("trx_rmsnorm_act_fwd", rc)
    _count()
    return y.view(x.shape)


def residual_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                     eps: float = 1e-6, return_sum: bool = False):
    """RMSNorm(x + residual) with the sum kept in fp32 on chip; optionally also returns the
    summed residual stream rounded to x's dtype."""
    dev = _need_cuda(x, residual, weight)
    if residual.shape != x.shape or residual.dtype != x.dtype:
        raise ValueError("residual must have the shape and dtype of x")
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2, r2 = _rows(x), _rows(residual)
    w = weight.detach().contiguous()
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    s = torch.empty_like(y) if return_sum else None
    with torch.cuda.device(dev):
        rc = _lib.load().trx_residual_rmsnorm_fwd(
            _ptr(x2), _ptr(r2), _ptr(w), _ptr(y), _ptr(s), None, x2.shape[0], x2.shape[1],
            _row_stride(x2), _row_stride(r2), x2.shape[1], x2.shape[1], float(eps), _code(x2),
            _code(w), _stream(dev))
    _lib.check("trx_residual_rmsnorm_fwd", rc)
    _count()
    y = y.view(x.shape)
    return (y, s.view(x.shape)) if return_sum else y


def residual_layernorm(x: torch.Tensor, residual: torch.Tensor, weight: Optional[torch.Tensor],
                       bias: Optional[torch.Tensor], eps: float = 1e-5,
                       return_sum: bool = False):
    """LayerNorm(x + residual) with the sum kept in fp32 on chip; the normalised value is rounded
    to x's dtype before the affine part, as the reference's fused module does. Optionally also
    returns the summed residual stream rounded to x's dtype."""
    dev = _need_cuda(x, residual, weight, bias)
    if residual.shape != x.shape or residual.dtype != x.dtype:
        raise ValueError("residual must have the shape and dtype of x")
    wb_dtype = weight.dtype if weight is not None else (bias.dtype if bias is not None else x.dtype)
    w = weight.detach().contiguous() if weight is not None else None
    b = bias.detach().to(wb_dtype).contiguous() if bias is not None else None
    for t in (w, b):
        if t is not None and t.numel() != x.shape[-1]:
            raise ValueError("weight/bias size does not match the normalised dim")
    x2, r2 = _rows(x), _rows(residual)
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    s = torch.empty_like(y) if return_sum else None
    with torch.cuda.device(dev):
        rc = _lib.load().trx_residual_layernorm_fwd(
            _ptr(x2), _ptr(r2), _ptr(w), _ptr(b), _ptr(y), _ptr(s), None, None, x2.shape[0],
            x2.shape[1], _row_stride(x2), _row_stride(r2), x2.shape[1], x2.shape[1], float(eps),
            _code(x2), _DTYPE_CODE[wb_dtype], _stream(dev))
    _lib.check("trx_residual_layernorm_fwd", rc)
    _count()
    y = y.view(x.shape)
    return (y, s.view(x.shape)) if return_sum else y


def residual_rmsnorm_quantize(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                              eps: float = 1e-6, return_sum: bool = False):
    """int8 codes and scales of RMSNorm(x + residual); equals
    quantize_rowwise(residual_rmsnorm(x, residual, weight, eps)) bit for bit."""
    dev = _need_cuda(x, residual, weight)
    if residual.shape != x.shape or residual.dtype != x.dtype:
        raise ValueError("residual must have the shape and dtype of x")
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2, r2 = _rows(x), _rows(residual)
    w = weight.detach().contiguous()
    codes = torch.empty((x2.shape[0], x2.shape[1]), dtype=torch.int8, device=dev)
    scales = torch.empty(x2.shape[0], dtype=torch.float32, device=dev)
    s = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev) if return_sum else None
    with torch.cuda.device(dev):
        rc = _lib.load().trx_residual_rmsnorm_quant_i8(
            _ptr(x2), _ptr(r2), _ptr(w), _ptr(codes), _ptr(scales), _ptr(s), x2.shape[0],
            x2.shape[1], _row_stride(x2), _row_stride(r2), x2.shape[1], x2.shape[1], float(eps),
            _code(x2), _code(w), _stream(dev))
    _lib.check("trx_residual_rmsnorm_quant_i8", rc)
    _count()
    out = (codes.view(x.shape), scales.view(x.shape[:-1]))
    return out + (s.view(x.shape),) if return_sum else out


# ----------------------------------------------------------------------------- RoPE
def _bshd(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 4:
        raise ValueError(f"expected (batch, seq, heads, head_dim), got {tuple(t.shape)}")
    return t if t.stride(-1) == 1 or t.numel() == 0 else t.contiguous()


def _tma_view(t: torch.Tensor) -> torch.Tensor:
    """A (B, S, H, D) view the attention kernel's tensor maps accept: unit head-dim stride, a
    16-byte aligned base and batch / seq / head strides that are multiples of 8 elements (a
    stride of 0, an expanded dim, is fine and stays as it is). Any other legal view (a slice
    along D at an odd offset, a head stride of 100, ...) is materialised once."""
    t = _bshd(t)
    if t.numel() == 0:
        return t
    ok = t.data_ptr() % 16 == 0 and all(
        t.shape[i] == 1 or t.stride(i) % 8 == 0 for i in range(3))
    return t if ok else t.contiguous()


def rope(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
         inverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Half-split rotary embedding of q (B,S,Hq,D) and k (B,S,Hk,D) in one launch.

    cos/sin are (S, D) (or anything that squeezes to it); only columns < D/2 are read.
    Tables must be float32 or have q's dtype.
    """
    dev = _need_cuda(q, k, cos, sin)
    if q.dtype != k.dtype:
        raise TypeError("q and k must share a dtype")
    q, k = _bshd(q), _bshd(k)
    B, S, Hq, D = q.shape
    if k.shape[0] != B or k.shape[1] != S or k.shape[3] != D:
        raise ValueError(f"k shape {tuple(k.shape)} does not match q {tuple(q.shape)}")
    cos2 = cos.reshape(-1, cos.shape[-1])
    sin2 = sin.reshape(-1, sin.shape[-1])
    if cos2.shape != sin2.shape or cos2.shape[0] < S or cos2.shape[1] < D // 2:
        raise ValueError("cos/sin tables must be (>= seq_len, >= head_dim/2) and alike")
    if cos2.dtype != sin2.dtype or cos2.dtype not in (torch.float32, q.dtype):
        cos2, sin2 = cos2.float(), sin2.float()
    cos2, sin2 = cos2.contiguous(), sin2.contiguous()
    qo = torch.empty((B, S, Hq, D), dtype=q.dtype, device=dev)
    ko = torch.empty((B, S, k.shape[2], D), dtype=k.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_rope_fwd(_ptr(q), _ptr(k), _ptr(cos2), _ptr(sin2), _ptr(qo), _ptr(ko),
                                      B, S, Hq, k.shape[2], D, I64x3(*q.stride()[:3]),
                                      I64x3(*k.stride()[:3]), I64x3(*qo.stride()[:3]),
                                      I64x3(*ko.stride()[:3]), cos2.stride(0), _code(cos2),
                                      _code(q), int(bool(inverse)), _stream(dev))
    _lib.check("trx_rope_fwd", rc)
    _count()
    return qo, ko


# ----------------------------------------------------------------------------- GLU
def glu(x: torch.Tensor, act: str) -> torch.Tensor:
    """x (..., 2H) -> (..., H): x[..., :H] * act(x[..., H:]); act in swiglu/geglu/reglu."""
    dev = _need_cuda(x)
    two_h = x.shape[-1]
    if two_h % 2:
        raise ValueError("last dimension must be even")
    h = two_h // 2
    x2 = _rows(x)
    y = torch.empty((x2.shape[0], h), dtype=x.dtype, device=dev)
    rs = _row_stride(x2)
    up_ptr = x2.data_ptr()
    gate_ptr = up_ptr + h * x2.element_size()
    with torch.cuda.device(dev):
        rc = _lib.load().trx_glu_fwd(ctypes.c_void_p(up_ptr), ctypes.c_void_p(gate_ptr), _ptr(y),
                                     x2.shape[0], h, rs, rs, h, GLU_ACTS[act], _code(x2),
                                     _stream(dev))
    _lib.check("trx_glu_fwd", rc)
    _count()
    return y.view(*x.shape[:-1], h)


def glu_pair(up: torch.Tensor, gate: torch.Tensor, act: str) -> torch.Tensor:
    """Separate up / gate tensors of equal shape (..., H) -> up * act(gate)."""
    dev = _need_cuda(up, gate)
    if up.shape != gate.shape or up.dtype != gate.dtype:
        raise ValueError("up and gate must have the same shape and dtype")
    u2, g2 = _rows(up), _rows(gate)
    y = torch.empty((u2.shape[0], u2.shape[1]), dtype=up.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().trx_glu_fwd(_ptr(u2), _ptr(g2), _ptr(y), u2.shape[0], u2.shape[1],
                                     _row_stride(u2), _row_stride(g2), u2.shape[1], GLU_ACTS[act],
                                     _code(u2), _stream(dev))
    _lib.check("trx_glu_fwd", rc)
    _count()
    return y.view(up.shape)


# ----------------------------------------------------------------------------- backward
def glu_backward(dy: torch.Tensor, x: torch.Tensor, act: str) -> torch.Tensor:
    """Gradient of glu(x, act) with respect to x (..., 2H), given dy (..., H): the two halves
    dy * act(gate) and dy * up * act'(gate) written into one tensor of x's shape."""
    dev = _need_cuda(dy, x)
    h = x.shape[-1] // 2
    if x.shape[-1] % 2 or dy.shape != x.shape[:-1] + (h,) or dy.dtype != x.dtype:
        raise ValueError("dy must have x's leading shape, half its last dimension and its dtype")
    x2, dy2 = _rows(x), _rows(dy)
    dx = torch.empty((x2.shape[0], 2 * h), dtype=x.dtype, device=dev)
    rs = _row_stride(x2)
    es = x2.element_size()
    with torch.cuda.device(dev):
        rc = _lib.load().trx_glu_bwd(
            _ptr(dy2), ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(x2.data_ptr() + h * es),
            ctypes.c_void_p(dx.data_ptr()), ctypes.c_void_p(dx.data_ptr() + h * es), x2.shape[0], h,
            _row_stride(dy2), rs, rs, 2 * h, 2 * h, GLU_ACTS[act], _code(x2), _stream(dev))
    _lib.check("trx_glu_bwd", rc)
    _count()
    return dx.view(x.shape)


def _norm_bwd_workspace(rows: int, cols: int, dev: torch.device) -> torch.Tensor:
    n = int(_lib.load().trx_norm_bwd_workspace_bytes(rows, cols))
    return torch.empty(n, dtype=torch.uint8, device=dev)


def rmsnorm_backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                     need_dw: bool = True, residual: Optional[torch.Tensor] = None,
                     activation: Optional[str] = None):
    """(dx, dw) of rmsnorm(x, weight, eps) given dy; dw is None when need_dw is False. The row
    statistics are recomputed from x; dw is summed in fp32 in a fixed order. With `residual`, the
    gradient of residual_rmsnorm(x, residual, ...): dx is then also the residual's gradient. With
    `activation`, the gradient of rmsnorm_activation(x, weight, eps, activation)."""
    if activation is not None and activation not in ROW_ACTIVATIONS:
        raise ValueError(f"Unsupported activation '{activation}'. "
                         f"Supported: {sorted(ROW_ACTIVATIONS)}")
    if activation is not None and residual is not None:
        raise ValueError("residual and activation cannot be combined")
    dev = _need_cuda(dy, x, weight, residual)
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise ValueError("dy must have the shape and dtype of x")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise ValueError("residual must have the shape and dtype of x")
    if weight.numel() != x.shape[-1]:
        raise ValueError(f"weight has {weight.numel()} elements, rows have {x.shape[-1]}")
    x2, dy2 = _rows(x), _rows(dy)
    w = weight.detach().contiguous()
    dx = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    dw = torch.empty(x2.shape[1], dtype=w.dtype, device=dev) if need_dw else None
    ws = _norm_bwd_workspace(x2.shape[0], x2.shape[1], dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if activation is not None:
            name = "trx_rmsnorm_act_bwd"
            rc = lib.trx_rmsnorm_act_bwd(
                _ptr(dy2), _ptr(x2), _ptr(w), _ptr(dx), _ptr(dw), x2.shape[0], x2.shape[1],
                _row_stride(dy2), _row_stride(x2), x2.shape[1], float(eps),
                ROW_ACTIVATIONS[activation], _code(x2), _code(w), _ptr(ws), ws.numel(),
                _stream(dev))
        elif residual is None:
            name = "trx_rmsnorm_bwd"
            rc = lib.trx_rmsnorm_bwd(
                _ptr(dy2), _ptr(x2), _ptr(w), _ptr(dx), _ptr(dw), x2.shape[0], x2.shape[1],
                _row_stride(dy2), _row_stride(x2), x2.shape[1], float(eps), _code(x2), _code(w),
                _ptr(ws), ws.numel(), _stream(dev))
        else:
            name = "trx_residual_rmsnorm_bwd"
            r2 = _rows(residual)
            rc = lib.trx_residual_rmsnorm_bwd(
                _ptr(dy2), _ptr(x2), _ptr(r2), _ptr(w), _ptr(dx), _ptr(dw), x2.shape[0],
                x2.shape[1], _row_stride(dy2), _row_stride(x2), _row_stride(r2), x2.shape[1],
                float(eps), _code(x2), _code(w), _ptr(ws), ws.numel(), _stream(dev))
    _lib.check(name, rc)
    _count()
    return dx.view(x.shape), (dw.view(weight.shape) if need_dw else None)


def layernorm_backward(dy: torch.Tensor, x: torch.Tensor, weight: Optional[torch.Tensor],
                       eps: float = 1e-5, need_dw: bool = True, need_db: bool = True,
                       residual: Optional[torch.Tensor] = None):
    """(dx, dw, db) of layernorm(x, weight, bias, eps) given dy; weight may be None (then dw is
    None); db is returned in the weight's dtype (x's dtype without a weight). With `residual`,
    the gradient of residual_layernorm(x, residual, ...): dx is then also the residual's."""
    dev = _need_cuda(dy, x, weight, residual)
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise ValueError("dy must have the shape and dtype of x")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise ValueError("residual must have the shape and dtype of x")
    if weight is not None and weight.numel() != x.shape[-1]:
        raise ValueError("weight size does not match the normalised dim")
    x2, dy2 = _rows(x), _rows(dy)
    w = weight.detach().contiguous() if weight is not None else None
    p_dtype = w.dtype if w is not None else x.dtype
    need_dw = need_dw and w is not None
    dx = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=dev)
    dw = torch.empty(x2.shape[1], dtype=p_dtype, device=dev) if need_dw else None
    db = torch.empty(x2.shape[1], dtype=p_dtype, device=dev) if need_db else None
    ws = _norm_bwd_workspace(x2.shape[0], x2.shape[1], dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        if residual is None:
            name = "trx_layernorm_bwd"
            rc = lib.trx_layernorm_bwd(
                _ptr(dy2), _ptr(x2), _ptr(w), _ptr(dx), _ptr(dw), _ptr(db), x2.shape[0],
                x2.shape[1], _row_stride(dy2), _row_stride(x2), x2.shape[1], float(eps), _code(x2),
                _DTYPE_CODE[p_dtype], _ptr(ws), ws.numel(), _stream(dev))
        else:
            name = "trx_residual_layernorm_bwd"
            r2 = _rows(residual)
            rc = lib.trx_residual_layernorm_bwd(
                _ptr(dy2), _ptr(x2), _ptr(r2), _ptr(w), _ptr(dx), _ptr(dw), _ptr(db), x2.shape[0],
                x2.shape[1], _row_stride(dy2), _row_stride(x2), _row_stride(r2), x2.shape[1],
                float(eps), _code(x2), _DTYPE_CODE[p_dtype], _ptr(ws), ws.numel(), _stream(dev))
    _lib.check(name, rc)
    _count()
    return dx.view(x.shape), dw, db


# ----------------------------------------------------------------------------- attention
_workspaces: dict = {}
_status_host: dict = {}  # device index -> pinned int32[1] mirror of the status word


def _dev_index(dev: torch.device) -> int:
    return dev.index if dev.index is not None else torch.cuda.current_device()


def _workspace(dev: torch.device) -> torch.Tensor:
    idx = _dev_index(dev)
    ws = _workspaces.get(idx)
    if ws is None:
        n = int(_lib.load().trx_attn_workspace_bytes())
        ws = torch.zeros(n, dtype=torch.uint8, device=torch.device("cuda", idx))
        _workspaces[idx] = ws
        _status_host[idx] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return ws


def _raise_if_failed(fn: str, dev: torch.device) -> None:
    """Host-side check of the status word's pinned mirror; no synchronisation. The mirror holds
    what the copy queued behind the most recent COMPLETED launch saw. Non-zero: a kernel gave up
    on a bounded wait, and it and every launch after it skipped their work, leaving their outputs
    unwritten. Both copies of the word are cleared (so that the next call runs again) and the
    failure is raised; outputs returned since the failing launch must be discarded."""
    host = _status_host[_dev_index(dev)]
    word = int(host[0])
    if word:
        _workspace(dev)[:4].zero_()
        host.zero_()
        raise _lib.TrinixB200Error(
            fn, _lib.TRX_ERR_DEVICE_STATUS,
            f"{_lib.load().trx_status_string(_lib.TRX_ERR_DEVICE_STATUS).decode()} "
            f"(status word {word:#x}); attention outputs produced since then are invalid")


def _queue_status_copy(ws: torch.Tensor, dev: torch.device) -> None:
    host = _status_host[_dev_index(dev)]
    rc = _lib.load().trx_attn_status(_ptr(ws), ctypes.c_void_p(host.data_ptr()), _stream(dev))
    if rc == _lib.TRX_ERR_DEVICE_STATUS:  # the mirror turned non-zero while this call ran
        _raise_if_failed("trx_attn_status", dev)
    _lib.check("trx_attn_status", rc)


def attention_status(device=None) -> int:
    """Status word of the attention workspace on `device` (synchronises). Non-zero means a
    bounded on-chip wait gave up in some earlier launch; the word is then cleared."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(dev)
    word = int(ws[:4].view(torch.int32).item())  # .item() waits for the stream
    if word:
        ws[:4].zero_()
    torch.cuda.current_stream(dev).synchronize()
    _status_host[_dev_index(dev)].zero_()
    return word


def dropout_seed() -> int:
    """A fresh 62-bit seed for one dropout call, drawn from torch's CPU generator: reproducible
    under torch.manual_seed, and no device synchronisation (the reference draws its seed with
    `.item()` on a CUDA tensor, trinix/kernels/attention_kernel.py:526-532)."""
    return int(torch.randint(0, 2 ** 62, (1,), dtype=torch.int64).item())


def _dense_mask(mask: torch.Tensor, B: int, Hq: int, Sq: int, Sk: int, act_dtype):
    """The mask as the kernel reads it: fp32 or the activation dtype, unit key stride, and the
    (batch, head, query) element strides of its broadcast view (shape rules of
    TritonAttentionKernel._prepare_mask, trinix/kernels/attention_kernel.py:479-495)."""
    m = mask.detach()
    if m.dtype == torch.bool:
        m = torch.zeros(m.shape, dtype=torch.float32, device=m.device).masked_fill_(m, float("-inf"))
    elif m.dtype not in (torch.float32, act_dtype):
        m = m.to(torch.float32)
    if m.dim() == 2:
        m = m[None, None]
    elif m.dim() == 3:
        m = m[:, None]
    elif m.dim() != 4:
        raise ValueError(f"Unsupported mask shape: {tuple(mask.shape)}")
    if m.shape[-2:] != (Sq, Sk) or m.shape[0] not in (1, B) or m.shape[1] not in (1, Hq):
        raise ValueError(f"mask shape {tuple(mask.shape)} does not broadcast to "
                         f"({B}, {Hq}, {Sq}, {Sk})")
    if m.stride(-1) != 1 and Sk > 1:
        m = m.contiguous()
    sb = 0 if m.shape[0] == 1 else m.stride(0)
    sh = 0 if m.shape[1] == 1 else m.stride(1)
    sq = m.stride(2) if Sq > 1 else max(Sk, m.stride(2))
    if sq < Sk:  # an expanded query dim: materialise, the kernel wants real rows
        m = m.contiguous()
        sb = 0 if m.shape[0] == 1 else m.stride(0)
        sh = 0 if m.shape[1] == 1 else m.stride(1)
        sq = m.stride(2)
    return m, (sb, sh, sq)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
              scale: Optional[float] = None, window: Optional[Tuple[int, int]] = None,
              alibi_slopes: Optional[torch.Tensor] = None, return_lse: bool = False,
              attn_mask: Optional[torch.Tensor] = None, dropout_p: float = 0.0,
              seed: Optional[int] = None, offset: int = 0):
    """softmax(scale * q k^T + bias) v; q (B,Sq,Hq,D), k/v (B,Sk,Hk,D), Hq % Hk == 0.

    Query head h reads kv head h // (Hq // Hk). window = (left, right) keeps keys with
    -left <= j - i <= right. alibi_slopes (Hq,) adds -slope * |i - j|. attn_mask is a dense
    additive mask (Sq,Sk), (B,Sq,Sk), (B,1,Sq,Sk) or (B,Hq,Sq,Sk), float (added to the scaled
    scores) or bool (True = hidden), broadcast by stride, never expanded. dropout_p in [0, 1)
    drops normalised probabilities (realised in steps of 1/256) with a Philox stream keyed by
    `seed` (drawn from torch's CPU generator when None) and `offset`; see dropout_seed().
    """
    dev = _need_cuda(q, k, v, alibi_slopes, attn_mask)
    if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("attention needs q, k, v of one dtype, bfloat16 or float16")
    if q.dim() == 4 and q.shape[-1] not in (64, 128) and 0 < q.shape[-1] < 128:
        # The kernel is built for head dims 64 and 128. Any smaller one runs as the next of the
        # two with zero columns appended: they add nothing to q.k and produce output columns that
        # are cut off again. Costs one padded copy of q, k, v; the scale keeps the true head dim.
        d_true = q.shape[-1]
        d_pad = 64 if d_true < 64 else 128
        if scale is None:
            scale = d_true ** -0.5
        pad = lambda t: torch.nn.functional.pad(t, (0, d_pad - d_true))
        res = attention(pad(q), pad(k), pad(v), causal=causal, scale=scale, window=window,
                        alibi_slopes=alibi_slopes, return_lse=return_lse, attn_mask=attn_mask,
                        dropout_p=dropout_p, seed=seed, offset=offset)
        if return_lse:
            return res[0][..., :d_true].contiguous(), res[1]
        return res[..., :d_true].contiguous()
    q, k, v = _tma_view(q), _tma_view(k), _tma_view(v)
    B, Sq, Hq, D = q.shape
    Bk, Sk, Hk, Dk = k.shape
    if (Bk, Dk) != (B, D) or v.shape != k.shape:
        raise ValueError(f"k {tuple(k.shape)} / v {tuple(v.shape)} do not match q {tuple(q.shape)}")
    if Hk == 0 or Hq % Hk:
        raise ValueError(f"query heads ({Hq}) must be a multiple of kv heads ({Hk})")
    if scale is None:
        scale = D ** -0.5
    wl, wr = (-1, -1)
    if window is not None:
        wl, wr = int(window[0]), int(window[1])
        if wl < 0 or wr < 0:
            raise ValueError("window sizes must be >= 0")
    slopes = None
    if alibi_slopes is not None:
        slopes = alibi_slopes.detach().reshape(-1).to(torch.float32).contiguous()
        if slopes.numel() != Hq:
            raise ValueError(f"alibi_slopes must have {Hq} entries")
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=dev)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=dev) if return_lse else None
    ws = _workspace(dev)
    # a failure recorded by an earlier launch surfaces here, before more work is queued
    _raise_if_failed("trx_attn_fwd", dev)
    if dropout_p:
        if not 0.0 <= dropout_p < 1.0:
            raise ValueError(f"dropout_p must be in [0, 1), got {dropout_p}")
        if seed is None:
            seed = dropout_seed()
        m, mstr = (None, (0, 0, Sk))
        if attn_mask is not None:
            m, mstr = _dense_mask(attn_mask, B, Hq, Sq, Sk, q.dtype)
        with torch.cuda.device(dev):
            rc = _lib.load().trx_attn_fwd_dropout(
                _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(slopes), _ptr(m),
                _code(m) if m is not None else 0, I64x3(*mstr), B, Sq, Sk, Hq, Hk, D,
                I64x3(*q.stride()[:3]), I64x3(*k.stride()[:3]), I64x3(*v.stride()[:3]),
                I64x3(*out.stride()[:3]), float(scale), int(bool(causal)), wl, wr, _code(q),
                float(dropout_p), int(seed) & (2 ** 64 - 1), int(offset) & 0xFFFFFFFF, _ptr(ws),
                ws.numel(), _stream(dev))
            _lib.check("trx_attn_fwd_dropout", rc)
            _queue_status_copy(ws, dev)
        _count()
        return (out, lse) if return_lse else out
    if attn_mask is not None:
        m, mstr = _dense_mask(attn_mask, B, Hq, Sq, Sk, q.dtype)
        with torch.cuda.device(dev):
            rc = _lib.load().trx_attn_fwd_mask(
                _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(slopes), _ptr(m), _code(m),
                I64x3(*mstr), B, Sq, Sk, Hq, Hk, D, I64x3(*q.stride()[:3]),
                I64x3(*k.stride()[:3]), I64x3(*v.stride()[:3]), I64x3(*out.stride()[:3]),
                float(scale), int(bool(causal)), wl, wr, _code(q), _ptr(ws), ws.numel(),
                _stream(dev))
            _lib.check("trx_attn_fwd_mask", rc)
            _queue_status_copy(ws, dev)
        _count()
        return (out, lse) if return_lse else out
    with torch.cuda.device(dev):
        rc = _lib.load().trx_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse),
                                      _ptr(slopes), B, Sq, Sk, Hq, Hk, D, I64x3(*q.stride()[:3]),
                                      I64x3(*k.stride()[:3]), I64x3(*v.stride()[:3]),
                                      I64x3(*out.stride()[:3]), float(scale), int(bool(causal)),
                                      wl, wr, _code(q), _ptr(ws), ws.numel(), _stream(dev))
        _lib.check("trx_attn_fwd", rc)
        _queue_status_copy(ws, dev)
    _count()
    return (out, lse) if return_lse else out
