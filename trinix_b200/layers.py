"""Host-side mirror of the reference's layer modules for the forward hot path.

Same class names, constructor arguments, size thresholds and error behaviour as
`trinix.layers` (file:line in each docstring), written against this package's kernel
classes, so code written for the reference runs unchanged on machines where the
reference package itself is not installed. When the reference IS installed,
`trinix_b200.install()` patches its own modules instead and these classes are not needed.

Routing rule, as in the reference: a module calls the kernel class when its `use_triton`
/ `kernel_type` flag allows it, the kernel class reports itself available (CUDA present)
and the size threshold is met; otherwise it runs the plain torch formula. On this
package's kernels the names "triton" and "flash" both mean the sm_100a backend.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .functional import triton_attn_func
from .kernels import (
    TritonFusedResidualLayerNormKernel,
    TritonFusedResidualRMSNormKernel,
    TritonFusedRMSNormActivationKernel,
    TritonGeGLUKernel,
    TritonLayerNormKernel,
    TritonReGLUKernel,
    TritonRMSNormKernel,
    TritonRoPEKernel,
    TritonSwiGLUKernel,
)


# ----------------------------------------------------------------------------- norms
class FastRMSNorm(nn.Module):
    """Mirror of trinix/layers/norm/rmsnorm.py:7-91 (kernel for hidden_size > 2048)."""

    KERNEL_MIN_HIDDEN = 2048

    def __init__(self, hidden_size: int, eps: float = 1e-6, use_triton: bool = True):
        super().__init__()
        self.hidden_size, self.eps, self.use_triton = hidden_size, eps, use_triton
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and TritonRMSNormKernel.is_available()
                and self.hidden_size > self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        dt = hidden_states.dtype
        h = hidden_states.to(torch.float32)
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * h.to(dt)

    def _triton_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        flat = hidden_states.reshape(-1, self.hidden_size)
        return TritonRMSNormKernel.apply(flat, self.weight, self.eps).view(hidden_states.shape)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                f"Expected hidden_states with last dimension {self.hidden_size}, "
                f"but got shape {hidden_states.shape}")
        if hidden_states.is_cuda and self._check_triton_availability():
            return self._triton_forward(hidden_states)
        return self._pytorch_forward(hidden_states)

    def extra_repr(self) -> str:
        backend = "triton" if self._check_triton_availability() else "pytorch"
        return f"hidden_size={self.hidden_size}, eps={self.eps}, backend={backend}"


class FastFusedResidualRMSNorm(nn.Module):
    """Mirror of trinix/layers/fused/residual_rmsnorm.py:7-92: RMSNorm(hidden_states + residual)
    with the sum formed in fp32 (kernel for hidden_size > 2048)."""

    KERNEL_MIN_HIDDEN = 2048

    def __init__(self, hidden_size: int, eps: float = 1e-6, use_triton: bool = True):
        super().__init__()
        self.hidden_size, self.eps, self.use_triton = hidden_size, eps, use_triton
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and TritonFusedResidualRMSNormKernel.is_available()
                and self.hidden_size > self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        dt = hidden_states.dtype
        s = hidden_states.to(torch.float32) + residual.to(torch.float32)
        s = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * s.to(dt)

    def _triton_forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        flat = hidden_states.reshape(-1, self.hidden_size)
        res = residual.reshape(-1, self.hidden_size)
        out = TritonFusedResidualRMSNormKernel.apply(flat, res, self.weight, self.eps)
        return out.view(hidden_states.shape)

    def forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                f"Expected hidden_states with last dimension {self.hidden_size}, "
                f"but got shape {hidden_states.shape}")
        if hidden_states.is_cuda and self._check_triton_availability():
            return self._triton_forward(hidden_states, residual)
        return self._pytorch_forward(hidden_states, residual)


class FastFusedResidualLayerNorm(nn.Module):
    """Mirror of trinix/layers/fused/residual_layernorm.py:7-93: LayerNorm(hidden_states +
    residual) with the sum and the statistics in fp32 and the affine part applied to the value
    rounded to the input dtype (kernel for hidden_size > 4096)."""

    KERNEL_MIN_HIDDEN = 4096

    def __init__(self, hidden_size: int, eps: float = 1e-5, use_triton: bool = True):
        super().__init__()
        self.hidden_size, self.eps, self.use_triton = hidden_size, eps, use_triton
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.bias = nn.Parameter(torch.zeros(hidden_size))

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and TritonFusedResidualLayerNormKernel.is_available()
                and self.hidden_size > self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        dt = hidden_states.dtype
        s = hidden_states.to(torch.float32) + residual.to(torch.float32)
        mean = s.mean(-1, keepdim=True)
        var = (s - mean).pow(2).mean(-1, keepdim=True)
        s = (s - mean) * torch.rsqrt(var + self.eps)
        return (self.weight * s.to(dt)) + self.bias

    def _triton_forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        flat = hidden_states.reshape(-1, self.hidden_size)
        res = residual.reshape(-1, self.hidden_size)
        out = TritonFusedResidualLayerNormKernel.apply(flat, res, self.weight, self.bias, self.eps)
        return out.view(hidden_states.shape)

    def forward(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                f"Expected hidden_states with last dimension {self.hidden_size}, "
                f"but got shape {hidden_states.shape}")
        if hidden_states.is_cuda and self._check_triton_availability():
            return self._triton_forward(hidden_states, residual)
        return self._pytorch_forward(hidden_states, residual)

    def extra_repr(self) -> str:
        backend = "triton" if self._check_triton_availability() else "pytorch"
        return f"hidden_size={self.hidden_size}, eps={self.eps}, backend={backend}"


class FastFusedRMSNormActivation(nn.Module):
    """Mirror of trinix/layers/fused/rmsnorm_activation.py:9-110: activation(RMSNorm(x)) with
    activation in {"mish", "quickgelu", "squared_relu"} (kernel for hidden_size > 2048)."""

    KERNEL_MIN_HIDDEN = 2048
    SUPPORTED = ("mish", "quickgelu", "squared_relu")

    def __init__(self, hidden_size: int, eps: float = 1e-6, activation: str = "mish",
                 use_triton: bool = True):
        super().__init__()
        if activation not in self.SUPPORTED:
            raise ValueError(f"Unsupported activation '{activation}'. "
                             f"Supported: {sorted(self.SUPPORTED)}")
        self.hidden_size, self.eps, self.activation = hidden_size, eps, activation
        self.use_triton = use_triton
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and TritonFusedRMSNormActivationKernel.is_available()
                and self.hidden_size > self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        dt = hidden_states.dtype
        h = hidden_states.to(torch.float32)
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)
        n = (self.weight * h.to(dt)).to(torch.float32)
        if self.activation == "mish":
            out = n * torch.tanh(F.softplus(n))
        elif self.activation == "quickgelu":
            out = n * torch.sigmoid(1.702 * n)
        else:
            out = torch.relu(n) ** 2
        return out.to(dt)

    def _triton_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        flat = hidden_states.reshape(-1, self.hidden_size)
        out = TritonFusedRMSNormActivationKernel.apply(flat, self.weight, self.eps, self.activation)
        return out.view(hidden_states.shape)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                f"Expected hidden_states with last dimension {self.hidden_size}, "
                f"but got shape {hidden_states.shape}")
        if hidden_states.is_cuda and self._check_triton_availability():
            return self._triton_forward(hidden_states)
        return self._pytorch_forward(hidden_states)


class FastLayerNorm(nn.Module):
    """Mirror of trinix/layers/norm/layernorm.py:7-105 (kernel for hidden_size > 4096)."""

    KERNEL_MIN_HIDDEN = 4096

    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True,
                 use_triton: bool = True):
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps, self.elementwise_affine, self.use_triton = eps, elementwise_affine, use_triton
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(self.normalized_shape))
            self.bias = nn.Parameter(torch.zeros(self.normalized_shape))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and TritonLayerNormKernel.is_available()
                and len(self.normalized_shape) == 1
                and self.normalized_shape[0] > self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, input: torch.Tensor) -> torch.Tensor:
        w = self.weight.to(input.dtype) if self.weight is not None else None
        b = self.bias.to(input.dtype) if self.bias is not None else None
        return F.layer_norm(input, self.normalized_shape, w, b, self.eps)

    def _triton_forward(self, input: torch.Tensor) -> torch.Tensor:
        w = self.weight.to(input.dtype) if self.weight is not None else None
        b = self.bias.to(input.dtype) if self.bias is not None else None
        flat = input.reshape(-1, self.normalized_shape[0])
        return TritonLayerNormKernel.apply(flat, w, b, self.eps).view(input.shape)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if tuple(input.shape[-len(self.normalized_shape):]) != self.normalized_shape:
            raise ValueError(
                f"Expected input shape ending with {self.normalized_shape}, but got {input.shape}")
        if input.is_cuda and self._check_triton_availability():
            return self._triton_forward(input)
        return self._pytorch_forward(input)


# ----------------------------------------------------------------------------- GLUs
class _FastGLU(nn.Module):
    """Shared body of the three gated units: x[..., :H] * act(x[..., H:]); kernel for H >= 512."""

    KERNEL_MIN_HIDDEN = 512
    _kernel = None
    _name = "GLU"

    def __init__(self, hidden_size: int, use_triton: bool = True):
        super().__init__()
        self.hidden_size, self.use_triton = hidden_size, use_triton

    @staticmethod
    def _act(x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def _check_triton_availability(self) -> bool:
        return (self.use_triton and self._kernel.is_available()
                and self.hidden_size >= self.KERNEL_MIN_HIDDEN)

    def _pytorch_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        x1, x2 = hidden_states.split(hidden_states.shape[-1] // 2, dim=-1)
        return x1 * self._act(x2)

    def _triton_forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self._kernel.apply(hidden_states)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape[-1] % 2 != 0:
            raise ValueError(
                f"Expected hidden_states with even last dimension, "
                f"but got shape {hidden_states.shape}")
        if hidden_states.is_cuda and self._check_triton_availability():
            return self._triton_forward(hidden_states)
        return self._pytorch_forward(hidden_states)

    def extra_repr(self) -> str:
        return f"hidden_size={self.hidden_size}, use_triton={self.use_triton}"


class FastSwiGLU(_FastGLU):
    """Mirror of trinix/layers/activation/swigelu.py:7-67."""
    _kernel = TritonSwiGLUKernel
    _act = staticmethod(F.silu)


class FastGeGLU(_FastGLU):
    """Mirror of trinix/layers/activation/geglu.py (tanh-approximated GELU, :47-52)."""
    _kernel = TritonGeGLUKernel
    _act = staticmethod(lambda x: F.gelu(x, approximate="tanh"))


class FastReGLU(_FastGLU):
    """Mirror of trinix/layers/activation/reglu.py:47-52."""
    _kernel = TritonReGLUKernel
    _act = staticmethod(F.relu)


# ----------------------------------------------------------------------------- position
class FastRoPEPositionEmbedding(nn.Module):
    """Mirror of trinix/layers/embeddings/rope.py:13-134.

    forward(x, seq_len) returns (cos, sin) of shape (seq_len, dim) in x's dtype;
    apply_rotary_pos_emb rotates q and k of shape (B, S, H, D). The kernel is used for
    CUDA tensors with H*D > 2048, S > 512 and no position_ids (rope.py:81-109).
    """

    def __init__(self, dim: int, max_position_embeddings: int = 2048, base: float = 10000.0,
                 use_triton: bool = True):
        super().__init__()
        self.dim, self.max_position_embeddings, self.base = dim, max_position_embeddings, base
        self.use_triton = use_triton
        inv_freq = 1.0 / base ** (torch.arange(0, dim, 2).float() / dim)
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._table_key, self._tables = None, None

    def forward(self, x: torch.Tensor, seq_len: Optional[int] = None):
        """(cos, sin) of shape (seq_len, dim) in x's dtype. The angles are always built in
        fp32 from `base` and `dim`: the reference builds them from its `inv_freq` buffer, which
        `module.to(torch.bfloat16)` silently rounds to bf16 (positions above 256 then collapse
        onto each other); this mirror keeps the buffer for state-dict compatibility only."""
        if seq_len is None:
            seq_len = x.shape[-2]
        # the tables depend on (seq_len, device, dtype) only: the last pair is kept, which saves
        # a dozen small launches per forward in a decoder stack
        key = (int(seq_len), x.device, x.dtype)
        if self._table_key != key:
            inv_freq = 1.0 / self.base ** (
                torch.arange(0, self.dim, 2, device=x.device, dtype=torch.float32) / self.dim)
            pos = torch.arange(seq_len, device=x.device, dtype=torch.float32)
            angles = torch.outer(pos, inv_freq)
            table = torch.cat((angles, angles), dim=-1)
            self._tables = (table.cos().to(x.dtype), table.sin().to(x.dtype))
            self._table_key = key
        return self._tables

    @staticmethod
    def _rotate_half(x: torch.Tensor) -> torch.Tensor:
        half = x.shape[-1] // 2
        return torch.cat((-x[..., half:], x[..., :half]), dim=-1)

    def _check_triton_availability(self, q: torch.Tensor) -> bool:
        if not (self.use_triton and TritonRoPEKernel.is_available() and q.is_cuda):
            return False
        if q.dim() < 4:
            return False
        return q.shape[2] * q.shape[3] > 2048 and q.shape[1] > 512

    def _apply_rope_pytorch(self, q, k, cos, sin):
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return q * c + self._rotate_half(q) * s, k * c + self._rotate_half(k) * s

    def _apply_rope_with_position_ids(self, q, k, cos, sin, position_ids):
        cos = cos.reshape(-1, cos.shape[-1])[position_ids].unsqueeze(2)
        sin = sin.reshape(-1, sin.shape[-1])[position_ids].unsqueeze(2)
        return q * cos + self._rotate_half(q) * sin, k * cos + self._rotate_half(k) * sin

    def apply_rotary_pos_emb(self, q, k, cos, sin, position_ids: Optional[torch.Tensor] = None):
        if position_ids is not None:
            return self._apply_rope_with_position_ids(q, k, cos, sin, position_ids)
        if self._check_triton_availability(q):
            return TritonRoPEKernel.apply(q, k, cos, sin)
        return self._apply_rope_pytorch(q, k, cos, sin)


class FastALiBiPositionEmbedding(nn.Module):
    """Mirror of trinix/layers/embeddings/alibi.py:12-90: per-head slopes and the dense
    bias -slope * |i - j| of shape (batch, heads, S, S). The attention kernel only needs
    `slopes`; the dense bias exists for the torch path."""

    def __init__(self, num_heads: int, max_seq_len: int = 2048, use_triton: bool = True):
        super().__init__()
        self.num_heads, self.max_seq_len, self.use_triton = num_heads, max_seq_len, use_triton
        self.register_buffer("slopes", self._get_slopes(num_heads), persistent=False)

    @staticmethod
    def _get_slopes(num_heads: int) -> torch.Tensor:
        def geometric(n):
            first = 2.0 ** (-(2.0 ** (-(math.log2(n) - 3))))
            return [first ** (i + 1) for i in range(n)]

        if math.log2(num_heads).is_integer():
            vals = geometric(num_heads)
        else:
            base = 2 ** math.floor(math.log2(num_heads))
            vals = geometric(base) + geometric(2 * base)[0::2][: num_heads - base]
        return torch.tensor(vals, dtype=torch.float32)

    def forward(self, seq_len: int, batch_size: int = 1) -> torch.Tensor:
        idx = torch.arange(seq_len, device=self.slopes.device)
        dist = (idx[None, :] - idx[:, None]).abs()
        bias = -(dist[None] * self.slopes[:, None, None])
        return bias.unsqueeze(0).expand(batch_size, -1, -1, -1) if batch_size > 1 else bias[None]


# ----------------------------------------------------------------------------- attention
class FastBaseAttention(nn.Module):
    """Mirror of trinix/layers/attention/base.py:27-459, restricted to the options the
    forward hot path uses: kernel_type in {'flash', 'triton', 'pytorch'}, causal,
    position_method in {'none', 'rope', 'alibi'}, sliding window, q/k norm.

    Deliberate differences from the reference, each replacing a defect on its kernel path:
    * no silent fallback: an error inside the kernel path propagates (base.py:435-439
      swallows it and reruns in torch);
    * the sliding window reaches the kernel as (window, 0)/(window, window) bounds, not as the
      dense mask of base.py:222-237, which is NaN wherever a key is visible;
    * ALiBi reaches the kernel once, as slopes (the reference adds the dense bias to the
      mask and passes the slopes as well, grouped_query_attention.py:201 + base.py:415-417).
    """

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 kernel_type: str = "flash", causal: bool = False,
                 position_method: Union[str, nn.Module] = "none", max_seq_len: int = 2048,
                 rope_base: float = 10000.0, use_sliding_window: bool = False,
                 sliding_window_size: Optional[int] = None, qk_norm: bool = False,
                 qk_norm_type: str = "rmsnorm", use_triton_norm: bool = True,
                 use_triton_embeddings: bool = True, add_zero_attn: bool = False):
        super().__init__()
        assert embed_dim % num_heads == 0, (
            f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        assert num_heads > 0, f"num_heads must be positive, got {num_heads}"
        if kernel_type not in ("flash", "triton", "pytorch"):
            raise ValueError(f"kernel_type must be 'flash', 'triton' or 'pytorch', got {kernel_type}")
        if use_sliding_window and sliding_window_size is None:
            raise ValueError("sliding_window_size is required when use_sliding_window is True")
        if add_zero_attn:
            raise NotImplementedError("add_zero_attn is outside the forward hot path")
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.head_dim = embed_dim // num_heads
        self.scale = self.head_dim ** -0.5
        self.dropout, self.causal, self.kernel_type = dropout, causal, kernel_type
        self.use_sliding_window, self.sliding_window_size = use_sliding_window, sliding_window_size
        self.qk_norm, self.qk_norm_type = qk_norm, qk_norm_type
        if qk_norm:
            norm_cls = FastRMSNorm if qk_norm_type == "rmsnorm" else FastLayerNorm
            self.q_norm = norm_cls(self.head_dim, use_triton=use_triton_norm)
            self.k_norm = norm_cls(self.head_dim, use_triton=use_triton_norm)
        if isinstance(position_method, nn.Module):
            raise NotImplementedError("custom position modules are outside the forward hot path")
        self.position_method = position_method
        if position_method == "rope":
            self.position_embedding = FastRoPEPositionEmbedding(
                self.head_dim, max_seq_len, rope_base, use_triton=use_triton_embeddings)
        elif position_method == "alibi":
            self.position_embedding = FastALiBiPositionEmbedding(
                num_heads, max_seq_len, use_triton=use_triton_embeddings)
        elif position_method == "none":
            self.position_embedding = None
        else:
            raise ValueError(f"unknown position_method {position_method!r}")

    # -- helpers ---------------------------------------------------------------------
    def _uses_kernel(self, q: torch.Tensor) -> bool:
        return self.kernel_type in ("flash", "triton") and q.is_cuda

    def _window_mask(self, seq_q: int, seq_k: int, device) -> torch.Tensor:
        d = torch.arange(seq_k, device=device)[None, :] - torch.arange(seq_q, device=device)[:, None]
        w = self.sliding_window_size
        visible = (d >= -w) & (d <= (0 if self.causal else w))
        return torch.zeros(seq_q, seq_k, device=device).masked_fill(~visible, float("-inf"))

    def _apply_pytorch_attention(self, q, k, v, attn_mask=None):
        """Same arithmetic as base.py:347-400: bmm, scale, causal fill, additive mask, softmax, bmm."""
        B, S, H, D = q.shape
        Sk = k.shape[1]
        qf = q.transpose(1, 2).reshape(B * H, S, D)
        kf = k.transpose(1, 2).reshape(B * H, Sk, D)
        vf = v.transpose(1, 2).reshape(B * H, Sk, D)
        w = torch.bmm(qf, kf.transpose(-2, -1)) * self.scale
        if self.causal:
            w.masked_fill_(torch.triu(torch.ones(S, Sk, device=q.device), diagonal=1).bool(),
                           float("-inf"))
        if attn_mask is not None:
            m = attn_mask
            if m.dim() == 4:
                m = m.expand(B, H, S, Sk).reshape(B * H, S, Sk)
            elif m.dim() == 2:
                m = m.unsqueeze(0)
            w = w + m.to(w.dtype)
        w = F.dropout(F.softmax(w, dim=-1), p=self.dropout, training=self.training)
        return torch.bmm(w, vf).reshape(B, H, S, D).transpose(1, 2)

    def forward_attention(self, q, k, v, attn_mask=None):
        """q (B,S,H,D); k, v (B,Sk,Hkv,D) with Hkv dividing H. Returns (B,S,H,D)."""
        if self._uses_kernel(q):
            window = None
            if self.use_sliding_window:
                w = self.sliding_window_size
                window = (w, 0 if self.causal else w)
            slopes = self.position_embedding.slopes if self.position_method == "alibi" else None
            return triton_attn_func(q, k, v, attn_mask=attn_mask, softmax_scale=self.scale,
                                    dropout_p=self.dropout if self.training else 0.0,
                                    causal=self.causal, window_size=window, alibi_slopes=slopes)
        g = q.shape[2] // k.shape[2]
        if g > 1:
            k, v = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
        mask = attn_mask
        if self.use_sliding_window:
            wm = self._window_mask(q.shape[1], k.shape[1], q.device)
            mask = wm if mask is None else mask + wm
        if self.position_method == "alibi":
            bias = self.position_embedding(max(q.shape[1], k.shape[1]), 1)
            bias = bias[:, :, : q.shape[1], : k.shape[1]]
            mask = bias if mask is None else mask + bias
        return self._apply_pytorch_attention(q, k, v, mask)


class FastGroupedQueryAttention(FastBaseAttention):
    """Mirror of trinix/layers/attention/grouped_query_attention.py:58-207.

    forward(hidden_states) -> (output, present_key_value). With `tile_kv=True` (what the
    reference does, :140-145/:189-190) K and V are first copied out to all query heads;
    `tile_kv=False` hands the Hkv-head tensors to the kernel, which maps query head h to
    kv head h // groups itself — same result, no copy.
    """

    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: int, dropout: float = 0.0,
                 bias: bool = True, kernel_type: str = "flash", causal: bool = False,
                 head_dim: Optional[int] = None, position_method: Union[str, nn.Module] = "none",
                 max_seq_len: int = 2048, rope_base: float = 10000.0,
                 use_sliding_window: bool = False, sliding_window_size: Optional[int] = None,
                 qk_norm: bool = False, qk_norm_type: str = "rmsnorm",
                 use_triton_norm: bool = True, use_triton_embeddings: bool = True,
                 tile_kv: bool = True):
        assert num_heads % num_kv_heads == 0, (
            f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        inner = num_heads * head_dim if head_dim is not None else embed_dim
        super().__init__(inner, num_heads, dropout, bias, kernel_type, causal, position_method,
                         max_seq_len, rope_base, use_sliding_window, sliding_window_size, qk_norm,
                         qk_norm_type, use_triton_norm, use_triton_embeddings, False)
        self.num_kv_heads = num_kv_heads
        self.num_key_value_groups = num_heads // num_kv_heads
        self.tile_kv = tile_kv
        self.q_proj = nn.Linear(embed_dim, num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(embed_dim, num_kv_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(embed_dim, num_kv_heads * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(num_heads * self.head_dim, embed_dim, bias=bias)
        for proj in (self.q_proj, self.k_proj, self.v_proj, self.o_proj):
            nn.init.xavier_uniform_(proj.weight)
            if proj.bias is not None:
                nn.init.zeros_(proj.bias)

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_embeddings=None, position_ids: Optional[torch.Tensor] = None,
                past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                use_cache: bool = False, **kwargs):
        B, S, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(B, S, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(B, S, self.num_kv_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(B, S, self.num_kv_heads, self.head_dim)
        if self.position_method == "rope":
            cos, sin = self.position_embedding(q, S)
            q, k = self.position_embedding.apply_rotary_pos_emb(q, k, cos, sin, position_ids)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        present = None
        if past_key_value is not None:
            k = torch.cat([past_key_value[0].transpose(1, 2), k], dim=1)
            v = torch.cat([past_key_value[1].transpose(1, 2), v], dim=1)
        if use_cache:
            present = (k.transpose(1, 2), v.transpose(1, 2))  # (B, Hkv, S, D) like the reference
        if self.tile_kv and self.num_key_value_groups > 1:
            k = k.repeat_interleave(self.num_key_value_groups, dim=2)
            v = v.repeat_interleave(self.num_key_value_groups, dim=2)
        out = self.forward_attention(q, k, v, attention_mask)
        return self.o_proj(out.reshape(B, S, -1)), present


class FastMultiQueryAttention(FastGroupedQueryAttention):
    """Mirror of trinix/layers/attention/multi_query_attention.py: one shared kv head."""

    def __init__(self, embed_dim: int, num_heads: int, **kwargs):
        super().__init__(embed_dim, num_heads, 1, **kwargs)
