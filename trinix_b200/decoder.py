"""The Llama-2-7B-shaped decoder layer of the benchmark configuration, composed from the
`Fast*` modules with its projection weights held as per-row int8.

    h = x + Attn(RMSNorm(x));   y = h + down(SwiGLU(cat[up(n), gate(n)])),   n = RMSNorm(h)

Attention is FastGroupedQueryAttention (causal, RoPE, grouped_query_attention.py:58-207 of the
reference), the MLP activation FastSwiGLU (activation/swigelu.py:47-52: first half linear,
second half through SiLU). Every projection weight is stored as (int8 codes [out, in], fp32
scale [out]) and dequantised to bf16 by the dequantise kernel on every forward, then handed to
cuBLAS through `F.linear`.

Two ways through the same arithmetic:
  forward_modules  the composition as a user of the reference would write it: two norms, the
                   attention module (K/V tiled to all query heads when the module does so), two
                   separate up / gate GEMMs concatenated for the GLU module, residual adds in
                   torch;
  forward_fused    what the kernels allow on top: K/V handed to the kernel at their own head
                   count, up and gate as ONE GEMM that writes the GLU module's concatenated
                   input directly, the first residual add folded into the second norm
                   (residual_rmsnorm with the summed stream returned) and the second one into
                   the last GEMM's epilogue (addmm, beta = 1).
`modules` is the namespace the module classes come from: this package (default) or an
installed Trinix after `install()`.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from . import ops

WEIGHT_NAMES = ("wq", "wk", "wv", "wo", "w_up", "w_gate", "w_down")


class Int8DecoderLayer:
    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: int, ffn_dim: int,
                 weights: Dict[str, torch.Tensor], max_seq_len: int = 2048,
                 kernel_type: str = "triton", modules=None, eps: float = 1e-6,
                 rope_base: float = 10000.0):
        """`weights`: CUDA tensors [out, in] for WEIGHT_NAMES, any float dtype; they are rounded
        to bf16 and quantised here. Norm weights are ones (bf16)."""
        if modules is None:
            import trinix_b200 as modules  # noqa: PLC0415
        self.E, self.Hq, self.Hkv, self.FF = embed_dim, num_heads, num_kv_heads, ffn_dim
        dev = weights["wq"].device
        self.store = {n: ops.quantize_rowwise(weights[n].detach().to(torch.bfloat16).contiguous())
                      for n in WEIGHT_NAMES}
        # one [2*FF, E] store for the single up/gate GEMM of forward_fused (per-row scales, so
        # stacking the rows changes no code and no scale)
        self.store["w_up_gate"] = (
            torch.cat([self.store["w_up"][0], self.store["w_gate"][0]], dim=0),
            torch.cat([self.store["w_up"][1], self.store["w_gate"][1]], dim=0))
        kw = dict(bias=False, kernel_type=kernel_type, causal=True, position_method="rope",
                  max_seq_len=max_seq_len, rope_base=rope_base)
        self.attn = params_to_bf16(
            modules.FastGroupedQueryAttention(embed_dim, num_heads, num_kv_heads, **kw).to(dev))
        self.attn_native = None
        if modules.__name__ == "trinix_b200":  # the mirror module can skip the K/V tiling copy
            self.attn_native = params_to_bf16(modules.FastGroupedQueryAttention(
                embed_dim, num_heads, num_kv_heads, tile_kv=False, **kw).to(dev))
        self.norm1 = params_to_bf16(modules.FastRMSNorm(embed_dim, eps=eps).to(dev))
        self.norm2 = params_to_bf16(modules.FastRMSNorm(embed_dim, eps=eps).to(dev))
        self.act = modules.FastSwiGLU(ffn_dim)
        self.eps = eps

    def dequantised(self, names) -> Dict[str, torch.Tensor]:
        return {n: ops.dequantize_rowwise(self.store[n][0], self.store[n][1], torch.bfloat16)
                for n in names}

    @staticmethod
    def _load(attn, w) -> None:
        attn.q_proj.weight.data, attn.k_proj.weight.data = w["wq"], w["wk"]
        attn.v_proj.weight.data, attn.o_proj.weight.data = w["wv"], w["wo"]

    @torch.no_grad()
    def forward_modules(self, x: torch.Tensor) -> torch.Tensor:
        w = self.dequantised(WEIGHT_NAMES)
        self._load(self.attn, w)
        h = x + self.attn(self.norm1(x))[0]
        n = self.norm2(h)
        ff = self.act(torch.cat([F.linear(n, w["w_up"]), F.linear(n, w["w_gate"])], dim=-1))
        return h + F.linear(ff, w["w_down"])

    @torch.no_grad()
    def forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        if self.attn_native is None:
            raise RuntimeError("forward_fused needs this package's own modules")
        w = self.dequantised(("wq", "wk", "wv", "wo", "w_up_gate", "w_down"))
        self._load(self.attn_native, w)
        a = self.attn_native(self.norm1(x))[0]
        # residual add and the second norm in one pass: n = RMSNorm(a + x), h = a + x
        n, h = ops.residual_rmsnorm(a, x, self.norm2.weight, self.eps, return_sum=True)
        ff = self.act(F.linear(n, w["w_up_gate"]))
        # last residual add in the GEMM's epilogue (beta = 1)
        return torch.addmm(h.view(-1, self.E), ff.view(-1, self.FF), w["w_down"].t()).view_as(h)

    def reference_weights(self) -> Dict[str, torch.Tensor]:
        """The dequantised bf16 weights (plus unit norm weights) on the CPU, under the names a
        CPU restatement of the layer takes."""
        p: Dict[str, torch.Tensor] = {n: t.cpu() for n, t in self.dequantised(WEIGHT_NAMES).items()}
        p["attn_norm"] = torch.ones(self.E, dtype=torch.bfloat16)
        p["ffn_norm"] = torch.ones(self.E, dtype=torch.bfloat16)
        return p


def params_to_bf16(module: torch.nn.Module) -> torch.nn.Module:
    """Cast the PARAMETERS of a module tree to bf16 and leave its buffers alone. `module.bfloat16()`
    would also down-cast the float buffers the reference's position embeddings compute from
    (`inv_freq`, trinix/layers/embeddings/rope.py:61-62; `slopes`, embeddings/alibi.py:44-45, both
    non-persistent): RoPE angles then come from bf16 positions and frequencies — positions above
    256 are not even representable — and are wrong by whole radians at long range."""
    for p in module.parameters():
        p.data = p.data.to(torch.bfloat16)
    return module


def random_layer_weights(embed_dim: int, num_heads: int, num_kv_heads: int, ffn_dim: int,
                         device, seed: int = 0, std: float = 0.02,
                         generator: Optional[torch.Generator] = None) -> Dict[str, torch.Tensor]:
    """N(0, std) projection weights of the layer, drawn on the CPU in WEIGHT_NAMES order."""
    g = generator or torch.Generator().manual_seed(seed)
    d = embed_dim // num_heads
    shapes = {"wq": (embed_dim, embed_dim), "wk": (num_kv_heads * d, embed_dim),
              "wv": (num_kv_heads * d, embed_dim), "wo": (embed_dim, embed_dim),
              "w_up": (ffn_dim, embed_dim), "w_gate": (ffn_dim, embed_dim),
              "w_down": (embed_dim, ffn_dim)}
    return {n: (std * torch.randn(*shapes[n], generator=g)).to(device) for n in WEIGHT_NAMES}
