"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself.

    TRINIX_REFERENCE=/path/to/trinix-reference python tests/golden/make_golden.py

Imports the unmodified reference package (Trinix 0.1.4), runs its PyTorch backend on CPU
(no CUDA here, so every module takes `_pytorch_forward`) on small seeded inputs and stores
inputs and outputs in `reference_vectors.npz`. bf16 tensors are stored as their uint16 bit
patterns (key suffix `_bf16`). The reference has no int8 code, so there are no int8 vectors.
"""
import os
import sys

import numpy as np
import torch

REF = os.environ.get("TRINIX_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "trinix")):
    raise SystemExit("set TRINIX_REFERENCE to a checkout of the reference (the folder holding trinix/)")
sys.path.insert(0, REF)

import trinix  # noqa: E402
from trinix.layers.activation.geglu import FastGeGLU  # noqa: E402
from trinix.layers.activation.reglu import FastReGLU  # noqa: E402
from trinix.layers.activation.swigelu import FastSwiGLU  # noqa: E402
from trinix.layers.attention.base import FastBaseAttention  # noqa: E402
from trinix.layers.attention.grouped_query_attention import FastGroupedQueryAttention  # noqa: E402
from trinix.layers.embeddings.alibi import FastALiBiPositionEmbedding  # noqa: E402
from trinix.layers.embeddings.rope import FastRoPEPositionEmbedding  # noqa: E402
from trinix.layers.norm.layernorm import FastLayerNorm  # noqa: E402
from trinix.layers.norm.rmsnorm import FastRMSNorm  # noqa: E402
from trinix.layers.fused.residual_layernorm import FastFusedResidualLayerNorm  # noqa: E402
from trinix.layers.fused.residual_rmsnorm import FastFusedResidualRMSNorm  # noqa: E402
from trinix.layers.fused.rmsnorm_activation import FastFusedRMSNormActivation  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
vec = {}


def put(name, t):
    t = t.detach()
    if t.dtype == torch.bfloat16:
        vec[name + "_bf16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
    else:
        vec[name] = t.contiguous().numpy()


torch.set_num_threads(1)
g = torch.Generator().manual_seed(0)

with torch.no_grad():
    # --- RMSNorm, the CPU-runnable baseline configuration (768, eps 1e-6, fp32), cut to 8 rows
    x = torch.randn(4, 128, 768, generator=g)
    w = 1 + 0.02 * torch.randn(768, generator=g)
    m = FastRMSNorm(768, eps=1e-6, use_triton=False)
    m.weight.copy_(w)
    xs = x[:1, :8].contiguous()
    put("rms_f32_x", xs); put("rms_f32_w", w); put("rms_f32_y", m(xs))
    # bf16 activations and bf16 weight
    xb = torch.randn(12, 512, generator=g).bfloat16()
    wb = (1 + 0.02 * torch.randn(512, generator=g)).bfloat16()
    mb = FastRMSNorm(512, eps=1e-6, use_triton=False).bfloat16()
    mb.weight.copy_(wb)
    put("rms_bf16_x", xb); put("rms_bf16_w", wb); put("rms_bf16_y", mb(xb))

    # --- LayerNorm fp32 with affine, bf16 without
    xl = torch.randn(6, 768, generator=g)
    wl = 1 + 0.1 * torch.randn(768, generator=g)
    bl = 0.1 * torch.randn(768, generator=g)
    ml = FastLayerNorm(768, eps=1e-5, use_triton=False)
    ml.weight.copy_(wl); ml.bias.copy_(bl)
    put("ln_f32_x", xl); put("ln_f32_w", wl); put("ln_f32_b", bl); put("ln_f32_y", ml(xl))
    xlb = torch.randn(16, 320, generator=g).bfloat16()
    mlb = FastLayerNorm(320, elementwise_affine=False, use_triton=False)
    put("ln_bf16_x", xlb); put("ln_bf16_y", mlb(xlb))

    # --- fused residual + RMSNorm, bf16 (sum formed in fp32)
    xr = torch.randn(10, 512, generator=g).bfloat16()
    rr = torch.randn(10, 512, generator=g).bfloat16()
    wr = (1 + 0.05 * torch.randn(512, generator=g)).bfloat16()
    mr = FastFusedResidualRMSNorm(512, eps=1e-6, use_triton=False).bfloat16()
    mr.weight.copy_(wr)
    put("resrms_x", xr); put("resrms_r", rr); put("resrms_w", wr); put("resrms_y", mr(xr, rr))

    # --- RoPE: fp32 tables (built from an fp32 dummy) and bf16 tables (built from q)
    rope = FastRoPEPositionEmbedding(64, 2048, 10000.0, use_triton=False)
    q = torch.randn(2, 24, 4, 64, generator=g).bfloat16()
    k = torch.randn(2, 24, 2, 64, generator=g).bfloat16()
    cos32, sin32 = rope(torch.empty(0, dtype=torch.float32), seq_len=24)
    qo, ko = rope.apply_rotary_pos_emb(q, k, cos32, sin32)
    put("rope_q", q); put("rope_k", k); put("rope_cos_f32", cos32); put("rope_sin_f32", sin32)
    put("rope_qo_f32tab", qo); put("rope_ko_f32tab", ko)  # fp32 results (type promotion)
    cosb, sinb = rope(q, seq_len=24)
    qob, kob = rope.apply_rotary_pos_emb(q, k, cosb, sinb)
    put("rope_cos", cosb); put("rope_sin", sinb); put("rope_qo", qob); put("rope_ko", kob)

    # --- GLUs, bf16 and fp32
    xg = torch.randn(12, 2 * 96, generator=g) * 2.0
    for name, cls in (("swiglu", FastSwiGLU), ("geglu", FastGeGLU), ("reglu", FastReGLU)):
        mod = cls(96, use_triton=False)
        put(f"{name}_f32_x", xg); put(f"{name}_f32_y", mod(xg))
        put(f"{name}_x", xg.bfloat16()); put(f"{name}_y", mod(xg.bfloat16()))

    # --- ALiBi slopes
    for n in (8, 12, 32):
        put(f"alibi_slopes_{n}", FastALiBiPositionEmbedding(n, use_triton=False).slopes)
    put("alibi_bias_4_6", FastALiBiPositionEmbedding(4, use_triton=False)._compute_alibi_pytorch(6, 1))

    # --- attention core (FastBaseAttention._apply_pytorch_attention), fp32 and bf16
    B, S, H, Hkv, D = 2, 24, 4, 2, 32
    qa = torch.randn(B, S, H, D, generator=g)
    ka = torch.randn(B, S, Hkv, D, generator=g)
    va = torch.randn(B, S, Hkv, D, generator=g)
    gqa = FastGroupedQueryAttention(H * D, H, Hkv, bias=False, kernel_type="pytorch", causal=True)
    tile = lambda t: gqa._tile_kv_heads(t.transpose(1, 2), H // Hkv).transpose(1, 2)
    put("attn_q", qa); put("attn_k", ka); put("attn_v", va)
    for causal in (False, True):
        core = FastBaseAttention(H * D, H, kernel_type="pytorch", causal=causal)
        put(f"attn_out_causal{int(causal)}", core._apply_pytorch_attention(qa, tile(ka), tile(va)))
        put(f"attn_out_bf16_causal{int(causal)}",
            core._apply_pytorch_attention(qa.bfloat16(), tile(ka).bfloat16(), tile(va).bfloat16()))
    # causal + ALiBi bias passed as a 4-D additive mask
    alibi = FastALiBiPositionEmbedding(H, use_triton=False)
    bias = alibi._compute_alibi_pytorch(S, B)
    core = FastBaseAttention(H * D, H, kernel_type="pytorch", causal=True)
    put("attn_out_alibi", core._apply_pytorch_attention(qa, tile(ka), tile(va), bias.contiguous()))
    put("attn_tile_order", tile(torch.arange(Hkv).float().view(1, 1, Hkv, 1).expand(1, 1, Hkv, 1)))

    # --- whole GQA module (rope + causal), fp32, PyTorch backend
    torch.manual_seed(1)
    mod = FastGroupedQueryAttention(64, 4, 2, bias=False, kernel_type="pytorch", causal=True,
                                    position_method="rope", max_seq_len=64)
    xh = torch.randn(2, 16, 64, generator=g)
    put("gqa_x", xh)
    for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
        put(f"gqa_{n}", getattr(mod, n).weight)
    put("gqa_out", mod(xh)[0])

    # --- fused RMSNorm + activation (own generator: the vectors above keep their values)
    g2 = torch.Generator().manual_seed(2)
    xa = (torch.randn(9, 512, generator=g2) * 3).bfloat16()
    wa = (1 + 0.1 * torch.randn(512, generator=g2)).bfloat16()
    put("rmsact_x", xa); put("rmsact_w", wa)
    for act in ("mish", "quickgelu", "squared_relu"):
        ma = FastFusedRMSNormActivation(512, eps=1e-6, activation=act, use_triton=False).bfloat16()
        ma.weight.copy_(wa)
        put(f"rmsact_{act}_y", ma(xa))
        m32 = FastFusedRMSNormActivation(512, eps=1e-6, activation=act, use_triton=False)
        m32.weight.copy_(wa.float())
        put(f"rmsact_{act}_y_f32w", m32(xa))          # fp32 weight: product promoted to fp32
        put(f"rmsact_{act}_y_f32", m32(xa.float()))   # fp32 activations

    # --- fused residual + LayerNorm (own generator), bf16 / fp32 parameters / fp32 activations
    g3 = torch.Generator().manual_seed(3)
    xl2 = (torch.randn(11, 384, generator=g3) * 2 + 0.5).bfloat16()
    rl2 = torch.randn(11, 384, generator=g3).bfloat16()
    wl2 = (1 + 0.1 * torch.randn(384, generator=g3)).bfloat16()
    bl2 = (0.1 * torch.randn(384, generator=g3)).bfloat16()
    put("resln_x", xl2); put("resln_r", rl2); put("resln_w", wl2); put("resln_b", bl2)
    mlr = FastFusedResidualLayerNorm(384, eps=1e-5, use_triton=False).bfloat16()
    mlr.weight.copy_(wl2); mlr.bias.copy_(bl2)
    put("resln_y", mlr(xl2, rl2))
    mlr32 = FastFusedResidualLayerNorm(384, eps=1e-5, use_triton=False)
    mlr32.weight.copy_(wl2.float()); mlr32.bias.copy_(bl2.float())
    put("resln_y_f32w", mlr32(xl2, rl2))                   # fp32 parameters: promoted to fp32
    put("resln_y_f32", mlr32(xl2.float(), rl2.float()))    # fp32 activations

# --- gradients through the reference's PyTorch backend (own generator)
g4 = torch.Generator().manual_seed(4)


for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
    xg_ = torch.randn(12, 640, generator=g4).to(dt)
    dy_ = torch.randn(12, 640, generator=g4).to(dt)
    wg_ = (1 + 0.1 * torch.randn(640, generator=g4)).to(dt)
    bg_ = (0.1 * torch.randn(640, generator=g4)).to(dt)
    mr_ = FastRMSNorm(640, eps=1e-6, use_triton=False).to(dt)

    # the module's own forward, with its weight parameter as the leaf
    mr_.weight.data.copy_(wg_)
    xl_ = xg_.detach().clone().requires_grad_(True)
    out_ = mr_(xl_)
    dx_, dw_ = torch.autograd.grad(out_, [xl_, mr_.weight], dy_.to(out_.dtype))
    put(f"bwd_rms_{tag}_x", xg_); put(f"bwd_rms_{tag}_dy", dy_); put(f"bwd_rms_{tag}_w", wg_)
    put(f"bwd_rms_{tag}_dx", dx_); put(f"bwd_rms_{tag}_dw", dw_)

    ml_ = FastLayerNorm(640, eps=1e-5, use_triton=False).to(dt)
    ml_.weight.data.copy_(wg_); ml_.bias.data.copy_(bg_)
    xl_ = xg_.detach().clone().requires_grad_(True)
    out_ = ml_(xl_)
    dx_, dw_, db_ = torch.autograd.grad(out_, [xl_, ml_.weight, ml_.bias], dy_.to(out_.dtype))
    put(f"bwd_ln_{tag}_b", bg_)
    put(f"bwd_ln_{tag}_dx", dx_); put(f"bwd_ln_{tag}_dw", dw_); put(f"bwd_ln_{tag}_db", db_)

    xu_ = (torch.randn(10, 2 * 160, generator=g4) * 2).to(dt)
    dyu_ = torch.randn(10, 160, generator=g4).to(dt)
    put(f"bwd_glu_{tag}_x", xu_); put(f"bwd_glu_{tag}_dy", dyu_)
    for name, cls in (("swiglu", FastSwiGLU), ("geglu", FastGeGLU), ("reglu", FastReGLU)):
        xl_ = xu_.detach().clone().requires_grad_(True)
        out_ = cls(160, use_triton=False)(xl_)
        (dxu_,) = torch.autograd.grad(out_, [xl_], dyu_.to(out_.dtype))
        put(f"bwd_{name}_{tag}_dx", dxu_)

# RoPE: gradients of apply_rotary_pos_emb with respect to q and k (bf16 tables, built from q)
rope_b = FastRoPEPositionEmbedding(64, 2048, 10000.0, use_triton=False)
qb_ = torch.randn(2, 24, 4, 64, generator=g4).bfloat16()
kb_ = torch.randn(2, 24, 2, 64, generator=g4).bfloat16()
gq_ = torch.randn(2, 24, 4, 64, generator=g4).bfloat16()
gk_ = torch.randn(2, 24, 2, 64, generator=g4).bfloat16()
cosb_, sinb_ = rope_b(qb_, seq_len=24)
ql_ = qb_.detach().clone().requires_grad_(True)
kl_ = kb_.detach().clone().requires_grad_(True)
qo_, ko_ = rope_b.apply_rotary_pos_emb(ql_, kl_, cosb_, sinb_)
dq_, dk_ = torch.autograd.grad([qo_, ko_], [ql_, kl_], [gq_.to(qo_.dtype), gk_.to(ko_.dtype)])
put("bwd_rope_gq", gq_); put("bwd_rope_gk", gk_); put("bwd_rope_cos", cosb_); put("bwd_rope_sin", sinb_)
put("bwd_rope_dq", dq_); put("bwd_rope_dk", dk_)

np.savez_compressed(OUT, **vec)
print("wrote", OUT, os.path.getsize(OUT), "bytes;", len(vec), "arrays; trinix", trinix.__version__)
