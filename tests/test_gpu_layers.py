"""Drop-in behaviour on the GPU: the mirror modules (and, where it is installed, the patched
reference) reach the sm_100a kernels through the kernel classes, and a decoder layer built
from them matches the CPU oracle."""
import warnings

import pytest
import torch
import torch.nn.functional as F

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import rel_err

pytestmark = pytest.mark.gpu


def _spy(monkeypatch, cls):
    calls = []
    orig = cls.apply
    monkeypatch.setattr(cls, "apply", staticmethod(lambda *a, **k: (calls.append(1), orig(*a, **k))[1]))
    return calls


def test_modules_route_to_kernels_above_thresholds(cuda, monkeypatch):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 600, 4096, generator=g).bfloat16()
    rms_calls = _spy(monkeypatch, T.kernels.TritonRMSNormKernel)
    m = T.FastRMSNorm(4096).to(cuda).bfloat16()
    y = m(x.to(cuda))
    assert len(rms_calls) == 1 and y.dtype == torch.bfloat16
    assert rel_err(y.cpu(), R.rmsnorm_ref(x, torch.ones(4096).bfloat16(), 1e-6)) <= 1e-2
    small = T.FastRMSNorm(768).to(cuda)
    small(torch.randn(4, 768, device=cuda))
    assert len(rms_calls) == 1  # 768 <= 2048: the module's own torch path, as in the reference
    glu_calls = _spy(monkeypatch, T.kernels.TritonSwiGLUKernel)
    xg = torch.randn(3, 50, 2 * 11008, generator=g).bfloat16()
    yg = T.FastSwiGLU(11008)(xg.to(cuda))
    assert len(glu_calls) == 1 and rel_err(yg.cpu(), R.swiglu_ref(xg)) <= 1e-2
    ln_calls = _spy(monkeypatch, T.kernels.TritonLayerNormKernel)
    ln = T.FastLayerNorm(8192).to(cuda).bfloat16()
    xl = torch.randn(5, 8192, generator=g).bfloat16()
    yl = ln(xl.to(cuda))
    assert len(ln_calls) == 1
    assert rel_err(yl.cpu(), R.layernorm_ref(xl, torch.ones(8192), torch.zeros(8192), 1e-5)) <= 1e-2
    rope_calls = _spy(monkeypatch, T.kernels.TritonRoPEKernel)
    rope = T.FastRoPEPositionEmbedding(128, 2048).to(cuda)
    q = torch.randn(1, 600, 32, 128, generator=g).bfloat16().to(cuda)
    k = torch.randn(1, 600, 8, 128, generator=g).bfloat16().to(cuda)
    cos, sin = rope(q, 600)
    rope.apply_rotary_pos_emb(q, k, cos, sin)
    assert len(rope_calls) == 1
    rope.apply_rotary_pos_emb(q[:, :100], k[:, :100], cos[:100], sin[:100])
    assert len(rope_calls) == 1  # S <= 512 stays on torch, as in the reference


def test_autograd_contract(cuda):
    """Norms, GLUs and RoPE are differentiable through the backward kernels; attention is forward
    only (as in the reference) and says so instead of silently producing no gradient."""
    m = T.FastRMSNorm(4096).to(cuda).bfloat16()
    x = torch.randn(4, 4096, device=cuda, dtype=torch.bfloat16)
    y = m(x)  # weight requires grad and grad mode is on
    y.float().sum().backward()
    assert m.weight.grad is not None and m.weight.grad.shape == (4096,)
    with torch.no_grad():
        assert m(x).grad_fn is None
    q = torch.randn(1, 128, 2, 128, device=cuda, dtype=torch.bfloat16, requires_grad=True)
    with pytest.raises(NotImplementedError):
        T.TritonAttentionKernel.apply(q, q, q, causal=True).float().sum().backward()


def _layer_weights(E, Hq, Hkv, FF, seed=0):
    g = torch.Generator().manual_seed(seed)
    D = E // Hq
    shapes = {"wq": (E, E), "wk": (Hkv * D, E), "wv": (Hkv * D, E), "wo": (E, E),
              "w_gate": (FF, E), "w_up": (FF, E), "w_down": (E, FF)}
    return {n: 0.02 * torch.randn(*s, generator=g) for n, s in shapes.items()}


@pytest.mark.parametrize("kernel_type,tile_kv", [("triton", True), ("flash", False)])
def test_decoder_layer_int8_weights_matches_oracle(cuda, kernel_type, tile_kv):
    """Llama-shaped pre-norm layer (scaled down in width only where the dispatch thresholds
    allow): RMSNorm -> GQA(rope, causal) -> residual -> RMSNorm -> SwiGLU MLP -> residual,
    projection weights stored as per-row int8 and dequantised to bf16 by the kernel."""
    E, Hq, Hkv, FF, B, S = 4096, 32, 8, 1024, 2, 640
    w = _layer_weights(E, Hq, Hkv, FF)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, S, E, generator=g).bfloat16()
    # int8 weight store: quantise on the GPU, check against the oracle, dequantise on the GPU
    dq = {}
    for n, t in w.items():
        codes, scales = T.quantize_rowwise(t.bfloat16().to(cuda))
        rc, rs = R.quantize_rowwise_ref(t.bfloat16())
        assert torch.equal(codes.cpu(), rc) and torch.equal(scales.cpu(), rs)
        dq[n] = T.dequantize_rowwise(codes, scales, torch.bfloat16)
        assert torch.equal(dq[n].cpu(), R.dequantize_rowwise_ref(rc, rs, torch.bfloat16))
    attn = T.FastGroupedQueryAttention(E, Hq, Hkv, bias=False, kernel_type=kernel_type,
                                       causal=True, position_method="rope", max_seq_len=2048,
                                       tile_kv=tile_kv).to(cuda).bfloat16()
    n1, n2 = T.FastRMSNorm(E).to(cuda).bfloat16(), T.FastRMSNorm(E).to(cuda).bfloat16()
    act = T.FastSwiGLU(FF)
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("error")  # any fallback warning is a failure
        for n, p in (("wq", attn.q_proj), ("wk", attn.k_proj), ("wv", attn.v_proj), ("wo", attn.o_proj)):
            p.weight.copy_(dq[n])
        xd = x.to(cuda)
        h = xd + attn(n1(xd))[0]
        nn2 = n2(h)
        ff = act(torch.cat([F.linear(nn2, dq["w_up"]), F.linear(nn2, dq["w_gate"])], dim=-1))
        y = h + F.linear(ff, dq["w_down"])
    assert T.attention_status(cuda) == 0
    p = {n: t.cpu() for n, t in dq.items()}
    p["attn_norm"] = torch.ones(E).bfloat16()
    p["ffn_norm"] = torch.ones(E).bfloat16()
    ref = R.decoder_layer_ref(x, p, Hq, Hkv)
    assert y.dtype == torch.bfloat16 and y.shape == ref.shape
    # Both pipelines round every GEMM / norm / attention output to bf16 but accumulate in
    # different orders, so they are compared through the exact (fp32) evaluation of the same
    # layer: the kernel path must be as close to it as the reference's bf16 path is.
    exact = R.decoder_layer_ref(x.float(), {n: t.float() for n, t in p.items()}, Hq, Hkv)
    e_ref = (ref.float() - exact).abs()
    e_gpu = (y.float().cpu() - exact).abs()
    assert float(e_gpu.max()) <= 2.0 * float(e_ref.max()) + 1e-2
    assert float(e_gpu.mean()) <= 1.5 * float(e_ref.mean()) + 1e-4
    assert rel_err(y.cpu(), ref, floor_frac=1.0) <= 1e-1


def test_fused_rmsnorm_int8_module_equals_the_two_modules(cuda):
    """fuse(FastRMSNorm, RowwiseInt8Quant) runs one kernel and returns exactly what the two
    modules return one after the other."""
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(3, 50, 4096, generator=g) * 2).bfloat16().to(cuda)
    norm = T.FastRMSNorm(4096, eps=1e-6).to(cuda).bfloat16()
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(4096, generator=g))
    fused = T.fuse(norm, T.RowwiseInt8Quant())
    before = T.ops.launch_count
    codes, scales = fused(x)
    assert T.ops.launch_count == before + 1
    codes2, scales2 = T.RowwiseInt8Quant()(norm(x))
    assert torch.equal(codes, codes2) and torch.equal(scales, scales2)
    assert codes.shape == x.shape and scales.shape == x.shape[:-1]
