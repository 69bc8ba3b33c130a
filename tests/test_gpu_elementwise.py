"""Parity of the streaming kernels (GLUs, RoPE) with the CPU oracle, through the C ABI."""
import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import Golden, bf16_ulps, rel_err

pytestmark = pytest.mark.gpu
G = Golden()
GLU = {"swiglu": (T.TritonSwiGLUKernel, R.swiglu_ref), "geglu": (T.TritonGeGLUKernel, R.geglu_ref),
       "reglu": (T.TritonReGLUKernel, R.reglu_ref)}


@pytest.mark.parametrize("name", list(GLU))
def test_glu_golden(cuda, name):
    kern, _ = GLU[name]
    y = kern.apply(G(f"{name}_f32_x").to(cuda)).cpu()
    torch.testing.assert_close(y, G(f"{name}_f32_y"), rtol=2e-5, atol=2e-6)
    yb = kern.apply(G(f"{name}_x").to(cuda)).cpu()
    assert rel_err(yb, G(f"{name}_y")) <= 1e-2


@pytest.mark.parametrize("name", list(GLU))
@pytest.mark.parametrize("shape", [(1, 16), (3, 2 * 100), (2, 5, 2 * 11008), (7, 2 * 1021),
                                   (1030, 2 * 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_glu_shapes(cuda, name, shape, dtype):
    kern, ref = GLU[name]
    g = torch.Generator().manual_seed(len(shape) + shape[-1])
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    x.view(-1)[:4] = torch.tensor([-100.0, 100.0, 0.0, -20.0]).to(dtype)  # saturation, no NaN
    y = kern.apply(x.to(cuda)).cpu()
    r = ref(x)
    assert y.shape == r.shape and y.dtype == dtype
    assert not torch.isnan(y.float()).any()
    # fp32: tanh-GELU cancels (1 + tanh) for negative gates, so a few 1e-7 of absolute
    # difference between the two tanh implementations is all that can be asked there
    f32_tol = 2e-4 if name == "geglu" else 2e-5
    assert rel_err(y, r) <= (f32_tol if dtype == torch.float32 else 1e-2)
    if dtype == torch.bfloat16:
        # same rounding order as the oracle: where the output is not vanishingly small (tanh
        # GELU cancels to ~0 for very negative gates) results are at most 1 bf16 ulp apart
        d = bf16_ulps(y, r)
        big = r.float().abs() >= 1e-2 * float(r.float().pow(2).mean().sqrt())
        assert int(d[big].max()) <= 1 and float((d[big] > 0).float().mean()) < 5e-3


def test_glu_separate_pointers_match_concatenated(cuda):
    g = torch.Generator().manual_seed(0)
    gate = torch.randn(4, 64, 11008, generator=g).bfloat16().to(cuda)
    up = torch.randn(4, 64, 11008, generator=g).bfloat16().to(cuda)
    a = T.glu_pair(up, gate, "swiglu")
    b = T.glu(torch.cat([up, gate], dim=-1), "swiglu")  # gate is the SECOND half
    assert torch.equal(a, b)
    ref = R.swiglu_ref(torch.cat([up, gate], dim=-1).cpu())
    assert rel_err(a.cpu(), ref) <= 1e-2


def test_rope_golden_bit_exact(cuda):
    q, k = G("rope_q").to(cuda), G("rope_k").to(cuda)
    # fp32 tables: the oracle's result is fp32 (type promotion); the kernel rounds it once
    qo, ko = T.TritonRoPEKernel.apply(q, k, G("rope_cos_f32").to(cuda), G("rope_sin_f32").to(cuda))
    assert torch.equal(qo.cpu(), G("rope_qo_f32tab").bfloat16())
    assert torch.equal(ko.cpu(), G("rope_ko_f32tab").bfloat16())
    # tables in the activation dtype (what the reference's attention modules pass)
    qo, ko = T.TritonRoPEKernel.apply(q, k, G("rope_cos").to(cuda), G("rope_sin").to(cuda))
    assert torch.equal(qo.cpu(), G("rope_qo")) and torch.equal(ko.cpu(), G("rope_ko"))


@pytest.mark.parametrize("B,S,Hq,Hk,D", [(2, 600, 32, 8, 128), (1, 7, 3, 1, 64), (2, 33, 5, 5, 32),
                                         (1, 5, 2, 2, 6), (1, 2048, 4, 1, 128)])
@pytest.mark.parametrize("dtype,table", [(torch.bfloat16, torch.float32),
                                         (torch.bfloat16, torch.bfloat16),
                                         (torch.float16, torch.float16),
                                         (torch.float32, torch.float32)])
def test_rope_shapes(cuda, B, S, Hq, Hk, D, dtype, table):
    g = torch.Generator().manual_seed(S + D)
    q = torch.randn(B, S, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, S, Hk, D, generator=g).to(dtype)
    cos, sin = R.rope_tables_ref(D, S, 10000.0, table)
    rq, rk = R.rope_ref(q, k, cos, sin)
    qo, ko = T.rope(q.to(cuda), k.to(cuda), cos.to(cuda), sin.to(cuda))
    assert qo.dtype == dtype and qo.shape == q.shape and ko.shape == k.shape
    if dtype == torch.float32:
        assert torch.equal(qo.cpu(), rq) and torch.equal(ko.cpu(), rk)
    else:
        assert torch.equal(qo.cpu(), rq.to(dtype)) and torch.equal(ko.cpu(), rk.to(dtype))
    # inverse rotation restores the input up to rounding
    if table == torch.float32:
        qb, kb = T.rope(qo, ko, cos.to(cuda), sin.to(cuda), inverse=True)
        assert rel_err(qb.cpu(), q, floor_frac=1.0) <= (1e-5 if dtype == torch.float32 else 2e-2)


def test_rope_strided_views_from_fused_qkv(cuda):
    """q/k taken as views of one fused projection output (non-contiguous head stride)."""
    g = torch.Generator().manual_seed(1)
    B, S, H, D = 2, 520, 8, 128
    qkv = torch.randn(B, S, 3, H, D, generator=g).bfloat16()
    q, k, _ = qkv.unbind(2)
    cos, sin = R.rope_tables_ref(D, S, 10000.0, torch.float32)
    rq, rk = R.rope_ref(q, k, cos, sin)
    dq, dk, _ = qkv.to(cuda).unbind(2)
    assert not dq.is_contiguous()
    qo, ko = T.rope(dq, dk, cos.to(cuda), sin.to(cuda))
    assert torch.equal(qo.cpu(), rq.bfloat16()) and torch.equal(ko.cpu(), rk.bfloat16())


def test_empty_inputs_every_op(cuda):
    """Zero rows / tokens / queries: every entry point returns an empty result of the right
    shape and dtype without launching anything."""
    from trinix_b200 import ops
    w = torch.ones(4096, device=cuda, dtype=torch.bfloat16)
    x0 = torch.empty(0, 4096, device=cuda, dtype=torch.bfloat16)
    before = ops.launch_count
    assert T.ops.rmsnorm(x0, w, 1e-6).shape == (0, 4096)
    assert T.ops.layernorm(x0, w, w, 1e-5).shape == (0, 4096)
    c, s = T.quantize_rowwise(x0)
    assert c.shape == (0, 4096) and c.dtype == torch.int8 and s.shape == (0,)
    assert T.dequantize_rowwise(c, s, torch.bfloat16).shape == (0, 4096)
    c, s = T.rmsnorm_quantize(x0, w, 1e-6)
    assert c.shape == (0, 4096) and s.shape == (0,)
    y, h = T.ops.residual_rmsnorm(x0, x0, w, 1e-6, return_sum=True)
    assert y.shape == (0, 4096) and h.shape == (0, 4096)
    y, h = T.ops.residual_layernorm(x0, x0, w, w, 1e-5, return_sum=True)
    assert y.shape == (0, 4096) and h.shape == (0, 4096)
    assert T.ops.glu(torch.empty(0, 2 * 512, device=cuda, dtype=torch.bfloat16), "swiglu").shape == (0, 512)
    q0 = torch.empty(0, 16, 4, 128, device=cuda, dtype=torch.bfloat16)
    cos = torch.ones(16, 128, device=cuda)
    qo, ko = T.ops.rope(q0, q0, cos, cos)
    assert qo.shape == q0.shape and ko.shape == q0.shape
    assert T.attention(q0, q0, q0, causal=True).shape == q0.shape
    qz = torch.empty(2, 0, 4, 128, device=cuda, dtype=torch.bfloat16)      # no queries
    kz = torch.randn(2, 64, 4, 128, device=cuda).bfloat16()
    assert T.attention(qz, kz, kz).shape == qz.shape
    torch.cuda.synchronize(cuda)
    assert T.attention_status(cuda) == 0
    # no keys at all: every row's softmax is empty, the output is defined as 0
    qn = torch.randn(1, 130, 2, 128, device=cuda).bfloat16()
    kn = torch.empty(1, 0, 2, 128, device=cuda, dtype=torch.bfloat16)
    out = T.attention(qn, kn, kn)
    assert out.shape == qn.shape and float(out.float().abs().max()) == 0.0
    assert ops.launch_count >= before
