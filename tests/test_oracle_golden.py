"""The CPU oracle against vectors produced by the reference itself (tests/golden/).

Same torch ops in the same order, so on the machine that generated the vectors the match is
bit-exact; the tolerances below only absorb differences between CPU vector units
(reduction order inside ATen kernels) on other hosts.
"""
import pytest
import torch

from oracle import reference_port as R
from tests.util import Golden, bf16_ulps

G = Golden()
F32_TOL = dict(rtol=2e-6, atol=2e-6)


def test_rmsnorm_fp32_baseline_config():
    y = R.rmsnorm_ref(G("rms_f32_x"), G("rms_f32_w"), 1e-6)
    torch.testing.assert_close(y, G("rms_f32_y"), **F32_TOL)


def test_rmsnorm_bf16():
    y = R.rmsnorm_ref(G("rms_bf16_x"), G("rms_bf16_w"), 1e-6)
    assert y.dtype == torch.bfloat16
    assert int(bf16_ulps(y, G("rms_bf16_y")).max()) <= 1


def test_rmsnorm_fp32_weight_promotes():
    y = R.rmsnorm_ref(G("rms_bf16_x"), G("rms_bf16_w").float(), 1e-6)
    assert y.dtype == torch.float32  # reference behaviour: weight * x.to(input_dtype)


def test_residual_rmsnorm():
    y = R.residual_rmsnorm_ref(G("resrms_x"), G("resrms_r"), G("resrms_w"), 1e-6)
    assert y.dtype == torch.bfloat16
    assert int(bf16_ulps(y, G("resrms_y")).max()) <= 1


def test_residual_layernorm():
    x, r, w, b = G("resln_x"), G("resln_r"), G("resln_w"), G("resln_b")
    y = R.residual_layernorm_ref(x, r, w, b, 1e-5)
    assert y.dtype == torch.bfloat16
    assert int(bf16_ulps(y, G("resln_y")).max()) <= 1
    y32w = R.residual_layernorm_ref(x, r, w.float(), b.float(), 1e-5)
    assert y32w.dtype == torch.float32  # reference behaviour: fp32 parameters promote
    torch.testing.assert_close(y32w, G("resln_y_f32w"), **F32_TOL)
    y32 = R.residual_layernorm_ref(x.float(), r.float(), w.float(), b.float(), 1e-5)
    torch.testing.assert_close(y32, G("resln_y_f32"), **F32_TOL)


@pytest.mark.parametrize("act", ["mish", "quickgelu", "squared_relu"])
def test_rmsnorm_activation(act):
    x, w = G("rmsact_x"), G("rmsact_w")
    y = R.rmsnorm_activation_ref(x, w, 1e-6, act)
    assert y.dtype == torch.bfloat16
    assert int(bf16_ulps(y, G(f"rmsact_{act}_y")).max()) <= 1
    # fp32 weight: the product stays in fp32 before the activation, the result is bf16 again
    y32w = R.rmsnorm_activation_ref(x, w.float(), 1e-6, act)
    assert y32w.dtype == torch.bfloat16
    assert int(bf16_ulps(y32w, G(f"rmsact_{act}_y_f32w")).max()) <= 1
    y32 = R.rmsnorm_activation_ref(x.float(), w.float(), 1e-6, act)
    torch.testing.assert_close(y32, G(f"rmsact_{act}_y_f32"), rtol=2e-6, atol=2e-6)


def test_layernorm():
    y = R.layernorm_ref(G("ln_f32_x"), G("ln_f32_w"), G("ln_f32_b"), 1e-5)
    torch.testing.assert_close(y, G("ln_f32_y"), **F32_TOL)
    yb = R.layernorm_ref(G("ln_bf16_x"), None, None, 1e-5)
    assert int(bf16_ulps(yb, G("ln_bf16_y")).max()) <= 1


def test_rope_tables_and_rotation():
    cos32, sin32 = R.rope_tables_ref(64, 24, 10000.0, torch.float32)
    torch.testing.assert_close(cos32, G("rope_cos_f32"), rtol=0, atol=1e-6)
    torch.testing.assert_close(sin32, G("rope_sin_f32"), rtol=0, atol=1e-6)
    qo, ko = R.rope_ref(G("rope_q"), G("rope_k"), G("rope_cos_f32"), G("rope_sin_f32"))
    assert qo.dtype == torch.float32
    assert torch.equal(qo, G("rope_qo_f32tab")) and torch.equal(ko, G("rope_ko_f32tab"))
    qb, kb = R.rope_ref(G("rope_q"), G("rope_k"), G("rope_cos"), G("rope_sin"))
    assert qb.dtype == torch.bfloat16
    assert torch.equal(qb, G("rope_qo")) and torch.equal(kb, G("rope_ko"))


@pytest.mark.parametrize("name,fn", [("swiglu", R.swiglu_ref), ("geglu", R.geglu_ref),
                                     ("reglu", R.reglu_ref)])
def test_glu(name, fn):
    torch.testing.assert_close(fn(G(f"{name}_f32_x")), G(f"{name}_f32_y"), **F32_TOL)
    assert int(bf16_ulps(fn(G(f"{name}_x")), G(f"{name}_y")).max()) <= 1


def test_alibi():
    for n in (8, 12, 32):
        torch.testing.assert_close(R.alibi_slopes_ref(n), G(f"alibi_slopes_{n}"), rtol=1e-7, atol=0)
    # the benchmark's closed form 2^(-8(i+1)/32) equals the reference's slopes for 32 heads
    closed = torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)])
    torch.testing.assert_close(R.alibi_slopes_ref(32), closed, rtol=1e-6, atol=0)
    b = R.alibi_bias_ref(R.alibi_slopes_ref(4), 6, 6).unsqueeze(0)
    torch.testing.assert_close(b, G("alibi_bias_4_6"), rtol=1e-7, atol=0)


def test_attention_core_and_kv_tiling():
    q, k, v = G("attn_q"), G("attn_k"), G("attn_v")
    order = R.tile_kv_heads_ref(torch.arange(2).float().view(1, 1, 2, 1), 2)
    assert torch.equal(order, G("attn_tile_order"))
    kt, vt = R.tile_kv_heads_ref(k, 2), R.tile_kv_heads_ref(v, 2)
    for causal in (False, True):
        out = R.attention_ref(q, kt, vt, None, causal)
        torch.testing.assert_close(out, G(f"attn_out_causal{int(causal)}"), rtol=1e-5, atol=1e-6)
        ob = R.attention_ref(q.bfloat16(), kt.bfloat16(), vt.bfloat16(), None, causal)
        assert int(bf16_ulps(ob.contiguous(), G(f"attn_out_bf16_causal{int(causal)}")).max()) <= 2
    out = R.attention_variant_ref(q, k, v, None, True, None, R.alibi_slopes_ref(4))
    torch.testing.assert_close(out, G("attn_out_alibi"), rtol=1e-5, atol=1e-6)


def test_window_mask_restatement():
    m = R.window_mask_ref(6, 6, 2, 0)
    for i in range(6):
        for j in range(6):
            visible = -2 <= j - i <= 0
            assert (m[i, j] == 0) == visible and (m[i, j] == float("-inf")) == (not visible)
    # window (L, 0) equals causal attention restricted to the last L+1 keys
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 9, 2, 8, generator=g) for _ in range(3))
    a = R.attention_variant_ref(q, k, v, None, False, (3, 0), None)
    b = R.attention_variant_ref(q, k, v, None, True, (3, 3), None)
    torch.testing.assert_close(a, b)
    assert not torch.isnan(a).any()


def test_gqa_module_composition():
    """decoder pieces composed like FastGroupedQueryAttention.forward (rope + causal)."""
    x = G("gqa_x")
    B, S, E = x.shape
    H, Hkv, D = 4, 2, E // 4
    import torch.nn.functional as F
    q = F.linear(x, G("gqa_q_proj")).view(B, S, H, D)
    k = F.linear(x, G("gqa_k_proj")).view(B, S, Hkv, D)
    v = F.linear(x, G("gqa_v_proj")).view(B, S, Hkv, D)
    cos, sin = R.rope_tables_ref(D, S, 10000.0, x.dtype)
    q, k = R.rope_ref(q, k, cos, sin)
    a = R.attention_variant_ref(q, k, v, D ** -0.5, True)
    out = F.linear(a.reshape(B, S, -1), G("gqa_o_proj"))
    torch.testing.assert_close(out, G("gqa_out"), rtol=1e-5, atol=1e-6)


def _close_grad(a, b, tag):
    """Gradient from the restated forward under autograd against the reference's own."""
    assert a.dtype == b.dtype and a.shape == b.shape
    if tag == "f32":
        torch.testing.assert_close(a, b, rtol=2e-5, atol=2e-6)
    else:  # same ops in the same order; a host's vector units may flip a last bit
        assert int(bf16_ulps(a, b).max()) <= 2


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_gradients_of_the_restated_forwards_match_the_reference(tag):
    x, dy, w, b = (G(f"bwd_rms_{tag}_x"), G(f"bwd_rms_{tag}_dy"), G(f"bwd_rms_{tag}_w"),
                   G(f"bwd_ln_{tag}_b"))
    dx, dw = R.autograd_ref(lambda a, ww: R.rmsnorm_ref(a, ww, 1e-6), [x, w], dy)
    _close_grad(dx, G(f"bwd_rms_{tag}_dx"), tag)
    _close_grad(dw, G(f"bwd_rms_{tag}_dw"), tag)
    # ATen's CPU layer-norm backward splits the rows over its threads and adds the per-thread
    # partial sums of dgamma / dbeta in the storage dtype, so in bf16 they depend on the thread
    # count; the vectors were generated on one thread
    threads = torch.get_num_threads()
    torch.set_num_threads(1)
    try:
        dx, dw, db = R.autograd_ref(lambda a, ww, bb: R.layernorm_ref(a, ww, bb, 1e-5),
                                    [x, w, b], dy)
    finally:
        torch.set_num_threads(threads)
    _close_grad(dx, G(f"bwd_ln_{tag}_dx"), tag)
    _close_grad(dw, G(f"bwd_ln_{tag}_dw"), tag)
    _close_grad(db, G(f"bwd_ln_{tag}_db"), tag)
    xg, dyg = G(f"bwd_glu_{tag}_x"), G(f"bwd_glu_{tag}_dy")
    for name, fn in (("swiglu", R.swiglu_ref), ("geglu", R.geglu_ref), ("reglu", R.reglu_ref)):
        (dxg,) = R.autograd_ref(fn, [xg], dyg)
        _close_grad(dxg, G(f"bwd_{name}_{tag}_dx"), tag)


def test_rope_gradient_is_the_inverse_rotation():
    cos, sin = G("bwd_rope_cos"), G("bwd_rope_sin")
    gq, gk = G("bwd_rope_gq"), G("bwd_rope_gk")
    q0, k0 = torch.zeros_like(gq), torch.zeros_like(gk)
    dq, dk, _, _ = R.autograd_ref(R.rope_ref, [q0, k0, cos, sin], (gq, gk))
    assert int(bf16_ulps(dq, G("bwd_rope_dq")).max()) <= 1
    assert int(bf16_ulps(dk, G("bwd_rope_dk")).max()) <= 1



def test_philox_known_answers_and_dropout_mask_shape():
    """The generator behind the attention dropout stream, against the three known-answer vectors
    its authors publish for Philox4x32 with 10 rounds, and the keep mask built from it."""
    import numpy as np
    kat = [((0, 0, 0, 0), (0, 0), "6627e8d5 e169c58d bc57ac4c 9b00dbd8"),
           ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, "408f276d 41c83b0e a20bc7c6 6d5451fd"),
           ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
            "d16cfe09 94fdcceb 5001e420 24126ea1")]
    for ctr, key, want in kat:
        out = R.philox4x32_10(np.array(ctr, dtype=np.uint32), key)
        assert " ".join("%08x" % int(v) for v in out) == want
    assert [R.dropout_threshold(p) for p in (0.0, 0.001, 0.1, 0.5, 0.999)] == [0, 1, 26, 128, 255]
    keep = R.dropout_keep_mask_ref(seed=1234, offset=7, B=2, H=3, Sq=40, Sk=50, dropout_p=0.25)
    assert keep.shape == (2, 3, 40, 50) and keep.dtype == torch.bool
    assert abs(float(keep.float().mean()) - 0.75) < 0.02
    # a pure function of its arguments: another offset gives another mask, the same one the same
    assert torch.equal(keep, R.dropout_keep_mask_ref(1234, 7, 2, 3, 40, 50, 0.25))
    assert not torch.equal(keep, R.dropout_keep_mask_ref(1234, 8, 2, 3, 40, 50, 0.25))
    # a longer key range extends the mask, it does not reshuffle it
    assert torch.equal(keep, R.dropout_keep_mask_ref(1234, 7, 2, 3, 40, 64, 0.25)[..., :50])
