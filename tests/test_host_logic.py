"""Host-side logic that needs no GPU: routing of the mirror modules, error behaviour of the
kernel classes on CPU tensors, batch sharding, and patching of an installed reference."""
import os
import sys
import warnings

import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from trinix_b200 import sharding
from tests.util import Golden, bf16_ulps, reference_path

G = Golden()
REFERENCE_DIR = reference_path() or ""
no_cuda = not torch.cuda.is_available()


def test_kernel_classes_report_unavailable_without_cuda():
    if no_cuda:
        for cls in T.kernels.KERNEL_CLASSES.values():
            assert cls.is_available() is False


def test_ops_reject_cpu_tensors_loudly():
    x = torch.randn(4, 64)
    with pytest.raises(ValueError):
        T.rmsnorm(x, torch.ones(64))
    with pytest.raises(ValueError):
        T.quantize_rowwise(x)
    with pytest.raises(ValueError):
        T.glu(x, "swiglu")
    q = torch.randn(1, 8, 2, 64)
    with pytest.raises(ValueError):
        T.triton_attn_func(q, q, q)  # same message class as the reference (CUDA only)
    with pytest.raises(ValueError):
        T.attention(q.bfloat16(), q.bfloat16(), q.bfloat16())


def test_mirror_modules_take_torch_path_on_cpu_and_match_oracle():
    x = G("rms_f32_x")
    m = T.FastRMSNorm(768, eps=1e-6)
    with torch.no_grad():
        m.weight.copy_(G("rms_f32_w"))
        torch.testing.assert_close(m(x), G("rms_f32_y"), rtol=2e-6, atol=2e-6)
        ln = T.FastLayerNorm(768, eps=1e-5)
        ln.weight.copy_(G("ln_f32_w")); ln.bias.copy_(G("ln_f32_b"))
        torch.testing.assert_close(ln(G("ln_f32_x")), G("ln_f32_y"), rtol=2e-6, atol=2e-6)
        fr = T.FastFusedResidualRMSNorm(512, eps=1e-6).bfloat16()
        fr.weight.copy_(G("resrms_w"))
        assert torch.equal(fr(G("resrms_x"), G("resrms_r")), G("resrms_y"))
        fl = T.FastFusedResidualLayerNorm(384, eps=1e-5).bfloat16()
        fl.weight.copy_(G("resln_w")); fl.bias.copy_(G("resln_b"))
        assert int(bf16_ulps(fl(G("resln_x"), G("resln_r")), G("resln_y")).max()) <= 1
        for name, cls in (("swiglu", T.FastSwiGLU), ("geglu", T.FastGeGLU), ("reglu", T.FastReGLU)):
            torch.testing.assert_close(cls(96)(G(f"{name}_f32_x")), G(f"{name}_f32_y"),
                                       rtol=2e-6, atol=2e-6)
        rope = T.FastRoPEPositionEmbedding(64, 2048, 10000.0)
        cos, sin = rope(torch.empty(0, dtype=torch.float32), seq_len=24)
        torch.testing.assert_close(cos, G("rope_cos_f32"), rtol=0, atol=1e-6)
        qo, ko = rope.apply_rotary_pos_emb(G("rope_q"), G("rope_k"), G("rope_cos_f32"),
                                           G("rope_sin_f32"))
        assert torch.equal(qo, G("rope_qo_f32tab")) and torch.equal(ko, G("rope_ko_f32tab"))
        for n in (8, 12, 32):
            torch.testing.assert_close(T.FastALiBiPositionEmbedding(n).slopes,
                                       G(f"alibi_slopes_{n}"), rtol=1e-7, atol=0)


def test_mirror_gqa_module_matches_reference_module_output():
    x = G("gqa_x")
    mod = T.FastGroupedQueryAttention(64, 4, 2, bias=False, kernel_type="triton", causal=True,
                                      position_method="rope", max_seq_len=64)
    with torch.no_grad():
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            getattr(mod, n).weight.copy_(G(f"gqa_{n}"))
        out, present = mod(x)
        assert present is None
        torch.testing.assert_close(out, G("gqa_out"), rtol=1e-5, atol=1e-6)
        # native-GQA routing (no K/V tiling) gives the same numbers on the torch path
        mod.tile_kv = False
        torch.testing.assert_close(mod(x)[0], G("gqa_out"), rtol=1e-5, atol=1e-6)


def test_mirror_sliding_window_and_alibi_cpu_paths_are_finite_and_match_oracle():
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 20, 4, 16, generator=g)
    k = torch.randn(1, 20, 2, 16, generator=g)
    v = torch.randn(1, 20, 2, 16, generator=g)
    base = T.FastBaseAttention(64, 4, kernel_type="pytorch", causal=True, use_sliding_window=True,
                               sliding_window_size=5)
    out = base.forward_attention(q, k, v)
    ref = R.attention_variant_ref(q, k, v, 16 ** -0.5, True, (5, 0))
    assert not torch.isnan(out).any()
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-6)
    ab = T.FastBaseAttention(64, 4, kernel_type="pytorch", causal=True, position_method="alibi")
    ref = R.attention_variant_ref(q, k, v, 16 ** -0.5, True, None, R.alibi_slopes_ref(4))
    torch.testing.assert_close(ab.forward_attention(q, k, v), ref, rtol=1e-5, atol=1e-6)


def test_module_error_behaviour_matches_reference():
    with pytest.raises(ValueError, match="last dimension"):
        T.FastRMSNorm(64)(torch.randn(2, 32))
    with pytest.raises(ValueError, match="even last dimension"):
        T.FastSwiGLU(8)(torch.randn(2, 7))
    with pytest.raises(ValueError):
        T.FastLayerNorm(64)(torch.randn(2, 32))
    with pytest.raises(AssertionError):
        T.FastGroupedQueryAttention(64, 4, 3)
    with pytest.raises(ValueError, match="CUDA"):  # a mask does not open a CPU path
        T.TritonAttentionKernel.apply(*([torch.zeros(1, 1, 1, 64)] * 3), attn_mask=torch.zeros(1, 1))
    with pytest.raises(ValueError, match="CUDA"):  # nor does dropout
        T.TritonAttentionKernel.apply(*([torch.zeros(1, 1, 1, 64)] * 3), dropout_p=0.1)


def test_shard_bounds_cover_everything_once():
    for n in (0, 1, 7, 16, 32768):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and b >= a
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_DIR, "trinix")),
                    reason="reference package not present on this machine")
def test_install_patches_the_reference_in_place():
    sys.path.insert(0, REFERENCE_DIR)
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            import trinix
            from trinix.kernels import TritonRMSNormKernel as RefRMS
            from trinix.layers.attention import base as ref_base
            from trinix.layers.norm.rmsnorm import FastRMSNorm as RefFastRMSNorm
        before = RefRMS.__dict__["apply"]
        T.install(strict=True)
        try:
            # the class object the layer module imported is the one that got rebound
            import trinix.layers.norm.rmsnorm as ref_mod
            assert ref_mod.TritonRMSNormKernel is RefRMS
            assert RefRMS.apply.__module__ == "trinix_b200.kernels"
            assert RefRMS.is_available() == T.TritonRMSNormKernel.is_available()
            assert ref_base.flash_attn_func is T.flash_attn_func
            assert ref_base.FLASH_ATTN_AVAILABLE and ref_base.TRITON_AVAILABLE
            import trinix.layers.attention.functional as ref_fn
            assert ref_fn.triton_attn_func is T.triton_attn_func
            # CPU tensors still take the reference's own torch path, unchanged results
            m = RefFastRMSNorm(768, eps=1e-6)
            with torch.no_grad():
                m.weight.copy_(G("rms_f32_w"))
                torch.testing.assert_close(m(G("rms_f32_x")), G("rms_f32_y"), rtol=2e-6, atol=2e-6)
            # the fused kernel classes live in trinix.kernels.fused and are rebound there
            from trinix.kernels.fused import (TritonFusedResidualLayerNormKernel as RefResLN,
                                              TritonFusedResidualRMSNormKernel as RefRes,
                                              TritonFusedRMSNormActivationKernel as RefAct)
            assert RefRes.apply.__module__ == "trinix_b200.kernels"
            assert RefResLN.apply.__module__ == "trinix_b200.kernels"
            assert RefAct.apply.__module__ == "trinix_b200.kernels"
            # the reference's own fuse() now knows the int8 pattern
            ref_fused = trinix.fuse(RefFastRMSNorm(4096), T.RowwiseInt8Quant())
            assert isinstance(ref_fused, T.FastFusedRMSNormInt8) and ref_fused.hidden_size == 4096
            # strict mode: the reference's silent-fallback warning is an error
            with pytest.raises(UserWarning):
                warnings.warn("Triton attention kernel failed: x, falling back to PyTorch")
        finally:
            T.uninstall()
        assert RefRMS.__dict__["apply"] is before
        import trinix.fusion as ref_fusion
        assert (RefFastRMSNorm, T.RowwiseInt8Quant) not in ref_fusion._FUSION_REGISTRY
    finally:
        sys.path.remove(REFERENCE_DIR)


def test_fuse_registry_mirrors_the_reference_contract():
    """fuse(norm, quant) finds the fused module and shares the norm's weight; an unknown chain
    warns and runs sequentially (trinix/fusion.py:31-77); fewer than two modules is an error."""
    import warnings
    import torch.nn as nn
    norm = T.FastRMSNorm(4096, eps=1e-5)
    fused = T.fuse(norm, T.RowwiseInt8Quant())
    assert isinstance(fused, T.FastFusedRMSNormInt8)
    assert fused.weight is norm.weight and fused.eps == 1e-5 and fused.hidden_size == 4096
    with pytest.raises(ValueError):
        T.fuse(norm)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        seq = T.fuse(norm, nn.Identity())
    assert isinstance(seq, nn.Sequential) and any("No fused kernel" in str(x.message) for x in w)
    with pytest.raises(ValueError, match="last dimension"):
        fused(torch.zeros(2, 8))
    with pytest.raises(ValueError, match="CUDA"):   # no CPU path behind the fused module
        fused(torch.zeros(2, 4096))
