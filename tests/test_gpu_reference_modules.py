"""The drop-in claim itself, on a GPU: the UNCHANGED module classes of the reference package,
after `trinix_b200.install(strict=True)`, reach the sm_100a kernels and match the CPU oracle.

The reference is imported from $TRINIX_REFERENCE or from the untracked install under
baseline/_ref (python -m pip install --no-index --no-deps --target baseline/_ref <reference>).
Each attention test records what the reference's module hands to the kernel boundary — the
tensors that reach `trinix_b200.ops.attention` — because that is where the reference's own
habits show: K/V tiled to all query heads as transposed non-contiguous views
(grouped_query_attention.py:189-194), a dense ALiBi bias merged into the mask AND the slopes
(:201 + base.py:415-417), a sliding-window mask that is NaN wherever a key is visible
(base.py:222-237) next to window_size=(w, w) (base.py:419-421).
"""
import sys
import warnings

import pytest
import torch
import torch.nn.functional as F

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import reference_path, rel_err
from trinix_b200.decoder import params_to_bf16

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture()
def ref(cuda):
    """The reference package with its kernel classes routed to this backend (strict: the
    reference's silent fallback warning is an error)."""
    path = reference_path()
    if path is None:
        pytest.skip("reference package not present (set TRINIX_REFERENCE or install it under "
                    "baseline/_ref)")
    sys.path.insert(0, path)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import trinix
    T.install(strict=True)
    try:
        yield trinix
    finally:
        T.uninstall()
        sys.path.remove(path)


@pytest.fixture()
def seen(monkeypatch):
    """Every call that crosses into ops.attention: shapes, strides, mask and flags."""
    calls = []
    orig = T.ops.attention

    def spy(q, k, v, **kw):
        m = kw.get("attn_mask")
        calls.append({"q": tuple(q.shape), "k": tuple(k.shape), "k_stride": tuple(k.stride()),
                      "k_contiguous": k.is_contiguous(), "mask_shape": None if m is None else tuple(m.shape),
                      "mask_dtype": None if m is None else m.dtype,
                      "mask_nan": None if m is None else bool(torch.isnan(m).any()),
                      "slopes": kw.get("alibi_slopes") is not None,
                      "window": kw.get("window"), "causal": kw.get("causal")})
        return orig(q, k, v, **kw)

    monkeypatch.setattr(T.ops, "attention", spy)
    return calls


def test_reference_norm_glu_rope_modules_run_these_kernels(cuda, ref):
    before = T.ops.launch_count
    x = torch.randn(8, 4096, device=cuda, dtype=torch.bfloat16)
    m = ref.FastRMSNorm(4096).to(cuda).bfloat16()
    assert rel_err(m(x).cpu(), R.rmsnorm_ref(x.cpu(), torch.ones(4096).bfloat16(), 1e-6)) <= 1e-2
    xg = torch.randn(8, 2048, device=cuda, dtype=torch.bfloat16)
    assert rel_err(ref.FastSwiGLU(1024)(xg).cpu(), R.swiglu_ref(xg.cpu())) <= 1e-2
    assert rel_err(ref.FastGeGLU(1024)(xg).cpu(), R.geglu_ref(xg.cpu())) <= 1e-2
    from trinix.layers.activation.reglu import FastReGLU  # not re-exported at the top level
    assert rel_err(FastReGLU(1024)(xg).cpu(), R.reglu_ref(xg.cpu())) <= 1e-2
    ln = ref.FastLayerNorm(8192).to(cuda).bfloat16()
    xl = torch.randn(5, 8192, device=cuda, dtype=torch.bfloat16)
    assert rel_err(ln(xl).cpu(), R.layernorm_ref(xl.cpu(), torch.ones(8192), torch.zeros(8192), 1e-5)) <= 1e-2
    rope = ref.FastRoPEPositionEmbedding(128, 2048).to(cuda)
    q = torch.randn(1, 600, 32, 128, device=cuda, dtype=torch.bfloat16)
    k = torch.randn(1, 600, 8, 128, device=cuda, dtype=torch.bfloat16)
    cos, sin = rope(q, 600)
    qo, ko = rope.apply_rotary_pos_emb(q, k, cos, sin)
    rq, rk = R.rope_ref(q.cpu(), k.cpu(), cos.cpu(), sin.cpu())
    assert torch.equal(qo.cpu(), rq.to(qo.dtype)) and torch.equal(ko.cpu(), rk.to(ko.dtype))
    assert T.ops.launch_count - before == 6  # one kernel of this library per module call


def _gqa_oracle(x, w, Hq, Hkv, mask=None, causal=True, rope=True):
    """The reference's FastGroupedQueryAttention.forward (grouped_query_attention.py:147-207)
    through its PyTorch backend, restated with the oracle's pieces."""
    B, S, E = x.shape
    D = E // Hq
    q = F.linear(x, w["wq"]).view(B, S, Hq, D)
    k = F.linear(x, w["wk"]).view(B, S, Hkv, D)
    v = F.linear(x, w["wv"]).view(B, S, Hkv, D)
    if rope:
        cos, sin = R.rope_tables_ref(D, S, 10000.0, dtype=x.dtype)
        q, k = R.rope_ref(q, k, cos, sin)
    g = Hq // Hkv
    a = R.attention_ref(q, R.tile_kv_heads_ref(k, g), R.tile_kv_heads_ref(v, g), D ** -0.5, causal,
                        mask)
    return F.linear(a.reshape(B, S, -1), w["wo"])


def _load(attn, w, dev):
    with torch.no_grad():
        for n, p in (("wq", attn.q_proj), ("wk", attn.k_proj), ("wv", attn.v_proj),
                     ("wo", attn.o_proj)):
            p.weight.copy_(w[n].to(dev))


def _weights(E, Hq, Hkv, seed=0):
    g = torch.Generator().manual_seed(seed)
    D = E // Hq
    return {n: (0.02 * torch.randn(*s, generator=g)).bfloat16()
            for n, s in (("wq", (E, E)), ("wk", (Hkv * D, E)), ("wv", (Hkv * D, E)), ("wo", (E, E)))}


def _judge(y, x, w, Hq, Hkv, **kw):
    """Against the bf16 oracle through the exact (fp32) evaluation, as the layer tests do."""
    ref = _gqa_oracle(x, w, Hq, Hkv, **kw)  # an fp32 mask is added in place to bf16 scores
    exact = _gqa_oracle(x.float(), {n: t.float() for n, t in w.items()}, Hq, Hkv, **kw)
    e_ref, e_gpu = (ref.float() - exact).abs(), (y.float().cpu() - exact).abs()
    assert float(e_gpu.max()) <= 2.0 * float(e_ref.max()) + 1e-2
    assert float(e_gpu.mean()) <= 1.5 * float(e_ref.mean()) + 1e-4


def test_reference_gqa_module_rope_causal_at_the_layer_shape(cuda, ref, seen):
    """FastGroupedQueryAttention(4096, 32, 8, kernel_type='triton', causal, rope) of the
    reference on one sequence [1, 2048, 4096]: what reaches the kernel are K/V already tiled to
    32 heads, as transposed non-contiguous views, and no mask."""
    E, Hq, Hkv, S = 4096, 32, 8, 2048
    # parameters in bf16, buffers left in fp32: module.bfloat16() would also down-cast inv_freq,
    # and the reference's tables (rope.py:69-79) would then be built from bf16 positions
    assert ref.FastRoPEPositionEmbedding(128).bfloat16().inv_freq.dtype == torch.bfloat16
    attn = params_to_bf16(ref.FastGroupedQueryAttention(
        E, Hq, Hkv, bias=False, kernel_type="triton", causal=True, position_method="rope",
        max_seq_len=S).to(cuda))
    assert attn.position_embedding.inv_freq.dtype == torch.float32
    w = _weights(E, Hq, Hkv)
    _load(attn, w, cuda)
    x = torch.randn(1, S, E, generator=torch.Generator().manual_seed(1)).bfloat16()
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("error")  # the reference's fallback warning fails the test
        y = attn(x.to(cuda))[0]
    assert T.attention_status(cuda) == 0
    assert len(seen) == 1
    c = seen[0]
    assert c["q"] == (1, S, Hq, 128) and c["k"] == (1, S, Hq, 128)      # tiled to 32 heads
    assert not c["k_contiguous"] and c["k_stride"] == (Hq * S * 128, 128, S * 128, 1)
    assert c["mask_shape"] is None and c["causal"] is True and c["window"] is None
    _judge(y, x, w, Hq, Hkv)


def test_reference_gqa_module_alibi_reaches_the_kernel_as_mask_plus_slopes(cuda, ref, seen):
    """position_method='alibi': the reference's module merges the dense bias into the mask
    (grouped_query_attention.py:201) and its kernel path passes the slopes as well
    (base.py:415-417), so its own Triton kernel would add the bias twice
    (attention_kernel.py:385-388 on top of the mask). The drop-in computes exactly what it is
    handed — mask + slopes — i.e. the oracle's attention with twice the bias. The dense-bias
    module is asked for its torch path (use_triton_embeddings=False): the reference's dense
    ALiBi kernel is not part of this backend."""
    E, Hq, Hkv, S = 1024, 8, 2, 1024
    attn = params_to_bf16(ref.FastGroupedQueryAttention(
        E, Hq, Hkv, bias=False, kernel_type="triton", causal=True, position_method="alibi",
        max_seq_len=S, use_triton_embeddings=False).to(cuda))
    assert attn.position_embedding.slopes.dtype == torch.float32
    w = _weights(E, Hq, Hkv, seed=2)
    _load(attn, w, cuda)
    x = torch.randn(2, S, E, generator=torch.Generator().manual_seed(3)).bfloat16()
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("error")
        y = attn(x.to(cuda))[0]
    assert T.attention_status(cuda) == 0
    c = seen[0]
    assert c["mask_shape"] == (2, Hq, S, S) and c["mask_dtype"] == torch.float32
    assert c["slopes"] and c["mask_nan"] is False
    bias = R.alibi_bias_ref(R.alibi_slopes_ref(Hq), S, S)                    # (H, S, S)
    twice = (2.0 * bias).unsqueeze(0).expand(2, -1, -1, -1)
    _judge(y, x, w, Hq, Hkv, mask=twice, rope=False)


def test_reference_gqa_module_sliding_window_hands_over_a_nan_mask(cuda, ref, seen):
    """use_sliding_window=True: the reference builds (1 - window_mask) * -inf, which is NaN
    wherever a key is visible (base.py:232), and passes window_size=(w, w) beside it even when
    causal (base.py:419-421). Its own PyTorch backend returns NaN for every element on that
    mask; the drop-in, computing what it is handed, returns the same. The working form of the
    window is the functional API's window_size and this package's mirror module, which never
    build that mask."""
    E, Hq, Hkv, S, W = 1024, 8, 2, 600, 128
    attn = ref.FastGroupedQueryAttention(E, Hq, Hkv, bias=False, kernel_type="triton", causal=True,
                                         position_method="none", use_sliding_window=True,
                                         sliding_window_size=W).to(cuda).bfloat16()
    w = _weights(E, Hq, Hkv, seed=4)
    _load(attn, w, cuda)
    x = torch.randn(1, S, E, generator=torch.Generator().manual_seed(5)).bfloat16()
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("error")
        y = attn(x.to(cuda))[0]
    torch.cuda.synchronize()
    c = seen[0]
    assert c["mask_shape"] == (S, S) and c["mask_nan"] is True
    assert c["window"] == (W, W) and c["causal"] is True
    assert T.attention_status(cuda) == 0
    # the reference's own PyTorch backend on the mask it built: NaN everywhere
    attn_cpu = ref.FastGroupedQueryAttention(E, Hq, Hkv, bias=False, kernel_type="pytorch",
                                             causal=True, position_method="none",
                                             use_sliding_window=True, sliding_window_size=W)
    _load(attn_cpu, {n: t.float() for n, t in w.items()}, "cpu")
    with torch.no_grad():
        y_ref = attn_cpu(x.float())[0]
    assert torch.isnan(y_ref).all() and torch.isnan(y).all()
    # the same module options through this package's mirror: finite, and equal to the oracle
    mirror = T.FastGroupedQueryAttention(E, Hq, Hkv, bias=False, kernel_type="triton", causal=True,
                                         position_method="none", use_sliding_window=True,
                                         sliding_window_size=W).to(cuda).bfloat16()
    _load(mirror, w, cuda)
    with torch.no_grad():
        ym = mirror(x.to(cuda))[0]
    _judge(ym, x, w, Hq, Hkv, mask=R.window_mask_ref(S, S, W, 0), rope=False)


def test_reference_modules_compose_the_benchmark_layer(cuda, ref):
    """The cfg5 layer built from the REFERENCE's module classes (FastRMSNorm,
    FastGroupedQueryAttention, FastSwiGLU) over this backend, int8 weight store, one sequence,
    FFN 11008, against the oracle's layer."""
    from trinix_b200.decoder import Int8DecoderLayer, random_layer_weights
    E, Hq, Hkv, FF, S = 4096, 32, 8, 11008, 1024
    layer = Int8DecoderLayer(E, Hq, Hkv, FF, random_layer_weights(E, Hq, Hkv, FF, cuda, seed=7),
                             max_seq_len=S, modules=ref)
    assert type(layer.attn).__module__.startswith("trinix.")
    x = torch.randn(1, S, E, generator=torch.Generator().manual_seed(8)).bfloat16()
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        y = layer.forward_modules(x.to(cuda))
    assert T.attention_status(cuda) == 0
    p = layer.reference_weights()
    ref_y = R.decoder_layer_ref(x, p, Hq, Hkv)
    exact = R.decoder_layer_ref(x.float(), {n: t.float() for n, t in p.items()}, Hq, Hkv)
    e_ref, e_gpu = (ref_y.float() - exact).abs(), (y.float().cpu() - exact).abs()
    assert float(e_gpu.max()) <= 2.0 * float(e_ref.max()) + 1e-2
    assert float(e_gpu.mean()) <= 1.5 * float(e_ref.mean()) + 1e-4
