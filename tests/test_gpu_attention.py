"""Parity of the tcgen05 attention kernel with the CPU oracle (the reference's PyTorch
attention), through triton_attn_func / the C ABI. Tolerance from the project baseline:
2e-2 max abs error in bf16."""
import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import Golden

pytestmark = pytest.mark.gpu
G = Golden()
TOL = 2e-2


def _qkv(B, Sq, Sk, Hq, Hk, D, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, Sk, Hk, D, generator=g).to(dtype)
    v = torch.randn(B, Sk, Hk, D, generator=g).to(dtype)
    return q, k, v


def _check(cuda, q, k, v, causal=False, window=None, slopes=None, scale=None, tol=TOL):
    out = T.triton_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), softmax_scale=scale,
                             causal=causal, window_size=window,
                             alibi_slopes=None if slopes is None else slopes.to(cuda))
    assert T.attention_status(cuda) == 0, "a bounded wait inside the kernel gave up"
    assert out.shape == q.shape and out.dtype == q.dtype
    # the oracle in the kernel's input dtype (what the reference computes) and in fp32 (truth)
    ref = R.attention_variant_ref(q, k, v, scale, causal, window, slopes).float()
    ref32 = R.attention_variant_ref(q.float(), k.float(), v.float(), scale, causal, window,
                                    None if slopes is None else slopes.float())
    o = out.float().cpu()
    assert not torch.isnan(o).any()
    err, err32 = float((o - ref).abs().max()), float((o - ref32).abs().max())
    # The 16-bit oracle rounds scores and probabilities to the input dtype (base.py:373,394),
    # so it sits up to `oracle_noise` away from the exact result itself; the kernel must be
    # within tol of the exact result and within tol + that noise of the 16-bit oracle.
    oracle_noise = float((ref - ref32).abs().max())
    assert err32 <= tol and err <= tol + oracle_noise, (err, err32, oracle_noise)
    return out


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("S", [128, 256, 384, 1000])
def test_noncausal_mha(cuda, S, D):
    q, k, v = _qkv(1, S, S, 2, 2, D, seed=S + D)
    _check(cuda, q, k, v)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("S", [64, 129, 512, 777, 1536])
def test_causal_gqa(cuda, S, D):
    q, k, v = _qkv(2, S, S, 8, 2, D, seed=S)
    _check(cuda, q, k, v, causal=True)


def test_causal_mqa_with_expanded_kv_heads(cuda):
    """MQA as the reference's module presents it: one kv head expanded to all query heads
    (head stride 0), multi_query_attention.py:173-174."""
    q, k, v = _qkv(2, 300, 300, 4, 1, 128, seed=7)
    ref = R.attention_variant_ref(q, k, v, None, True).float()
    kd, vd = k.to("cuda").expand(-1, -1, 4, -1), v.to("cuda").expand(-1, -1, 4, -1)
    assert kd.stride(2) == 0
    out = T.triton_attn_func(q.to("cuda"), kd, vd, causal=True)
    assert T.attention_status() == 0
    assert float((out.float().cpu() - ref).abs().max()) <= TOL
    out1 = T.triton_attn_func(q.to("cuda"), k.to("cuda"), v.to("cuda"), causal=True)
    assert torch.equal(out, out1)  # native Hkv=1 and the expanded view are the same launch


def test_tiled_noncontiguous_kv_like_the_reference_module(cuda):
    """K/V tiled to all heads and handed over as transposed (B,S,H,D) views, the layout
    grouped_query_attention.py:189-194 produces."""
    q, k, v = _qkv(2, 260, 260, 8, 2, 128, seed=11)
    kt = R.tile_kv_heads_ref(k, 4).to("cuda").transpose(1, 2).contiguous().transpose(1, 2)
    vt = R.tile_kv_heads_ref(v, 4).to("cuda").transpose(1, 2).contiguous().transpose(1, 2)
    assert not kt.is_contiguous()
    out = T.triton_attn_func(q.to("cuda"), kt, vt, causal=True)
    native = T.triton_attn_func(q.to("cuda"), k.to("cuda"), v.to("cuda"), causal=True)
    assert T.attention_status() == 0
    assert torch.equal(out, native)


@pytest.mark.parametrize("S", [200, 1024])
def test_causal_alibi(cuda, S):
    H = 8
    q, k, v = _qkv(1, S, S, H, 2, 128, seed=S)
    slopes = R.alibi_slopes_ref(H)
    _check(cuda, q, k, v, causal=True, slopes=slopes)
    _check(cuda, q, k, v, causal=False, slopes=slopes)  # |i-j| on both sides


@pytest.mark.parametrize("Sq,Sk,causal,window", [
    (1300, 1300, True, None),          # many KV tiles, both Q tiles of a CTA, ragged tail
    (900, 900, False, (300, 0)),       # a window that ends at the query, no causal flag
    (1100, 1100, True, (200, 0)),      # causal and a left window: two boundary tiles per row block
    (130, 130, True, None),            # second Q tile nearly empty
    (256, 640, True, None),            # more keys than queries (top-left aligned mask)
])
def test_alibi_with_keys_visited_backwards(cuda, Sq, Sk, causal, window):
    """ALiBi under a causal mask, or a window that ends at the query, walks a row block's KV tiles
    from the last to the first; slopes from steep (an O rescale per tile in ascending order) to
    flat, grouped kv heads, head dims 128 and 64."""
    for D, H, Hk in ((128, 8, 2), (64, 4, 4)):
        q, k, v = _qkv(2, Sq, Sk, H, Hk, D, seed=Sq + D)
        slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / H) for i in range(H)])
        slopes[0] = 1.5  # steeper than any standard ALiBi head
        _check(cuda, q, k, v, causal=causal, window=window, slopes=slopes)


@pytest.mark.parametrize("S,window", [(700, (100, 0)), (1300, (256, 0)), (600, (64, 64)),
                                      (512, (0, 0)), (900, (1024, 0)), (520, (130, 7))])
def test_sliding_window(cuda, S, window):
    q, k, v = _qkv(1, S, S, 4, 2, 128, seed=S)
    _check(cuda, q, k, v, window=window)
    _check(cuda, q, k, v, causal=True, window=(window[0], max(window)))


def test_window_zero_zero_returns_v(cuda):
    q, k, v = _qkv(1, 300, 300, 2, 2, 64, seed=1)
    out = T.triton_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), window_size=(0, 0))
    assert torch.equal(out.cpu(), v)  # softmax over a single key is exactly 1


def test_cross_lengths_scale_and_fp16(cuda):
    q, k, v = _qkv(2, 200, 333, 4, 4, 128, seed=3)
    _check(cuda, q, k, v, scale=0.05)
    q, k, v = _qkv(1, 130, 70, 2, 1, 64, seed=4, dtype=torch.float16)
    _check(cuda, q, k, v, tol=5e-3)
    q, k, v = _qkv(1, 260, 130, 2, 1, 128, seed=5)
    _check(cuda, q, k, v, causal=True)  # rows beyond the key count see every key


def test_large_logits_trigger_rescale(cuda):
    """Row maxima that keep growing along the keys force the O-rescale path."""
    g = torch.Generator().manual_seed(0)
    S, D = 1024, 128
    q = torch.randn(1, S, 1, D, generator=g)
    k = torch.randn(1, S, 1, D, generator=g) * torch.linspace(0.2, 3.0, S).view(1, S, 1, 1)
    v = torch.randn(1, S, 1, D, generator=g)
    _check(cuda, q.bfloat16(), k.bfloat16(), v.bfloat16(), scale=0.5, tol=3e-2)


def test_lse_output(cuda):
    q, k, v = _qkv(1, 300, 300, 2, 2, 128, seed=2)
    out, lse = T.attention(q.to(cuda), k.to(cuda), v.to(cuda), causal=True, return_lse=True)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * 128 ** -0.5
    s = s.masked_fill(torch.triu(torch.ones(300, 300), 1).bool(), float("-inf"))
    torch.testing.assert_close(lse.cpu(), torch.logsumexp(s, -1), rtol=1e-3, atol=1e-3)


def test_golden_attention_vectors_from_the_reference(cuda):
    """The attention outputs the unmodified reference produced (its PyTorch backend, fp32 and
    bf16, head dim 32, GQA 4:2, causal / not / causal + ALiBi): the kernel meets them directly.
    Head dim 32 runs as 64 with zero columns appended."""
    q, k, v = (G(n).bfloat16().to(cuda) for n in ("attn_q", "attn_k", "attn_v"))
    for causal in (False, True):
        out = T.triton_attn_func(q, k, v, causal=causal)
        assert out.shape == q.shape
        want_bf16 = G(f"attn_out_bf16_causal{int(causal)}").float()
        want_f32 = G(f"attn_out_causal{int(causal)}")     # from the fp32 inputs
        assert float((out.float().cpu() - want_bf16).abs().max()) <= TOL
        assert float((out.float().cpu() - want_f32).abs().max()) <= 2 * TOL  # + input rounding
    out = T.triton_attn_func(q, k, v, causal=True, alibi_slopes=R.alibi_slopes_ref(4).to(cuda))
    assert float((out.float().cpu() - G("attn_out_alibi")).abs().max()) <= 2 * TOL
    assert T.attention_status(cuda) == 0
    # head dims between the two built ones, and the one beyond them
    g = torch.Generator().manual_seed(3)
    q96 = torch.randn(1, 200, 4, 96, generator=g).bfloat16()
    k96 = torch.randn(1, 200, 2, 96, generator=g).bfloat16()
    v96 = torch.randn(1, 200, 2, 96, generator=g).bfloat16()
    out96, lse96 = T.attention(q96.to(cuda), k96.to(cuda), v96.to(cuda), causal=True, return_lse=True)
    ref96 = R.attention_variant_ref(q96.float(), k96.float(), v96.float(), None, True)
    assert out96.shape == q96.shape and lse96.shape == (1, 4, 200)
    assert float((out96.float().cpu() - ref96).abs().max()) <= TOL
    q256 = torch.zeros(1, 128, 2, 256, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(T._lib.TrinixB200Error) as e:     # a clear error, no fallback
        T.triton_attn_func(q256, q256, q256)
    assert e.value.code == -6


def test_full_size_properties(cuda):
    """Benchmark geometry (S=4096, 32 query / 8 kv heads, D=128), one batch element:
    causal output row 0 equals v[0]; batch sharding is bit-identical; window (S, 0) == causal."""
    g = torch.Generator(device=cuda).manual_seed(0)
    B, S, H, Hk, D = 2, 4096, 32, 8, 128
    q = torch.randn(B, S, H, D, generator=g, device=cuda).bfloat16()
    k = torch.randn(B, S, Hk, D, generator=g, device=cuda).bfloat16()
    v = torch.randn(B, S, Hk, D, generator=g, device=cuda).bfloat16()
    out = T.triton_attn_func(q, k, v, causal=True)
    assert T.attention_status(cuda) == 0
    assert torch.equal(out[:, 0], v[:, 0].repeat_interleave(4, dim=1))
    parts = torch.cat([T.triton_attn_func(q[b:b + 1], k[b:b + 1], v[b:b + 1], causal=True)
                       for b in range(B)])
    assert torch.equal(out, parts)
    w = T.triton_attn_func(q, k, v, window_size=(S, 0))
    assert torch.equal(out, w)
    # against torch's own fused attention on the GPU (a library used as checker only)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(4, 1),
        v.transpose(1, 2).repeat_interleave(4, 1), is_causal=True).transpose(1, 2)
    assert float((out.float() - ref.float()).abs().max()) <= TOL


def _mask_ref(q, k, v, mask4, causal, scale=None):
    """The reference's PyTorch attention (base.py:347-400) with K/V tiled to all query heads
    and the mask expanded to (B, H, Sq, Sk), in the input dtype and in fp32."""
    g = q.shape[2] // k.shape[2]
    kt, vt = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
    B, Sq, H, _ = q.shape
    m = mask4.expand(B, H, Sq, k.shape[1]).float()
    ref = R.attention_ref(q, kt, vt, scale, causal, m.to(q.dtype)).float()
    ref32 = R.attention_ref(q.float(), kt.float(), vt.float(), scale, causal, m)
    return ref, ref32


@pytest.mark.parametrize("mask_kind", ["2d_f32", "3d_bool", "4d_b1", "4d_bh_bf16"])
@pytest.mark.parametrize("Sq,Sk,D", [(300, 300, 128), (257, 640, 64)])
def test_dense_additive_mask(cuda, mask_kind, Sq, Sk, D):
    """attn_mask in every shape _prepare_mask accepts (attention_kernel.py:479-495), float and
    bool, broadcast by stride: parity with the reference's PyTorch path on the expanded mask."""
    B, Hq, Hk = 2, 4, 2
    q, k, v = _qkv(B, Sq, Sk, Hq, Hk, D, seed=Sq + Sk)
    g = torch.Generator().manual_seed(7)
    if mask_kind == "2d_f32":
        mask = torch.randn(Sq, Sk, generator=g)
        mask[:, Sk // 3: Sk // 2] = float("-inf")          # a hidden band
        mask4 = mask[None, None]
    elif mask_kind == "3d_bool":
        hidden = torch.rand(B, Sq, Sk, generator=g) < 0.3
        hidden[..., 0] = False                              # no fully hidden row
        mask = hidden
        mask4 = torch.zeros(B, 1, Sq, Sk).masked_fill_(hidden[:, None], float("-inf"))
    elif mask_kind == "4d_b1":
        mask = torch.randn(B, 1, Sq, Sk, generator=g) * 2
        mask4 = mask
    else:
        mask = (torch.randn(B, Hq, Sq, Sk, generator=g) * 2).bfloat16()
        mask4 = mask.float()
    out = T.triton_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), attn_mask=mask.to(cuda))
    assert T.attention_status(cuda) == 0
    ref, ref32 = _mask_ref(q, k, v, mask4, False)
    o = out.float().cpu()
    assert not torch.isnan(o).any()
    err, err32 = float((o - ref).abs().max()), float((o - ref32).abs().max())
    noise = float((ref - ref32).abs().max())
    assert err32 <= TOL and err <= TOL + noise, (err, err32, noise)


def test_dense_mask_combines_with_causal_and_alibi(cuda):
    B, S, Hq, Hk, D = 1, 400, 4, 1, 128
    q, k, v = _qkv(B, S, S, Hq, Hk, D, seed=11)
    g = torch.Generator().manual_seed(3)
    mask = torch.randn(S, S, generator=g)
    slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625])
    out = T.triton_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), attn_mask=mask.to(cuda),
                             causal=True, alibi_slopes=slopes.to(cuda))
    assert T.attention_status(cuda) == 0
    i = torch.arange(S)
    alibi = -slopes[:, None, None] * (i[:, None] - i[None, :]).abs().float()   # (H, S, S)
    ref, ref32 = _mask_ref(q, k, v, (mask[None] + alibi)[None], True)
    o = out.float().cpu()
    err, err32 = float((o - ref).abs().max()), float((o - ref32).abs().max())
    noise = float((ref - ref32).abs().max())
    assert err32 <= TOL and err <= TOL + noise, (err, err32, noise)


@pytest.mark.parametrize("p_drop", [0.1, 0.5])
@pytest.mark.parametrize("Sq,Sk,D,causal,with_mask", [(300, 300, 128, True, False),
                                                      (257, 640, 64, False, True)])
def test_dropout_matches_the_rebuilt_keep_mask(cuda, p_drop, Sq, Sk, D, causal, with_mask):
    """dropout_p > 0: the kernel's Philox stream is rebuilt on the CPU element for element, so the
    comparison with the reference's PyTorch arithmetic (softmax, then dropout, then times V,
    base.py:394-397) is exact up to the usual tolerance, not statistical."""
    B, Hq, Hk = 2, 4, 2
    q, k, v = _qkv(B, Sq, Sk, Hq, Hk, D, seed=Sq + Sk + int(100 * p_drop))
    mask = None
    if with_mask:
        mask = torch.randn(B, 1, Sq, Sk, generator=torch.Generator().manual_seed(5))
    seed, offset = 0x1234_5678_9ABC_DEF0 >> 2, 3
    out, lse = T.attention(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal,
                           attn_mask=None if mask is None else mask.to(cuda), dropout_p=p_drop,
                           seed=seed, offset=offset, return_lse=True)
    assert T.attention_status(cuda) == 0
    keep = R.dropout_keep_mask_ref(seed, offset, B, Hq, Sq, Sk, p_drop)
    g = Hq // Hk
    kt, vt = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
    m4 = None if mask is None else mask.expand(B, Hq, Sq, Sk).contiguous()
    ref32 = R.attention_dropout_ref(q.float(), kt.float(), vt.float(), None, causal, m4, keep, p_drop)
    ref = R.attention_dropout_ref(q, kt, vt, None, causal,
                                  None if m4 is None else m4.to(q.dtype), keep, p_drop).float()
    o = out.float().cpu()
    err32, err = float((o - ref32).abs().max()), float((o - ref).abs().max())
    noise = float((ref - ref32).abs().max())
    tol = TOL / (1.0 - p_drop)  # kept probabilities are scaled up by 1 / (1 - p)
    assert err32 <= tol and err <= tol + noise, (err32, err, noise)
    # the LSE is that of the undropped scores (another instantiation of the kernel computes it
    # here, with its own rounding of the score arithmetic: close, not bit-equal)
    _, lse0 = T.attention(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal,
                          attn_mask=None if mask is None else mask.to(cuda), return_lse=True)
    torch.testing.assert_close(lse, lse0, rtol=1e-5, atol=1e-5)
    # same seed and offset: the same result bit for bit; another offset: another mask
    again = T.attention(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal,
                        attn_mask=None if mask is None else mask.to(cuda), dropout_p=p_drop,
                        seed=seed, offset=offset)
    other = T.attention(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal,
                        attn_mask=None if mask is None else mask.to(cuda), dropout_p=p_drop,
                        seed=seed, offset=offset + 1)
    assert torch.equal(again, out) and not torch.equal(other, out)


def test_dropout_keep_rate_and_module_path(cuda):
    """Statistics of the stream (v = 1 makes the output the kept mass of each row), and the
    module surface: training mode drops, eval mode does not, the seed follows torch.manual_seed."""
    B, S, H, D = 1, 2048, 2, 64
    q = torch.zeros(B, S, H, D, dtype=torch.bfloat16, device=cuda)       # uniform probabilities
    v = torch.ones(B, S, H, D, dtype=torch.bfloat16, device=cuda)
    for p_drop in (0.1, 0.5):
        out = T.attention(q, q, v, dropout_p=p_drop, seed=99)
        thr = R.dropout_threshold(p_drop)
        # every row: sum_j keep_j / (S * (1 - p_eff)), mean 1, std sqrt(p / ((1 - p) S))
        m = out.float()[..., 0]
        assert abs(float(m.mean()) - 1.0) < 5e-3
        p_eff = thr / 256.0
        assert abs(float(m.std()) - (p_eff / ((1 - p_eff) * S)) ** 0.5) < 5e-3
    attn = T.FastGroupedQueryAttention(512, 8, 2, dropout=0.3, bias=False, kernel_type="triton",
                                       causal=True).to(cuda).bfloat16()
    x = torch.randn(2, 256, 512, device=cuda, dtype=torch.bfloat16)
    with torch.no_grad():
        attn.eval()
        e1, e2 = attn(x)[0], attn(x)[0]
        attn.train()
        torch.manual_seed(5)
        t1 = attn(x)[0]
        t2 = attn(x)[0]
        torch.manual_seed(5)
        t3 = attn(x)[0]
    assert torch.equal(e1, e2) and not torch.equal(t1, e1)
    assert not torch.equal(t1, t2) and torch.equal(t1, t3)
    assert T.attention_status(cuda) == 0
    with pytest.raises(ValueError):
        T.attention(q, q, v, dropout_p=1.0)


def test_dense_mask_rejects_bad_shapes(cuda):
    q, k, v = (t.to(cuda) for t in _qkv(2, 128, 128, 2, 2, 64))
    with pytest.raises(ValueError):
        T.triton_attn_func(q, k, v, attn_mask=torch.zeros(128, 64, device=cuda))
    with pytest.raises(ValueError):
        T.triton_attn_func(q, k, v, attn_mask=torch.zeros(3, 128, 128, device=cuda))
    with pytest.raises(ValueError):
        T.triton_attn_func(q, k, v, attn_mask=torch.zeros(1, 1, 1, 128, 128, device=cuda))


def test_launch_after_recorded_failure_raises_then_recovers(cuda):
    """A non-zero status word (a bounded wait gave up in some earlier launch) makes every later
    launch skip its work on the device. The host learns of it without a synchronisation: every
    attention call queues a 4-byte copy of the word into pinned memory and the next call checks
    that copy first, raising status -8 instead of handing back unwritten output. The word is set
    from the host here; no wait on the device is ever made to run out."""
    from trinix_b200 import ops
    q, k, v = (t.to(cuda) for t in _qkv(1, 512, 512, 4, 2, 128, seed=21))
    good = T.attention(q, k, v, causal=True)
    assert T.attention_status(cuda) == 0
    ops._workspace(cuda)[:4].view(torch.int32).fill_(4)     # as if a softmax wait had run out
    T.attention(q, k, v, causal=True)                        # skipped on the device; copy queued
    torch.cuda.synchronize(cuda)
    with pytest.raises(T._lib.TrinixB200Error) as e:         # first call that can know: raises
        T.attention(q, k, v, causal=True)
    assert e.value.code == -8 and "0x4" in str(e.value)
    again = T.attention(q, k, v, causal=True)                # both copies were cleared
    assert T.attention_status(cuda) == 0
    assert torch.equal(again, good)
    # the C-level form of the same check
    import ctypes
    lib = T._lib.load()
    host = torch.zeros(1, dtype=torch.int32).pin_memory()
    ws = ops._workspace(cuda)
    P = ctypes.c_void_p
    st = P(torch.cuda.current_stream(cuda).cuda_stream)
    ws[:4].view(torch.int32).fill_(2)
    assert lib.trx_attn_status(P(ws.data_ptr()), P(host.data_ptr()), st) == 0
    torch.cuda.synchronize(cuda)
    assert int(host[0]) == 2
    assert lib.trx_attn_status(P(ws.data_ptr()), P(host.data_ptr()), st) == -8
    assert lib.trx_attn_status(None, P(host.data_ptr()), st) == -1
    assert T.attention_status(cuda) == 2 and T.attention_status(cuda) == 0


def test_views_the_tensor_maps_cannot_take_are_materialised(cuda):
    """Legal strided views whose base is not 16-byte aligned or whose strides are not multiples
    of 8 elements (a slice along D at an offset of 4, a head stride of 132) run all the same."""
    g = torch.Generator().manual_seed(5)
    big = torch.randn(2, 200, 4, 136, generator=g).bfloat16().to(cuda)
    q, k, v = big[..., 4:132], big[..., 4:132].clone(), big[..., 8:136]
    assert q.data_ptr() % 16 != 0 and q.stride(-1) == 1
    out = T.triton_attn_func(q, k, v, causal=True)
    ref = T.triton_attn_func(q.contiguous(), k, v.contiguous(), causal=True)
    assert T.attention_status(cuda) == 0 and torch.equal(out, ref)
    odd = torch.randn(1, 150, 2, 132, generator=g).bfloat16().to(cuda)[..., :128]
    assert odd.stride(2) % 8 != 0
    out = T.triton_attn_func(odd, odd, odd)
    assert torch.equal(out, T.triton_attn_func(*(odd.contiguous(),) * 3))


def test_flash_stand_in_keeps_the_conventions_of_the_symbol_it_replaces(cuda):
    """flash_attn_func (the symbol bound at trinix/layers/attention/base.py:10-16): causal with
    Sq < Sk is aligned bottom-right (decode against a KV cache sees every cached key), unknown
    keywords raise instead of being dropped."""
    Sq, Sk = 70, 300
    q, k, v = _qkv(2, Sq, Sk, 4, 2, 128, seed=9)
    out = T.flash_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), causal=True)
    assert T.attention_status(cuda) == 0
    i, j = torch.arange(Sq)[:, None], torch.arange(Sk)[None, :]
    mask = torch.zeros(Sq, Sk).masked_fill_(j > i + (Sk - Sq), float("-inf"))
    kt, vt = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    ref32 = R.attention_ref(q.float(), kt.float(), vt.float(), None, False, mask)
    assert float((out.float().cpu() - ref32).abs().max()) <= TOL
    # one query row against the cache: sees all keys
    out1 = T.flash_attn_func(q[:, :1].to(cuda), k.to(cuda), v.to(cuda), causal=True)
    full = T.triton_attn_func(q[:, :1].to(cuda), k.to(cuda), v.to(cuda), causal=False)
    assert torch.equal(out1, full)
    # equal lengths: identical to triton_attn_func
    q2, k2, v2 = (t.to(cuda) for t in _qkv(1, 200, 200, 4, 4, 64, seed=2))
    assert torch.equal(T.flash_attn_func(q2, k2, v2, causal=True),
                       T.triton_attn_func(q2, k2, v2, causal=True))
    assert torch.equal(T.flash_attn_func(q2, k2, v2, window_size=(50, 0)),
                       T.triton_attn_func(q2, k2, v2, window_size=(50, 0)))
    with pytest.raises(TypeError):
        T.flash_attn_func(q2, k2, v2, softcap=30.0)
    with pytest.raises(NotImplementedError):
        T.flash_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), causal=True, window_size=(10, 0))


@pytest.mark.parametrize("Sq,Sk", [(1, 1000), (1, 128), (7, 2049), (130, 64)])
def test_decode_shapes_kv_longer_or_shorter_than_q(cuda, Sq, Sk):
    """KV-cache decode shapes (grouped_query_attention.py:179-187 concatenates past keys, so
    Sk > Sq, down to a single query row), GQA heads, no mask."""
    q, k, v = _qkv(2, Sq, Sk, 8, 2, 128, seed=Sq * 7 + Sk)
    _check(cuda, q, k, v)
