"""Parity at the benchmark configurations themselves: the shapes, head counts, slopes, window
and layer width that the benchmark times, compared with the CPU oracle (the reference's PyTorch
arithmetic) — one sequence of the batch at a time where the oracle's O(S^2) score tensor would
not fit otherwise — plus bit-identity of the full-batch launch with per-sequence launches."""
import json

import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import bf16_ulps, rel_err
from trinix_b200.decoder import Int8DecoderLayer, random_layer_weights

pytestmark = pytest.mark.gpu
TOL = 2e-2  # attention: max abs error in bf16

S4, HQ, HKV, D = 4096, 32, 8, 128
CFG4_SLOPES = torch.tensor([2.0 ** (-8.0 * (i + 1) / 32) for i in range(32)])
CFG4_VARIANTS = {
    "causal": dict(causal=True, window=None, slopes=None),
    "causal_alibi": dict(causal=True, window=None, slopes=CFG4_SLOPES),
    "window_1024_0": dict(causal=False, window=(1024, 0), slopes=None),
}


def _report(capsys, name, **facts):
    """One line per measured worst case, shown even when output is captured."""
    with capsys.disabled():
        print("\n[parity] " + name + " " + json.dumps(facts))


@pytest.mark.parametrize("variant", list(CFG4_VARIANTS))
def test_cfg4_attention_one_sequence_vs_oracle(cuda, capsys, variant):
    """q [1,4096,32,128], k/v [1,4096,8,128] bf16, scale 1/sqrt(128): causal; causal + ALiBi
    slopes 2^(-8(i+1)/32); window (1024, 0). The oracle runs eight query heads (two kv heads) at
    a time, in bf16 (what the reference computes) and on fp32 copies (the exact result)."""
    cfg = CFG4_VARIANTS[variant]
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, S4, HQ, D, generator=g).bfloat16()
    k = torch.randn(1, S4, HKV, D, generator=g).bfloat16()
    v = torch.randn(1, S4, HKV, D, generator=g).bfloat16()
    out = T.triton_attn_func(q.to(cuda), k.to(cuda), v.to(cuda), softmax_scale=D ** -0.5,
                             causal=cfg["causal"], window_size=cfg["window"],
                             alibi_slopes=None if cfg["slopes"] is None else cfg["slopes"].to(cuda))
    assert T.attention_status(cuda) == 0
    o = out.float().cpu()
    assert not torch.isnan(o).any()
    worst, worst32, noise_max = 0.0, 0.0, 0.0
    for h0 in range(0, HQ, 8):
        qs, ks, vs = q[:, :, h0:h0 + 8], k[:, :, h0 // 4:h0 // 4 + 2], v[:, :, h0 // 4:h0 // 4 + 2]
        sl = None if cfg["slopes"] is None else cfg["slopes"][h0:h0 + 8]
        ref = R.attention_variant_ref(qs, ks, vs, D ** -0.5, cfg["causal"], cfg["window"], sl).float()
        ref32 = R.attention_variant_ref(qs.float(), ks.float(), vs.float(), D ** -0.5,
                                        cfg["causal"], cfg["window"], sl)
        err = float((o[:, :, h0:h0 + 8] - ref).abs().max())
        err32 = float((o[:, :, h0:h0 + 8] - ref32).abs().max())
        noise = float((ref - ref32).abs().max())  # the bf16 oracle's own distance from exact
        assert err32 <= TOL and err <= TOL + noise, (variant, h0, err, err32, noise)
        worst, worst32, noise_max = max(worst, err), max(worst32, err32), max(noise_max, noise)
    _report(capsys, f"cfg4 {variant} [1,4096,32/8,128]", max_abs_vs_bf16_oracle=round(worst, 5),
            max_abs_vs_fp32_oracle=round(worst32, 5), bf16_oracle_vs_fp32_oracle=round(noise_max, 5))


def test_cfg4_batch16_launch_equals_sixteen_single_launches(cuda):
    """The benchmark's launch, q [16,4096,32,128]: every variant is bit-identical to sixteen
    launches of one sequence each (what a batch shard of one sequence per GPU computes)."""
    g = torch.Generator(device=cuda).manual_seed(0)
    q = torch.randn(16, S4, HQ, D, generator=g, device=cuda, dtype=torch.float32).bfloat16()
    k = torch.randn(16, S4, HKV, D, generator=g, device=cuda, dtype=torch.float32).bfloat16()
    v = torch.randn(16, S4, HKV, D, generator=g, device=cuda, dtype=torch.float32).bfloat16()
    for cfg in CFG4_VARIANTS.values():
        kw = dict(softmax_scale=D ** -0.5, causal=cfg["causal"], window_size=cfg["window"],
                  alibi_slopes=None if cfg["slopes"] is None else cfg["slopes"].to(cuda))
        full = T.triton_attn_func(q, k, v, **kw)
        for b in range(16):
            one = T.triton_attn_func(q[b:b + 1], k[b:b + 1], v[b:b + 1], **kw)
            assert torch.equal(full[b:b + 1], one), b
        del full
    assert T.attention_status(cuda) == 0


def test_cfg5_decoder_layer_one_sequence_both_compositions_vs_oracle(cuda, capsys):
    """The layer of the benchmark at full width: hidden 4096, 32 / 8 heads, FFN 11008, int8
    weight store, one sequence [1, 2048, 4096]. Both the module composition (two norms, K/V
    tiled, separate up / gate GEMMs) and the graph the benchmark times (native GQA heads, one
    up/gate GEMM, residual adds fused) against the oracle's layer in bf16; both pipelines round
    every GEMM / norm / attention output to bf16 with different accumulation orders, so they are
    judged through the exact (fp32) evaluation of the same layer."""
    E, FF, S = 4096, 11008, 2048
    w = random_layer_weights(E, HQ, HKV, FF, cuda, seed=0)
    layer = Int8DecoderLayer(E, HQ, HKV, FF, w, max_seq_len=S)
    # the int8 store itself is bit-exact against the oracle's quantiser
    for n in ("wq", "w_down"):
        rc, rs = R.quantize_rowwise_ref(w[n].bfloat16().cpu())
        assert torch.equal(layer.store[n][0].cpu(), rc) and torch.equal(layer.store[n][1].cpu(), rs)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, S, E, generator=g).bfloat16()
    p = layer.reference_weights()
    ref = R.decoder_layer_ref(x, p, HQ, HKV)
    exact = R.decoder_layer_ref(x.float(), {n: t.float() for n, t in p.items()}, HQ, HKV)
    e_ref = (ref.float() - exact).abs()
    y_mod = layer.forward_modules(x.to(cuda))
    y_fused = layer.forward_fused(x.to(cuda))
    assert T.attention_status(cuda) == 0
    for name, y in (("modules", y_mod), ("fused", y_fused)):
        assert y.dtype == torch.bfloat16 and y.shape == ref.shape
        e_gpu = (y.float().cpu() - exact).abs()
        assert float(e_gpu.max()) <= 2.0 * float(e_ref.max()) + 1e-2, name
        assert float(e_gpu.mean()) <= 1.5 * float(e_ref.mean()) + 1e-4, name
        assert rel_err(y.cpu(), ref, floor_frac=1.0) <= 1e-1, name
        _report(capsys, f"cfg5 layer [1,2048,4096] FF=11008 ({name})",
                max_abs_vs_exact=round(float(e_gpu.max()), 4),
                mean_abs_vs_exact=round(float(e_gpu.mean()), 5),
                oracle_bf16_max_abs_vs_exact=round(float(e_ref.max()), 4),
                oracle_bf16_mean_abs_vs_exact=round(float(e_ref.mean()), 5))
    # the two compositions differ only in rounding points
    assert rel_err(y_fused.cpu(), y_mod.cpu(), floor_frac=1.0) <= 1e-1


def test_cfg2b_norm_worst_case_at_the_benchmark_shape(cuda, capsys):
    """RMSNorm and the fused RMSNorm -> int8 on bf16 [16, 2048, 4096] (seed 0, weight
    1 + N(0, 0.02)): how far the worst element is from the oracle and how many elements lie
    beyond 1e-2 relative, measured over all 134 M elements and reported."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(16, 2048, 4096, generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(4096, generator=g)).bfloat16()
    y = T.ops.rmsnorm(x.to(cuda), w.to(cuda), 1e-6).cpu()
    ref = R.rmsnorm_ref(x, w, 1e-6)
    d = bf16_ulps(y, ref)
    rel = (y.double() - ref.double()).abs() / ref.double().abs().clamp_min(
        1e-2 * float(ref.double().pow(2).mean().sqrt()))
    beyond = int((rel > 1e-2).sum())
    i = int(rel.argmax())
    assert int(d.max()) <= 2 and beyond <= 1e-5 * y.numel()
    _report(capsys, "cfg2b RMSNorm bf16 [16,2048,4096]", elements=y.numel(),
            max_ulps=int(d.max()), differing=int((d > 0).sum()), beyond_1ulp=int((d > 1).sum()),
            beyond_1e2_relative=beyond, worst_relative=round(float(rel.flatten()[i]), 5),
            worst_kernel=float(y.flatten()[i]), worst_oracle=float(ref.flatten()[i]))
    codes, scales = T.rmsnorm_quantize(x.to(cuda), w.to(cuda), 1e-6)
    rc, rs = R.rmsnorm_quantize_ref(x, w, 1e-6)
    codes, scales = codes.cpu(), scales.cpu()
    diff = (codes.int() - rc.int()).abs()
    rows_other_absmax = int((scales.view(-1) != rs.view(-1)).sum())
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 5e-3
    # given the kernel's own bf16 norm (identical fp32 absmax) the codes are bit-exact
    c2, s2 = R.quantize_rowwise_ref(y)
    assert torch.equal(codes, c2) and torch.equal(scales, s2)
    _report(capsys, "cfg2b fused RMSNorm->int8 vs end-to-end oracle", codes_differing=int((diff > 0).sum()),
            max_code_difference=int(diff.max()), rows_with_other_absmax=rows_other_absmax,
            rows=scales.numel(), bit_exact_given_kernel_norm=True)
