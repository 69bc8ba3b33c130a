"""Parity of the row kernels (RMSNorm, LayerNorm, int8 quantise / dequantise, fused
RMSNorm->int8) with the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import trinix_b200 as T
from oracle import int8_numpy as N, reference_port as R
from tests.util import Golden, assert_norm_close, bf16_ulps, outlier_matrix, rel_err

pytestmark = pytest.mark.gpu
G = Golden()


def test_rmsnorm_fp32_baseline_config_golden(cuda):
    """FastRMSNorm(768, eps=1e-6) fp32 on the reference's own output vector."""
    y = T.TritonRMSNormKernel.apply(G("rms_f32_x").to(cuda), G("rms_f32_w").to(cuda), 1e-6)
    torch.testing.assert_close(y.cpu(), G("rms_f32_y"), rtol=1e-5, atol=1e-6)


def test_rmsnorm_fp32_full_config(cuda):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 128, 768, generator=g)
    w = 1 + 0.02 * torch.randn(768, generator=g)
    y, rstd = T.ops.rmsnorm(x.to(cuda), w.to(cuda), 1e-6, return_rstd=True)
    ref = R.rmsnorm_ref(x, w, 1e-6)
    torch.testing.assert_close(y.cpu(), ref, rtol=1e-5, atol=1e-6)
    ref_rstd = torch.rsqrt(x.pow(2).mean(-1) + 1e-6).flatten()
    torch.testing.assert_close(rstd.cpu(), ref_rstd, rtol=1e-6, atol=0)


@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 72), (5, 256), (7, 1000), (4, 2048),
                                       (64, 4096), (3, 4104), (2, 8192), (2, 16384), (2, 32768),
                                       (1, 65536 + 8), (2, 131080), (3, 777)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rmsnorm_shapes(cuda, rows, cols, dtype):
    g = torch.Generator().manual_seed(rows * 131 + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    y = T.ops.rmsnorm(x.to(cuda), w.to(cuda), 1e-6).cpu()
    ref = R.rmsnorm_ref(x, w, 1e-6)
    assert y.dtype == dtype and y.shape == x.shape
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(y, ref) <= tol
    if dtype == torch.bfloat16:
        # same rounding order as the oracle: at most 1 ulp apart, and almost everywhere equal
        d = bf16_ulps(y, ref)
        assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 2e-3


def test_rmsnorm_mixed_weight_dtype_and_strided_rows(cuda):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(16, 2, 4096, generator=g).bfloat16()
    w32 = 1 + 0.02 * torch.randn(4096, generator=g)
    xs = x.to(cuda)[:, 0, :]  # row stride 8192
    y = T.ops.rmsnorm(xs, w32.to(cuda), 1e-6).cpu()
    ref = R.rmsnorm_ref(x[:, 0, :], w32, 1e-6)  # fp32 (promotion); kernel returns bf16 of it
    assert y.dtype == torch.bfloat16
    assert int(bf16_ulps(y, ref.bfloat16()).max()) <= 1
    # unaligned base pointer -> scalar path, same numbers
    flat = torch.randn(4 * 520 + 1, generator=g).bfloat16()
    xu = flat[1:].view(4, 520)
    yu = T.ops.rmsnorm(flat.to(cuda)[1:].view(4, 520), torch.ones(520, device=cuda), 1e-6).cpu()
    assert rel_err(yu, R.rmsnorm_ref(xu, torch.ones(520), 1e-6)) <= 1e-2


def test_layernorm_golden_and_shapes(cuda):
    y = T.TritonLayerNormKernel.apply(G("ln_f32_x").to(cuda), G("ln_f32_w").to(cuda),
                                      G("ln_f32_b").to(cuda), 1e-5)
    torch.testing.assert_close(y.cpu(), G("ln_f32_y"), rtol=1e-5, atol=2e-6)
    yb = T.TritonLayerNormKernel.apply(G("ln_bf16_x").to(cuda), None, None, 1e-5)
    assert rel_err(yb.cpu(), G("ln_bf16_y")) <= 1e-2
    g = torch.Generator().manual_seed(4)
    for rows, cols, dtype in [(5, 8192, torch.bfloat16), (3, 4104, torch.float32),
                              (2, 1001, torch.float16), (9, 12288, torch.bfloat16)]:
        x = (torch.randn(rows, cols, generator=g) * 2 + 0.5).to(dtype)
        w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
        b = (0.1 * torch.randn(cols, generator=g)).to(dtype)
        y = T.ops.layernorm(x.to(cuda), w.to(cuda), b.to(cuda), 1e-5).cpu()
        assert rel_err(y, R.layernorm_ref(x, w, b, 1e-5)) <= (1e-4 if dtype == torch.float32 else 1e-2)
        y = T.ops.layernorm(x.to(cuda), w.to(cuda), None, 1e-5).cpu()
        assert rel_err(y, R.layernorm_ref(x, w, None, 1e-5)) <= (1e-4 if dtype == torch.float32 else 1e-2)


def _assert_quant_exact(x_cpu, codes, scales):
    rc, rs = R.quantize_rowwise_ref(x_cpu)
    assert torch.equal(scales.cpu().view(torch.int32), rs.view(torch.int32)), "scales differ"
    assert torch.equal(codes.cpu(), rc), "codes differ"


def test_quantize_benchmark_config_bit_exact(cuda):
    """bf16 [8192, 4096] ~ N(0,1) with 0.1% outliers x20: codes and scales bit-exact."""
    x = outlier_matrix(8192, 4096, seed=0).bfloat16()
    codes, scales = T.quantize_rowwise(x.to(cuda))
    assert codes.dtype == torch.int8 and scales.dtype == torch.float32
    _assert_quant_exact(x, codes, scales)
    # numpy restatement too
    bits = x.view(torch.int16).numpy().view(np.uint16)
    cn, sn = N.quantize_rowwise_np(N.bf16_bits_to_f32(bits[:512]))
    assert np.array_equal(codes[:512].cpu().numpy(), cn)
    deq = T.dequantize_rowwise(codes, scales, torch.bfloat16)
    ref = R.dequantize_rowwise_ref(codes.cpu(), scales.cpu(), torch.bfloat16)
    assert torch.equal(deq.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("rows,cols", [(1, 8), (4, 16), (3, 100), (5, 1000), (2, 4104),
                                       (3, 16384), (2, 40000), (1, 200000), (6, 11008)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantize_edge_cases_bit_exact(cuda, rows, cols, dtype):
    g = torch.Generator().manual_seed(cols)
    x = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    if rows > 1:
        x[1] = 0  # zero row -> scale 0, codes 0
    x[0, 0] = 127.0  # forces exact ties x.5 for small integers + 0.5
    if cols > 4:
        x[0, 1:5] = torch.tensor([0.5, 1.5, -2.5, 63.5]).to(dtype)
        x[0] = x[0].clamp(-127, 127)
    codes, scales = T.quantize_rowwise(x.to(cuda))
    _assert_quant_exact(x, codes, scales)
    for out_dtype in (torch.bfloat16, torch.float32):
        deq = T.dequantize_rowwise(codes, scales, out_dtype).cpu()
        ref = R.dequantize_rowwise_ref(codes.cpu(), scales.cpu(), out_dtype)
        assert torch.equal(deq.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32),
                           ref.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32))


@pytest.mark.parametrize("absmax", [127.0, 254.0, 1.0, 3.1415927, 100.0, 0.0078125, 12345.678])
def test_quantize_rounding_boundaries_bit_exact(cuda, absmax):
    """Quotients on and within a few fp32 ulps of every half-integer: the kernel's two-FMA
    bracket must hand exactly these values to its exact-quotient path, so codes stay bit-exact
    (the oracle rounds the IEEE quotient half to even)."""
    scale = np.float32(absmax) / np.float32(127.0)
    halves = (np.arange(-127, 127, dtype=np.float32) + np.float32(0.5))     # k + 0.5
    centre = (halves * scale).astype(np.float32)                           # x with x/scale ~ k+0.5
    rows = []
    for step in range(-6, 7):                                              # +- 6 ulps around it
        v = centre.copy()
        for _ in range(abs(step)):
            v = np.nextafter(v, np.float32(np.inf if step > 0 else -np.inf)).astype(np.float32)
        rows.append(v)
    x = torch.from_numpy(np.stack(rows))
    x = torch.cat([x, torch.full((x.shape[0], 2), float(absmax))], dim=1)  # fixes the row absmax
    x = torch.nn.functional.pad(x, (0, (-x.shape[1]) % 8)).contiguous()
    assert float(x.abs().max()) == float(np.float32(absmax))
    codes, scales = T.quantize_rowwise(x.to(cuda))
    _assert_quant_exact(x, codes, scales)
    # same, with the fp32 row long enough for the multi-warp configurations
    xl = x.repeat(1, 20).contiguous()
    codes, scales = T.quantize_rowwise(xl.to(cuda))
    _assert_quant_exact(xl, codes, scales)
    # 16-bit inputs: nearest representable values to the boundaries
    for dtype in (torch.bfloat16, torch.float16):
        xd = xl.to(dtype)
        if not torch.isfinite(xd.float()).all():
            continue
        codes, scales = T.quantize_rowwise(xd.to(cuda))
        _assert_quant_exact(xd, codes, scales)


def test_quantize_extreme_scales_bit_exact(cuda):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(6, 512, generator=g)
    x[0] *= 1e-30; x[1] *= 1e30; x[2] *= 1e-38; x[3] *= 3e37
    for dtype in (torch.float32, torch.bfloat16):
        xd = x.to(dtype)
        codes, scales = T.quantize_rowwise(xd.to(cuda))
        _assert_quant_exact(xd, codes, scales)


def test_fused_rmsnorm_quant_equals_unfused_bit_exact(cuda):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 512, 4096, generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(4096, generator=g)).bfloat16()
    xd, wd = x.to(cuda), w.to(cuda)
    codes, scales = T.rmsnorm_quantize(xd, wd, 1e-6)
    y = T.ops.rmsnorm(xd, wd, 1e-6)
    c2, s2 = T.quantize_rowwise(y)
    assert torch.equal(codes, c2) and torch.equal(scales.view(torch.int32), s2.view(torch.int32))
    # given the kernel's bf16 norm output, the oracle's quantiser reproduces codes and scales
    _assert_quant_exact(y.cpu(), codes, scales)
    # against the full CPU oracle only the fp32 reduction order of mean(x^2) differs
    rc, rs = R.rmsnorm_quantize_ref(x, w, 1e-6)
    dc = (codes.cpu().int() - rc.int()).abs()
    assert int(dc.max()) <= 1 and float((dc > 0).float().mean()) < 5e-3
    torch.testing.assert_close(scales.cpu(), rs, rtol=1e-2, atol=0)
    for rows, cols, dtype in [(3, 520, torch.bfloat16), (5, 777, torch.float16),
                              (2, 8192, torch.float32), (2, 70000, torch.bfloat16)]:
        xx = torch.randn(rows, cols, generator=g).to(dtype).to(cuda)
        ww = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).to(cuda)
        c, s = T.rmsnorm_quantize(xx, ww, 1e-6)
        c2, s2 = T.quantize_rowwise(T.ops.rmsnorm(xx, ww, 1e-6))
        assert torch.equal(c, c2) and torch.equal(s.view(torch.int32), s2.view(torch.int32))


def test_quantize_full_size_properties(cuda):
    """Size-independent properties at the benchmark's full size ([16,2048,4096] activations)."""
    g = torch.Generator(device=cuda).manual_seed(0)
    x = torch.randn(16, 2048, 4096, generator=g, device=cuda, dtype=torch.float32).bfloat16()
    w = torch.ones(4096, device=cuda, dtype=torch.bfloat16)
    codes, scales = T.rmsnorm_quantize(x, w, 1e-6)
    assert codes.shape == x.shape and scales.shape == x.shape[:-1]
    assert int(codes.abs().amax(-1).min()) == 127  # every row hits +-127 exactly once at least
    y = T.ops.rmsnorm(x, w, 1e-6)
    deq = T.dequantize_rowwise(codes, scales, torch.float32)
    assert bool(((deq - y.float()).abs() <= 0.5005 * scales.unsqueeze(-1)).all())
    # idempotence: re-quantising the dequantised codes (exact in fp32) returns the same codes
    c2, s2 = T.quantize_rowwise(deq)
    assert torch.equal(c2, codes)
    assert torch.equal(T.quantize_rowwise(y)[0], codes)


def test_residual_rmsnorm_golden_and_shapes(cuda):
    x, r, w = G("resrms_x"), G("resrms_r"), G("resrms_w")
    y = T.TritonFusedResidualRMSNormKernel.apply(x.to(cuda), r.to(cuda), w.to(cuda), 1e-6)
    assert int(bf16_ulps(y.cpu(), G("resrms_y")).max()) <= 1
    g = torch.Generator().manual_seed(11)
    for rows, cols, dtype in [(64, 4096, torch.bfloat16), (5, 8192, torch.bfloat16),
                              (3, 777, torch.bfloat16), (4, 4104, torch.float32),
                              (2, 40000, torch.float16), (3, 520, torch.float16)]:
        x = torch.randn(rows, cols, generator=g).to(dtype)
        r = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
        w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
        y, s = T.ops.residual_rmsnorm(x.to(cuda), r.to(cuda), w.to(cuda), 1e-6, return_sum=True)
        ref = R.residual_rmsnorm_ref(x, r, w, 1e-6)
        assert rel_err(y.cpu(), ref) <= (1e-5 if dtype == torch.float32 else 1e-2)
        # the summed residual stream is the fp32 sum rounded once to the activation dtype
        assert torch.equal(s.cpu(), (x.float() + r.float()).to(dtype))
        if dtype == torch.bfloat16:
            d = bf16_ulps(y.cpu(), ref)
            assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 2e-3


@pytest.mark.parametrize("xdtype,wdtype", [(torch.bfloat16, torch.float32),
                                           (torch.float16, torch.float32),
                                           (torch.bfloat16, torch.float16)])
def test_residual_rmsnorm_weight_of_another_dtype(cuda, xdtype, wdtype):
    """16-bit x and residual with a weight of another dtype (the state of a freshly built
    FastFusedResidualRMSNorm under autocast-style use: fp32 ones). The normalised row must be the
    fp32 SUM x + r, on the vector path (4096, 2048 columns) and on the scalar path (odd widths),
    for the plain and the int8 form."""
    g = torch.Generator().manual_seed(31)
    for rows, cols in [(64, 4096), (9, 2048), (5, 777), (3, 8200), (2, 33000)]:
        x = torch.randn(rows, cols, generator=g).to(xdtype)
        r = (torch.randn(rows, cols, generator=g) * 3).to(xdtype)
        w = (1 + 0.1 * torch.randn(cols, generator=g)).to(wdtype)
        xc, rc, wc = x.to(cuda), r.to(cuda), w.to(cuda)
        y, s = T.ops.residual_rmsnorm(xc, rc, wc, 1e-6, return_sum=True)
        # the oracle's product is promoted to the wider dtype; the kernel rounds it once to x's
        ref = R.residual_rmsnorm_ref(x, r, w, 1e-6).to(xdtype)
        assert y.dtype == xdtype
        assert rel_err(y.cpu(), ref) <= 1e-2
        assert float((y.cpu() != ref).float().mean()) < 2e-3
        assert torch.equal(s.cpu(), (x.float() + r.float()).to(xdtype))
        codes, scales = T.residual_rmsnorm_quantize(xc, rc, wc, 1e-6)
        c2, s2 = T.quantize_rowwise(y)
        assert torch.equal(codes, c2) and torch.equal(scales, s2)
    # the mirror module with its default fp32 weight on bf16 activations
    m = T.FastFusedResidualRMSNorm(4096).to(cuda)
    assert m.weight.dtype == torch.float32
    x = torch.randn(16, 4096, generator=g).bfloat16()
    r = (torch.randn(16, 4096, generator=g) * 2).bfloat16()
    with torch.no_grad():
        y = m(x.to(cuda), r.to(cuda))
    y = y[0] if isinstance(y, tuple) else y
    ref = R.residual_rmsnorm_ref(x, r, torch.ones(4096), 1e-6)
    assert rel_err(y.float().cpu(), ref.float()) <= 1e-2


def _assert_resln_close(y, x, r, w, b, eps=1e-5):
    """LayerNorm(x + r) against the oracle. fp32: 1e-5 relative. 16-bit: the kernel follows the
    oracle's rounding order round(round(w * round(n)) + b); the statistics can differ in their
    last fp32 bits (summation order), which now and then flips the inner rounding by one ulp. So:
    any difference in fewer than 0.2 % of the elements, beyond 1e-2 relative in at most 1e-5 of
    them, and never further than four rounding steps of the larger of the two terms of the final
    sum (plus 1e-5 absolute: where x + r sits on the row mean, the normalised value is only as
    good as the last bits of that mean)."""
    ref = R.residual_layernorm_ref(x, r, w, b, eps)
    if x.dtype == torch.float32:
        assert y.dtype == torch.float32 and rel_err(y, ref) <= 1e-5
        return
    ref = ref.to(x.dtype)  # fp32 parameters promote the oracle's result; the kernel rounds once
    assert y.dtype == ref.dtype and y.shape == ref.shape
    assert float((y != ref).float().mean()) < 2e-3
    err = (y.double() - ref.double()).abs()
    floor = 1e-2 * float(ref.double().pow(2).mean().sqrt())
    assert float((err > 1e-2 * ref.double().abs().clamp_min(floor)).float().mean()) <= 1e-5
    n = R.residual_layernorm_ref(x, r, None, None, eps).double()
    terms = (n * (w.double() if w is not None else 1.0)).abs()
    if b is not None:
        terms = torch.maximum(terms, b.double().abs().expand_as(terms))
    step = 2.0 ** (-7 if x.dtype == torch.bfloat16 else -10)
    assert bool((err <= 4 * step * terms + 1e-5).all()), float((err - 4 * step * terms).max())


def test_residual_layernorm_golden_and_shapes(cuda):
    """LayerNorm(x + residual) in one kernel against the reference's own vectors and the oracle:
    16-bit parameters (affine part rounded step by step), fp32 parameters (promoted), fp32 rows,
    missing weight / bias, rows on the vector and on the scalar path, the summed stream, and the
    mirror module above its kernel threshold."""
    x, r, w, b = G("resln_x"), G("resln_r"), G("resln_w"), G("resln_b")
    xc, rc = x.to(cuda), r.to(cuda)
    y = T.TritonFusedResidualLayerNormKernel.apply(xc, rc, w.to(cuda), b.to(cuda), 1e-5).cpu()
    assert int(bf16_ulps(y, G("resln_y")).max()) <= 1
    assert float((y != G("resln_y")).float().mean()) < 2e-3
    y = T.ops.residual_layernorm(xc, rc, w.float().to(cuda), b.float().to(cuda), 1e-5).cpu()
    assert int(bf16_ulps(y, G("resln_y_f32w").bfloat16()).max()) <= 1
    y = T.ops.residual_layernorm(xc.float(), rc.float(), w.float().to(cuda), b.float().to(cuda),
                                 1e-5).cpu()
    torch.testing.assert_close(y, G("resln_y_f32"), rtol=2e-5, atol=2e-6)
    g = torch.Generator().manual_seed(23)
    for rows, cols, dtype in [(64, 4096, torch.bfloat16), (5, 8192, torch.bfloat16),
                              (3, 777, torch.bfloat16), (4, 4104, torch.float32),
                              (2, 40000, torch.float16), (3, 520, torch.float16),
                              (304, 2048, torch.bfloat16), (9, 32768, torch.bfloat16),
                              (2, 65536, torch.float32)]:
        xs = (torch.randn(rows, cols, generator=g) + 0.3).to(dtype)
        rs = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
        ws = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
        bs = (0.1 * torch.randn(cols, generator=g)).to(dtype)
        xd, rd, wd, bd = xs.to(cuda), rs.to(cuda), ws.to(cuda), bs.to(cuda)
        y, s = T.ops.residual_layernorm(xd, rd, wd, bd, 1e-5, return_sum=True)
        _assert_resln_close(y.cpu(), xs, rs, ws, bs)
        assert torch.equal(s.cpu(), (xs.float() + rs.float()).to(dtype))
        _assert_resln_close(T.ops.residual_layernorm(xd, rd, None, None, 1e-5).cpu(),
                            xs, rs, None, None)
        _assert_resln_close(T.ops.residual_layernorm(xd, rd, wd, None, 1e-5).cpu(),
                            xs, rs, ws, None)
        if dtype != torch.float32:
            _assert_resln_close(T.ops.residual_layernorm(xd, rd, wd.float(), bd.float(), 1e-5).cpu(),
                                xs, rs, ws.float(), bs.float())
    # rows given as a strided view (row stride > C), through the mirror module
    big = torch.randn(6, 2 * 4104, generator=g).bfloat16()
    res = torch.randn(6, 4104, generator=g).bfloat16()
    m = T.FastFusedResidualLayerNorm(4104).bfloat16().to(cuda)
    with torch.no_grad():
        m.weight.copy_((1 + 0.1 * torch.randn(4104, generator=g)).bfloat16())
        m.bias.copy_((0.1 * torch.randn(4104, generator=g)).bfloat16())
        assert m._check_triton_availability()
        view = big.to(cuda)[:, :4104]
        y = m(view, res.to(cuda))
        _assert_resln_close(y.cpu(), big[:, :4104], res, m.weight.detach().cpu(),
                            m.bias.detach().cpu())
    with pytest.raises(ValueError):
        T.ops.residual_layernorm(xc, rc[:, :8], None, None)


def test_residual_rmsnorm_quant_equals_unfused_bit_exact(cuda):
    g = torch.Generator().manual_seed(12)
    for rows, cols, dtype in [(512, 4096, torch.bfloat16), (7, 1000, torch.bfloat16),
                              (3, 8192, torch.float32), (5, 12288, torch.float16)]:
        x = torch.randn(rows, cols, generator=g).to(dtype).to(cuda)
        r = torch.randn(rows, cols, generator=g).to(dtype).to(cuda)
        w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype).to(cuda)
        codes, scales, s = T.residual_rmsnorm_quantize(x, r, w, 1e-6, return_sum=True)
        y, s2 = T.ops.residual_rmsnorm(x, r, w, 1e-6, return_sum=True)
        c2, sc2 = T.quantize_rowwise(y)
        assert torch.equal(codes, c2) and torch.equal(scales.view(torch.int32), sc2.view(torch.int32))
        assert torch.equal(s, s2)
        _assert_quant_exact(y.cpu(), codes, scales)  # oracle quantiser on the kernel's norm output


@pytest.mark.parametrize("nvec", [32, 64, 128, 256, 512, 1024, 2048, 4096])
@pytest.mark.parametrize("rows", [1, 8, 19, 304])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_every_op_on_exact_width_rows(cuda, nvec, rows, dtype):
    """Rows of exactly threads x vectors width take the guard-free specialisation of every
    configuration (one warp per row up to 1024 threads per row); row counts that are and are
    not a multiple of the rows per CTA. All six ops against the oracle."""
    cols = nvec * (8 if dtype == torch.bfloat16 else 4)
    g = torch.Generator().manual_seed(nvec * 7 + rows)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    r = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    b = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    xc, rc, wc, bc = x.to(cuda), r.to(cuda), w.to(cuda), b.to(cuda)
    assert_norm_close(T.ops.rmsnorm(xc, wc, 1e-6).cpu(), R.rmsnorm_ref(x, w, 1e-6))
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert rel_err(T.ops.layernorm(xc, wc, bc, 1e-5).cpu(), R.layernorm_ref(x, w, b, 1e-5)) <= tol
    codes, scales = T.quantize_rowwise(xc)
    _assert_quant_exact(x, codes, scales)
    # fused == unfused, bit for bit, and the oracle's quantiser on the kernel's norm agrees
    y = T.ops.rmsnorm(xc, wc, 1e-6)
    fc, fs = T.rmsnorm_quantize(xc, wc, 1e-6)
    uc, us = T.quantize_rowwise(y)
    assert torch.equal(fc, uc) and torch.equal(fs, us)
    _assert_quant_exact(y.cpu(), fc, fs)
    if nvec <= 4096 // (2 if dtype == torch.bfloat16 else 1):
        yr, sr = T.ops.residual_rmsnorm(xc, rc, wc, 1e-6, return_sum=True)
        assert_norm_close(yr.cpu(), R.residual_rmsnorm_ref(x, r, w, 1e-6))
        assert rel_err(sr.cpu(), (x.float() + r.float()).to(dtype)) <= (1e-6 if dtype == torch.float32 else 4e-3)
        qc, qs, _ = T.ops.residual_rmsnorm_quantize(xc, rc, wc, 1e-6, return_sum=True)
        uc2, us2 = T.quantize_rowwise(yr)
        assert torch.equal(qc, uc2) and torch.equal(qs, us2)


@pytest.mark.parametrize("act", ["mish", "quickgelu", "squared_relu"])
def test_rmsnorm_activation_golden_and_shapes(cuda, act):
    """activation(RMSNorm(x)) in one kernel against the reference's own vectors and the oracle:
    bf16 weight (product rounded before the activation), fp32 weight (promoted), fp32 rows, and
    the module above its kernel threshold."""
    x, w = G("rmsact_x"), G("rmsact_w")
    y = T.ops.rmsnorm_activation(x.to(cuda), w.to(cuda), 1e-6, act).cpu()
    assert_norm_close(y, G(f"rmsact_{act}_y"))
    y = T.ops.rmsnorm_activation(x.to(cuda), w.float().to(cuda), 1e-6, act).cpu()
    assert_norm_close(y, G(f"rmsact_{act}_y_f32w"))
    y = T.ops.rmsnorm_activation(x.float().to(cuda), w.float().to(cuda), 1e-6, act).cpu()
    torch.testing.assert_close(y, G(f"rmsact_{act}_y_f32"), rtol=2e-5, atol=2e-6)
    g = torch.Generator().manual_seed(17)
    for rows, cols, dtype in [(40, 4096, torch.bfloat16), (3, 8192, torch.float16),
                              (5, 1000, torch.bfloat16), (2, 4104, torch.float32),
                              (7, 16384, torch.bfloat16)]:
        xs = (torch.randn(rows, cols, generator=g) * 4).to(dtype)
        ws = (1 + 0.2 * torch.randn(cols, generator=g)).to(dtype)
        out = T.TritonFusedRMSNormActivationKernel.apply(xs.to(cuda), ws.to(cuda), 1e-6, act).cpu()
        ref = R.rmsnorm_activation_ref(xs, ws, 1e-6, act)
        if dtype == torch.float32:
            assert rel_err(out, ref) <= 2e-5
        else:
            assert rel_err(out, ref) <= 1e-2
    m = T.FastFusedRMSNormActivation(4096, activation=act).to(cuda).bfloat16()
    xm = (torch.randn(2, 9, 4096, generator=g) * 2).bfloat16()
    before = T.ops.launch_count
    ym = m(xm.to(cuda))
    assert T.ops.launch_count == before + 1
    assert rel_err(ym.cpu(), R.rmsnorm_activation_ref(xm, m.weight.detach().cpu(), 1e-6, act)) <= 1e-2
    with pytest.raises(ValueError):
        T.ops.rmsnorm_activation(xm.to(cuda), m.weight, 1e-6, "gelu")


def test_fused_int8_many_rows_odd_count(cuda):
    """Many rows of the benchmark width (4096 bf16 columns, the guard-free specialisation, every
    CTA striding over several rows) with a row count that divides by nothing: fused equals
    unfused bit for bit, the oracle's quantiser agrees on the kernel's norm, and a sample of rows
    matches the end-to-end oracle."""
    R_, C_ = 24001, 4096
    g = torch.Generator(device=cuda).manual_seed(77)
    x = (torch.randn(R_, C_, generator=g, device=cuda) * 1.7).bfloat16()
    w = (1 + 0.1 * torch.randn(C_, generator=g, device=cuda)).bfloat16()
    codes, scales = T.rmsnorm_quantize(x, w, 1e-6)
    y = T.ops.rmsnorm(x, w, 1e-6)
    c2, s2 = T.quantize_rowwise(y)
    assert torch.equal(codes, c2) and torch.equal(scales, s2)
    # a strided input (row stride > C) takes the same path
    big = torch.zeros(R_, C_ + 64, device=cuda, dtype=torch.bfloat16)
    big[:, :C_] = x
    c3, s3 = T.rmsnorm_quantize(big[:, :C_], w, 1e-6)
    assert torch.equal(c3, codes) and torch.equal(s3, scales)
    rows = torch.tensor([0, 1, 2, 777, 5919, 5920, 11840, 17760, 23679, 23680, 24000], device=cuda)
    rc, rs = R.quantize_rowwise_ref(y[rows].cpu())
    assert torch.equal(codes[rows].cpu(), rc) and torch.equal(scales[rows].cpu(), rs)
    ref_c, ref_s = R.rmsnorm_quantize_ref(x[rows].cpu(), w.cpu(), 1e-6)
    assert int((codes[rows].cpu().int() - ref_c.int()).abs().max()) <= 1
    torch.testing.assert_close(scales[rows].cpu(), ref_s, rtol=1e-2, atol=0)
