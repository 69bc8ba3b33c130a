"""The three restatements of the int8 path (torch, numpy, C) agree bit for bit, and the
FMA-refined quotient used by the CUDA encoder equals the IEEE quotient."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import build_c, int8_numpy as N, reference_port as R
from tests.util import outlier_matrix


def _c_lib():
    lib = ctypes.CDLL(build_c.build())
    lib.oracle_quant_rowwise_bf16.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 2
    lib.oracle_dequant_rowwise_bf16.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 2
    return lib


def _cases():
    x = outlier_matrix(64, 4096, seed=0).bfloat16()
    x[3] = 0  # zero row
    x[5, 7] = 3.0e38  # huge scale
    x[6] = (x[6].float() * 1e-30).bfloat16()  # tiny scale
    return x


def test_torch_numpy_c_agree_bit_exact():
    x = _cases()
    codes_t, scales_t = R.quantize_rowwise_ref(x)
    bits = x.view(torch.int16).numpy().view(np.uint16)
    codes_n, scales_n = N.quantize_rowwise_np(N.bf16_bits_to_f32(bits))
    assert np.array_equal(codes_t.numpy(), codes_n)
    assert np.array_equal(scales_t.numpy().view(np.uint32), scales_n.view(np.uint32))
    lib = _c_lib()
    codes_c = np.empty(bits.shape, np.int8)
    scales_c = np.empty(bits.shape[0], np.float32)
    bits_c = np.ascontiguousarray(bits)
    lib.oracle_quant_rowwise_bf16(bits_c.ctypes.data, codes_c.ctypes.data, scales_c.ctypes.data,
                                  bits.shape[0], bits.shape[1])
    assert np.array_equal(codes_c, codes_n)
    assert np.array_equal(scales_c.view(np.uint32), scales_n.view(np.uint32))
    assert codes_n[3].max() == 0 and scales_n[3] == 0  # zero-row rule
    assert np.abs(codes_n.astype(np.int32)).max() == 127
    # dequantise
    deq_t = R.dequantize_rowwise_ref(codes_t, scales_t, torch.bfloat16)
    deq_n = N.f32_to_bf16_bits(N.dequantize_rowwise_np(codes_n, scales_n))
    assert np.array_equal(deq_t.view(torch.int16).numpy().view(np.uint16), deq_n)
    deq_c = np.empty(bits.shape, np.uint16)
    lib.oracle_dequant_rowwise_bf16(codes_c.ctypes.data, scales_c.ctypes.data, deq_c.ctypes.data,
                                    bits.shape[0], bits.shape[1])
    assert np.array_equal(deq_c, deq_n)


def test_round_half_even_and_clamp():
    # scale 1 exactly (absmax 127): ties must go to even
    x = torch.tensor([[127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 63.5]])
    codes, scales = R.quantize_rowwise_ref(x)
    assert scales.item() == 1.0
    assert codes.tolist() == [[127, 0, 2, 2, 0, -2, -2, 64]]


def test_quantize_roundtrip_error_bound():
    x = outlier_matrix(128, 1024, seed=1).bfloat16()
    codes, scales = R.quantize_rowwise_ref(x)
    deq = R.dequantize_rowwise_ref(codes, scales, torch.float32)
    err = (deq - x.float()).abs()
    assert bool((err <= 0.5005 * scales.unsqueeze(-1)).all())


def test_fused_oracle_is_norm_then_quant():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32, 512, generator=g).bfloat16()
    w = (1 + 0.02 * torch.randn(512, generator=g)).bfloat16()
    c1, s1 = R.rmsnorm_quantize_ref(x, w, 1e-6)
    y = R.rmsnorm_ref(x, w, 1e-6)
    assert y.dtype == torch.bfloat16
    c2, s2 = R.quantize_rowwise_ref(y)
    assert torch.equal(c1, c2) and torch.equal(s1, s2)


def _fma32(a, b, c):
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def test_refined_quotient_equals_ieee_division():
    """q = x*r; q += (x - q*s)*r, twice, with r = RN(1/s): the sequence the CUDA encoder uses
    instead of a division. Checked against numpy's IEEE float32 division over every bf16
    magnitude below the row maximum and over random fp32 values, for many scales."""
    rng = np.random.default_rng(0)
    allx = (np.arange(0, 1 << 16, dtype=np.uint32) << 16).view(np.float32)
    allx = allx[np.isfinite(allx)]
    for trial in range(60):
        am = np.float32(abs(rng.standard_normal()) * 10 ** rng.uniform(-6, 6) + 1e-12)
        s = am / np.float32(127)
        if not (1e-18 < s < 1e18):
            continue
        r = np.float32(1) / s
        for xs in (allx[np.abs(allx) <= am], (rng.uniform(-1, 1, 50000) * am).astype(np.float32)):
            xs = xs[np.abs(xs) >= am * 1e-7]
            sv, rv = np.full_like(xs, s), np.full_like(xs, r)
            q = xs * rv
            for _ in range(2):
                q = _fma32(_fma32(-q, sv, xs), rv, q)
            assert np.array_equal(q, xs / sv)
            codes = np.rint(q)
            assert np.abs(codes).max() <= 127


def test_magic_number_rounding_is_half_even():
    q = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5, 127.0, -127.0, 3.2], np.float32)
    y = q + np.float32(12582912.0)
    low = (y.view(np.uint32) & 0xFF).astype(np.uint8).view(np.int8)
    assert np.array_equal(low, np.rint(q).astype(np.int8))


def test_two_fma_bracket_never_disagrees_with_ieee_quotient():
    """The CUDA encoder's fast path: t_lo = rint(x*rcp_lo), t_hi = rint(x*rcp_hi) (each a single
    rounding of an exact product) with rcp_lo/hi = r * (1 -/+ 2^-21), r = the hardware's
    approximate 1/scale (within 2^-23; modelled here at both ends of a 2^-22 band and exact).
    Whenever the two agree they must equal rint(RN(x/scale)); the values where they differ
    (handed to the exact path) must be rare. Products of two fp32 values are exact in float64."""
    rng = np.random.default_rng(0)
    f32 = np.float32
    total = differ = 0
    for absmax in [1.0, 127.0, 3.1415927, 4.7, 100.0, 1e-3, 7.7e4, 0.33333334] + list(
            np.exp(rng.uniform(-20, 20, size=24))):
        scale = f32(absmax) / f32(127.0)
        # random values, plus a cloud of values a few ulps around every rounding boundary
        x = rng.uniform(-1.0, 1.0, size=200_000).astype(f32) * f32(absmax)
        halves = (np.arange(-127, 127, dtype=f32) + f32(0.5)) * scale
        cloud = [halves]
        for _ in range(8):
            cloud.append(np.nextafter(cloud[-1], f32(np.inf)).astype(f32))
        cloud.append(halves)
        for _ in range(8):
            cloud.append(np.nextafter(cloud[-1], f32(-np.inf)).astype(f32))
        x = np.concatenate([x] + cloud)
        x = x[np.abs(x) <= f32(absmax)]
        xb = N.bf16_bits_to_f32(N.f32_to_bf16_bits(x))  # what the benchmark feeds
        xb = xb[np.abs(xb) <= f32(absmax)]
        for rel in (-2.0 ** -22, 0.0, 2.0 ** -22):
            r = f32(np.float64(1.0) / np.float64(scale) * (1.0 + rel))
            rcp_lo = f32(r * f32(1.0 - 2.0 ** -21))
            rcp_hi = f32(r * f32(1.0 + 2.0 ** -21))
            for v in (x, xb):
                want = np.rint(v / scale)  # IEEE fp32 division, then half-even
                lo = np.rint(v.astype(np.float64) * np.float64(rcp_lo))
                hi = np.rint(v.astype(np.float64) * np.float64(rcp_hi))
                same = lo == hi
                assert np.array_equal(lo[same], want[same].astype(np.float64))
                if v is x:
                    total += 200_000
                    differ += int((~same[:200_000]).sum())
    assert differ / total < 1e-3, differ / total
