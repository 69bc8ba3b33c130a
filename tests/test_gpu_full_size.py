"""The benchmark configurations at their full sizes, checked through size-independent properties
and through the CPU oracle on a seeded sample of rows / tokens (the oracle on the whole tensor
would take minutes per case). The int8 and attention configurations have their full-size tests
next to their other tests (test_gpu_rowwise.py, test_gpu_attention.py)."""
import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import assert_norm_close, bf16_ulps, rel_err

pytestmark = pytest.mark.gpu


def _rand_bf16(cuda, *shape, seed):
    g = torch.Generator(device=cuda).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=cuda, dtype=torch.float32).bfloat16()


def test_rope_full_size(cuda):
    """q[8,2048,32,128], k[8,2048,8,128] bf16, fp32 tables, base 10000, positions 0..2047."""
    q, k = _rand_bf16(cuda, 8, 2048, 32, 128, seed=0), _rand_bf16(cuda, 8, 2048, 8, 128, seed=1)
    cos, sin = R.rope_tables_ref(128, 2048, 10000.0, torch.float32)
    cosd, sind = cos.to(cuda), sin.to(cuda)
    qo, ko = T.rope(q, k, cosd, sind)
    # position 0 has cos = 1, sin = 0: those rows come back bit for bit
    assert torch.equal(qo[:, 0], q[:, 0]) and torch.equal(ko[:, 0], k[:, 0])
    # a rotation preserves the length of every (x[i], x[i + 64]) pair, up to the output rounding
    for a, b in ((q, qo), (k, ko)):
        n_in = a[..., :64].float() ** 2 + a[..., 64:].float() ** 2
        n_out = b[..., :64].float() ** 2 + b[..., 64:].float() ** 2
        assert float(((n_out - n_in).abs() / (n_in + 1e-3)).max()) <= 2.0 ** -6
    # rotating back by the negated angle returns the input within the two output roundings (2^-6 of the
    # larger component of each pair bounds both)
    qb, kb = T.ops.rope(qo, ko, cosd, sind, inverse=True)
    for a, b in ((q, qb), (k, kb)):
        big = torch.maximum(a[..., :64].abs(), a[..., 64:].abs()).float().repeat(1, 1, 1, 2)
        assert bool(((b.float() - a.float()).abs() <= 2.0 ** -6 * big + 1e-6).all())
    # the oracle on a sample of batch elements / positions: bit for bit
    g = torch.Generator().manual_seed(2)
    pos = torch.randperm(2048, generator=g)[:48].sort().values
    qs, ks = q[3, pos].cpu().unsqueeze(0), k[3, pos].cpu().unsqueeze(0)
    rq, rk = R.rope_ref(qs, ks, cos[pos], sin[pos])
    assert torch.equal(qo[3, pos].cpu().unsqueeze(0), rq.bfloat16())
    assert torch.equal(ko[3, pos].cpu().unsqueeze(0), rk.bfloat16())


@pytest.mark.parametrize("name", ["swiglu", "geglu", "reglu"])
def test_glu_full_size(cuda, name):
    """Module input cat([up, gate]) of [8, 2048, 2 x 11008] bf16."""
    x = _rand_bf16(cuda, 8 * 2048, 2 * 11008, seed=3)
    y = T.glu(x, name)
    assert y.shape == (8 * 2048, 11008)
    # linear in `up`: doubling it (exact in bf16) doubles the output bit for bit
    x2 = x.clone()
    x2[:, :11008] *= 2
    assert torch.equal(T.glu(x2, name), y * 2)
    if name == "reglu":  # exact: zero wherever the gate is not positive, up * gate elsewhere
        gate, up = x[:, 11008:], x[:, :11008]
        assert bool((y[gate <= 0] == 0).all())
        assert torch.equal(y, (up.float() * gate.float().clamp_min(0)).bfloat16())
    # the oracle on a sample of rows
    g = torch.Generator().manual_seed(4)
    rows = torch.randperm(8 * 2048, generator=g)[:64]
    fn = {"swiglu": R.swiglu_ref, "geglu": R.geglu_ref, "reglu": R.reglu_ref}[name]
    ref = fn(x[rows.to(cuda)].cpu())
    got = y[rows.to(cuda)].cpu()
    assert rel_err(got, ref) <= 1e-2
    assert float((bf16_ulps(got, ref) > 1).float().mean()) <= 1e-4
    # backward at the same size: sampled rows against the float64 gradient
    dy = _rand_bf16(cuda, 8 * 2048, 11008, seed=5)
    dx = T.ops.glu_backward(dy, x, name)
    xs = x[rows.to(cuda)].cpu()
    (rg,) = R.autograd_ref(fn, [xs.double()], dy[rows.to(cuda)].cpu().double())
    assert rel_err(dx[rows.to(cuda)].cpu().double(), rg) <= 5e-3


def test_norms_full_size(cuda):
    """x[16, 2048, 4096] bf16, weight 1 + N(0, 0.02): RMSNorm (eps 1e-6) and LayerNorm (eps 1e-5)."""
    x = _rand_bf16(cuda, 16, 2048, 4096, seed=6)
    g = torch.Generator().manual_seed(7)
    w = (1 + 0.02 * torch.randn(4096, generator=g)).bfloat16()
    b = (0.02 * torch.randn(4096, generator=g)).bfloat16()
    wd, bd = w.to(cuda), b.to(cuda)
    y = T.ops.rmsnorm(x, wd, 1e-6)
    # scale invariance: RMSNorm(4 x) = RMSNorm(x) up to the eps term (4 x is exact in bf16)
    y4 = T.ops.rmsnorm(x * 4, wd, 1e-6)
    d = bf16_ulps(y4.cpu().flatten()[: 1 << 24], y.cpu().flatten()[: 1 << 24])
    # (a last-bit difference in rstd can flip the inner rounding, and the product with the weight
    # then now and then lands two ulps away: the same statement as tests.util.assert_norm_close)
    assert int(d.max()) <= 2 and float((d > 1).float().mean()) <= 1e-5
    assert float((d > 0).float().mean()) < 1e-3
    # every row of the normalised value has unit mean square (weight ~ 1: within a few per cent)
    ms = y.float().pow(2).mean(-1)
    assert float((ms - 1).abs().max()) <= 0.1
    # fused RMSNorm -> int8 on the same tensor equals quantise(norm) bit for bit
    codes, scales = T.rmsnorm_quantize(x, wd, 1e-6)
    c2, s2 = T.quantize_rowwise(y)
    assert torch.equal(codes, c2) and torch.equal(scales, s2)
    # the oracle on a sample of rows
    rows = torch.randperm(16 * 2048, generator=g)[:96].to(cuda)
    xs = x.view(-1, 4096)[rows].cpu()
    assert_norm_close(y.view(-1, 4096)[rows].cpu(), R.rmsnorm_ref(xs, w, 1e-6))
    yl = T.ops.layernorm(x, wd, bd, 1e-5)
    assert rel_err(yl.view(-1, 4096)[rows].cpu(), R.layernorm_ref(xs, w, b, 1e-5)) <= 1e-2
    # without the affine part every LayerNorm row has zero mean and unit mean square
    yn = T.ops.layernorm(x, None, None, 1e-5).float()
    assert float(yn.mean(-1).abs().max()) <= 1e-2
    assert float((yn.pow(2).mean(-1) - 1).abs().max()) <= 1e-2
    del yn
    # backward at the same size: determinism and sampled rows against the oracle's dx
    dy = _rand_bf16(cuda, 16 * 2048, 4096, seed=8)
    dx, dw = T.ops.rmsnorm_backward(dy, x.view(-1, 4096), wd, 1e-6)
    dx2, dw2 = T.ops.rmsnorm_backward(dy, x.view(-1, 4096), wd, 1e-6)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)
    rx, _ = R.autograd_ref(lambda a, ww: R.rmsnorm_ref(a, ww, 1e-6), [xs.double(), w.double()],
                           dy[rows].cpu().double())
    assert rel_err(dx[rows].cpu().double(), rx) <= 5e-3
    # dW against a float64 evaluation of sum_rows dy * n over all rows (torch, on the device)
    n = (x.view(-1, 4096).double() * torch.rsqrt(x.view(-1, 4096).double().pow(2).mean(-1, keepdim=True) + 1e-6))
    dw_ref = (dy.double() * n).sum(0)
    assert rel_err(dw.double().cpu(), dw_ref.cpu()) <= 5e-3
