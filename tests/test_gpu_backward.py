"""Backward kernels (RMSNorm, LayerNorm, GLUs, RoPE) against gradients of the reference's PyTorch
backend, through the kernel classes' autograd functions and the C ABI.

Two yardsticks. (1) The upcast oracle: autograd through the restated forward on `.double()`
inputs (LayerNorm and the GLUs then run in float64; the RMSNorm-family forwards cast to fp32
internally, as the reference's do, so for them this is the fp32 evaluation on exact inputs) — the
tighter truth; a 16-bit kernel result may differ from it by its one output rounding (half an ulp:
2^-9 relative for bf16, 2^-12 for fp16) plus fp32 summation order. (2) The
reference's own 16-bit autograd, which rounds every intermediate to the storage dtype (and, for
LayerNorm's dgamma / dbeta on CPU, adds partial sums in that dtype): looser by construction. A
norm's dx is a difference of terms of the size of the tensor's rms, each carrying such a rounding,
so against those vectors the bound is |a - b| <= 1e-2 (|b| + rms(b)). Relative errors elsewhere use
the floor of tests.util.rel_err (1 % of the tensor's rms)."""
import pytest
import torch

import trinix_b200 as T
from oracle import reference_port as R
from tests.util import Golden, rel_err

pytestmark = pytest.mark.gpu
G = Golden()

TOL32 = {torch.float32: 2e-5, torch.bfloat16: 5e-3, torch.float16: 1e-3}


def _chain_close(a, b) -> bool:
    """|a - b| <= 1e-2 (|b| + rms(b)): parity with a gradient whose intermediates were rounded to
    16 bits."""
    a, b = a.double(), b.double()
    return bool(((a - b).abs() <= 1e-2 * (b.abs() + b.pow(2).mean().sqrt())).all())


def _f(*ts):
    """Upcast for the oracle: float64, so that the oracle's own rounding is out of the picture."""
    return [None if t is None else t.double() for t in ts]


def _run_backward(fn, inputs, dy, cuda):
    """fn(*leaves) on CUDA leaves that all require grad; returns (output, grads) on the CPU."""
    leaves = [None if t is None else t.to(cuda).requires_grad_(True) for t in inputs]
    out = fn(*leaves)
    outs = out if isinstance(out, tuple) else (out,)
    dys = dy if isinstance(dy, tuple) else (dy,)
    torch.autograd.backward(list(outs), [d.to(cuda) for d in dys])
    return out, [None if t is None else t.grad.cpu() for t in leaves]


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_norm_gradients_golden(cuda, tag):
    """The reference's own gradient vectors (its modules under autograd, PyTorch backend)."""
    x, dy, w, b = (G(f"bwd_rms_{tag}_x"), G(f"bwd_rms_{tag}_dy"), G(f"bwd_rms_{tag}_w"),
                   G(f"bwd_ln_{tag}_b"))
    _, (dx, dw) = _run_backward(lambda a, ww: T.TritonRMSNormKernel.apply(a, ww, 1e-6), [x, w], dy, cuda)
    assert dx.dtype == x.dtype and dw.dtype == w.dtype
    close = (lambda a, b: rel_err(a, b) <= 2e-5) if tag == "f32" else _chain_close
    # dW / db are fp32 sums over the rows: 1e-4 of max(|ref|, 1 % rms), see the shape test
    close_sum = (lambda a, b: rel_err(a, b) <= 1e-4) if tag == "f32" else _chain_close
    assert close(dx, G(f"bwd_rms_{tag}_dx"))
    assert close_sum(dw, G(f"bwd_rms_{tag}_dw"))
    _, (dx, dw, db) = _run_backward(lambda a, ww, bb: T.TritonLayerNormKernel.apply(a, ww, bb, 1e-5),
                                    [x, w, b], dy, cuda)
    assert close(dx, G(f"bwd_ln_{tag}_dx"))
    if tag == "f32":
        assert close_sum(dw, G(f"bwd_ln_{tag}_dw")) and close_sum(db, G(f"bwd_ln_{tag}_db"))
    else:
        # ATen's CPU kernel adds the rows' contributions to dgamma / dbeta in bf16: its own error
        # is about 1 % of the vector's rms, so the bound against it is 5e-2 (|b| + rms(b)); the
        # fp32-upcast oracle is the tight check
        for mine, name in ((dw, "dw"), (db, "db")):
            ref = G(f"bwd_ln_{tag}_{name}").double()
            assert bool(((mine.double() - ref).abs() <= 5e-2 * (ref.abs() + ref.pow(2).mean().sqrt())).all())
        _, rw, rb = R.autograd_ref(lambda a, ww, bb: R.layernorm_ref(a, ww, bb, 1e-5), _f(x, w, b),
                                   dy.double())
        assert rel_err(dw.double(), rw) <= 5e-3 and rel_err(db.double(), rb) <= 5e-3


@pytest.mark.parametrize("tag", ["f32", "bf16"])
@pytest.mark.parametrize("name", ["swiglu", "geglu", "reglu"])
def test_glu_gradients_golden(cuda, tag, name):
    cls = {"swiglu": T.TritonSwiGLUKernel, "geglu": T.TritonGeGLUKernel, "reglu": T.TritonReGLUKernel}[name]
    x, dy = G(f"bwd_glu_{tag}_x"), G(f"bwd_glu_{tag}_dy")
    _, (dx,) = _run_backward(cls.apply, [x], dy, cuda)
    assert dx.shape == x.shape and dx.dtype == x.dtype
    if tag == "f32":
        # ATen's fp32 GELU-tanh backward forms 1 - tanh^2 with cancellation: its own vector sits
        # 1.1e-4 from the float64 gradient; the kernel (checked against float64 below) does not
        assert rel_err(dx, G(f"bwd_{name}_{tag}_dx")) <= (2e-4 if name == "geglu" else 2e-5)
        fn = {"swiglu": R.swiglu_ref, "geglu": R.geglu_ref, "reglu": R.reglu_ref}[name]
        (ref64,) = R.autograd_ref(fn, _f(x), dy.double())
        assert rel_err(dx.double(), ref64) <= 2e-5
    else:
        assert _chain_close(dx, G(f"bwd_{name}_{tag}_dx"))


def test_rope_gradients_golden(cuda):
    cos, sin = G("bwd_rope_cos").to(cuda), G("bwd_rope_sin").to(cuda)
    gq, gk = G("bwd_rope_gq"), G("bwd_rope_gk")
    q0, k0 = torch.randn(gq.shape).bfloat16(), torch.randn(gk.shape).bfloat16()
    _, (dq, dk) = _run_backward(lambda q, k: T.TritonRoPEKernel.apply(q, k, cos, sin), [q0, k0],
                                (gq, gk), cuda)
    # bf16 tables: every product and sum rounded, as the PyTorch path does — bit for bit
    assert torch.equal(dq, G("bwd_rope_dq")) and torch.equal(dk, G("bwd_rope_dk"))


@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 256), (7, 1000), (64, 4096), (3, 4104),
                                       (300, 2048), (2, 8192), (2, 16384), (3, 777), (2, 40000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_norm_backward_shapes(cuda, rows, cols, dtype):
    """Vector path (up to 1024 vectors per row) and scalar path (odd widths, wider rows), all
    dtypes, against the fp32-upcast oracle; LayerNorm also without weight / bias."""
    g = torch.Generator().manual_seed(rows * 977 + cols)
    x = (torch.randn(rows, cols, generator=g) + 0.2).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    b = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    tol = TOL32[dtype]
    # dw / db are fp32 sums over the rows: their error scales with the largest term, not with the
    # (possibly cancelled) result, so the fp32 bound for them is 1e-4 of max(|ref|, 1 % rms)
    tol_sum = max(tol, 1e-4)
    xc, dyc, wc = x.to(cuda), dy.to(cuda), w.to(cuda)

    dx, dw = T.ops.rmsnorm_backward(dyc, xc, wc, 1e-6)
    rx, rw = R.autograd_ref(lambda a, ww: R.rmsnorm_ref(a, ww, 1e-6), _f(x, w), dy.double())
    assert dx.dtype == dtype and dw.dtype == dtype
    assert rel_err(dx.cpu().double(), rx) <= tol
    assert rel_err(dw.cpu().double(), rw) <= tol_sum
    dx2, none = T.ops.rmsnorm_backward(dyc, xc, wc, 1e-6, need_dw=False)
    assert none is None and torch.equal(dx2, dx)

    dx, dw, db = T.ops.layernorm_backward(dyc, xc, wc, 1e-5)
    rx, rw, rb = R.autograd_ref(lambda a, ww, bb: R.layernorm_ref(a, ww, bb, 1e-5), _f(x, w, b),
                                dy.double())
    assert rel_err(dx.cpu().double(), rx) <= tol
    assert rel_err(dw.cpu().double(), rw) <= tol_sum
    assert rel_err(db.cpu().double(), rb) <= tol_sum
    dx, dw, db = T.ops.layernorm_backward(dyc, xc, None, 1e-5)
    (rx,) = R.autograd_ref(lambda a: R.layernorm_ref(a, None, None, 1e-5), _f(x), dy.double())
    assert dw is None and rel_err(dx.cpu().double(), rx) <= tol
    assert rel_err(db.cpu().double(), dy.double().sum(0)) <= tol_sum


@pytest.mark.parametrize("rows,cols,dtype", [(64, 4096, torch.bfloat16), (5, 1000, torch.bfloat16),
                                             (7, 8192, torch.float16), (3, 4104, torch.float32),
                                             (2, 40000, torch.bfloat16), (300, 512, torch.float32)])
def test_residual_norm_backward(cuda, rows, cols, dtype):
    """Residual forms: the gradient of norm(x + r) at the fp32 sum, one tensor for x and r, through
    the fused kernel classes' autograd functions, against the float64 oracle."""
    g = torch.Generator().manual_seed(rows * 13 + cols)
    x = (torch.randn(rows, cols, generator=g) + 0.2).to(dtype)
    r = (torch.randn(rows, cols, generator=g) * 2).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    b = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    tol, tol_sum = TOL32[dtype], max(TOL32[dtype], 1e-4)
    _, (dx, dr, dw) = _run_backward(
        lambda a, rr, ww: T.TritonFusedResidualRMSNormKernel.apply(a, rr, ww, 1e-6), [x, r, w], dy, cuda)
    rx, rr_, rw = R.autograd_ref(lambda a, rr, ww: R.residual_rmsnorm_ref(a, rr, ww, 1e-6),
                                 _f(x, r, w), dy.double())
    assert torch.equal(dx, dr) and dx.dtype == dtype
    assert rel_err(dx.double(), rx) <= tol and rel_err(dr.double(), rr_) <= tol
    assert rel_err(dw.double(), rw) <= tol_sum
    _, (dx, dr, dw, db) = _run_backward(
        lambda a, rr, ww, bb: T.TritonFusedResidualLayerNormKernel.apply(a, rr, ww, bb, 1e-5),
        [x, r, w, b], dy, cuda)
    rx, rr_, rw, rb = R.autograd_ref(lambda a, rr, ww, bb: R.residual_layernorm_ref(a, rr, ww, bb, 1e-5),
                                     _f(x, r, w, b), dy.double())
    assert torch.equal(dx, dr)
    assert rel_err(dx.double(), rx) <= tol
    assert rel_err(dw.double(), rw) <= tol_sum and rel_err(db.double(), rb) <= tol_sum
    # the same numbers as the unfused backward fed the rounded sum, where that sum is exact (fp32)
    if dtype == torch.float32:
        s = (x + r).to(cuda)
        ux, uw = T.ops.rmsnorm_backward(dy.to(cuda), s, w.to(cuda), 1e-6)
        fx, fw = T.ops.rmsnorm_backward(dy.to(cuda), x.to(cuda), w.to(cuda), 1e-6, residual=r.to(cuda))
        assert torch.equal(ux, fx) and torch.equal(uw, fw)


@pytest.mark.parametrize("act", ["mish", "quickgelu", "squared_relu"])
@pytest.mark.parametrize("rows,cols,dtype", [(64, 4096, torch.bfloat16), (5, 1000, torch.bfloat16),
                                             (7, 8192, torch.float16), (3, 4104, torch.float32),
                                             (2, 40000, torch.float32)])
def test_rmsnorm_activation_backward(cuda, act, rows, cols, dtype):
    """act(RMSNorm(x)): the chain rule through the activation inside the norm's backward kernel,
    through the fused kernel class's autograd function, against the float64 oracle."""
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(cols, generator=g)).to(dtype)
    _, (dx, dw) = _run_backward(
        lambda a, ww: T.TritonFusedRMSNormActivationKernel.apply(a, ww, 1e-6, act), [x, w], dy, cuda)
    rx, rw = R.autograd_ref(lambda a, ww: R.rmsnorm_activation_ref(a, ww, 1e-6, act), _f(x, w),
                            dy.double())
    assert dx.dtype == dtype and dw.dtype == dtype
    # fp32: dx = rstd (g - n mean(g n)) with |g| up to some 50 times the rms of dx here (inputs
    # times 3, act' up to 2 z), so its fp32 rounding noise is 1e-4 of max(|ref|, 1 % rms) on both
    # sides of the comparison
    assert rel_err(dx.double(), rx) <= max(TOL32[dtype], 1e-4)
    assert rel_err(dw.double(), rw) <= max(TOL32[dtype], 1e-4)
    # saturation: huge normalised values times huge weights stay finite
    xe = torch.tensor([[300.0, -300.0, 1.0, -1.0, 0.0, 2.0, -2.0, 5.0]]).to(dtype)
    we = torch.full((8,), 100.0).to(dtype)
    de, _ = T.ops.rmsnorm_backward(torch.ones(1, 8).to(dtype).to(cuda), xe.to(cuda), we.to(cuda),
                                   1e-6, activation=act)
    assert bool(torch.isfinite(de.float()).all())


def test_norm_backward_is_deterministic_and_reads_strided_rows(cuda):
    g = torch.Generator().manual_seed(5)
    big = torch.randn(2048, 2 * 4096, generator=g).bfloat16().to(cuda)
    x = big[:, :4096]                      # row stride 8192
    dy = torch.randn(2048, 4096, generator=g).bfloat16().to(cuda)
    w = (1 + 0.1 * torch.randn(4096, generator=g)).bfloat16().to(cuda)
    a = T.ops.rmsnorm_backward(dy, x, w, 1e-6)
    b = T.ops.rmsnorm_backward(dy, x.contiguous(), w, 1e-6)
    c = T.ops.rmsnorm_backward(dy, x, w, 1e-6)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1])
    # fp32 weight with bf16 rows: dw comes back in fp32
    dx, dw = T.ops.rmsnorm_backward(dy, x, w.float(), 1e-6)
    assert dw.dtype == torch.float32 and torch.equal(dx, a[0])
    rx, rw = R.autograd_ref(lambda xx, ww: R.rmsnorm_ref(xx, ww, 1e-6),
                            _f(x.cpu(), w.cpu()), dy.cpu().double())
    assert rel_err(dw.cpu().double(), rw) <= 1e-4
    assert rel_err(dx.cpu().double(), rx) <= 5e-3


@pytest.mark.parametrize("name", ["swiglu", "geglu", "reglu"])
@pytest.mark.parametrize("rows,h,dtype", [(16, 11008, torch.bfloat16), (5, 96, torch.float32),
                                          (3, 777, torch.bfloat16), (7, 520, torch.float16),
                                          (2, 4100, torch.float32), (1, 8, torch.bfloat16)])
def test_glu_backward_shapes(cuda, name, rows, h, dtype):
    g = torch.Generator().manual_seed(rows * 31 + h)
    x = (torch.randn(rows, 2 * h, generator=g) * 3).to(dtype)
    if name == "reglu":  # keep gates off the kink at 0, where the one-sided derivatives differ
        x[:, h:] = torch.where(x[:, h:] == 0, torch.ones_like(x[:, h:]), x[:, h:])
    dy = torch.randn(rows, h, generator=g).to(dtype)
    fn = {"swiglu": R.swiglu_ref, "geglu": R.geglu_ref, "reglu": R.reglu_ref}[name]
    dx = T.ops.glu_backward(dy.to(cuda), x.to(cuda), name).cpu()
    (ref,) = R.autograd_ref(fn, _f(x), dy.double())
    assert dx.dtype == dtype and dx.shape == x.shape
    assert rel_err(dx.double(), ref) <= TOL32[dtype]
    # extreme gates saturate instead of overflowing
    xe = torch.tensor([[1.0, -2.0, 3.0, 0.5, 90.0, -90.0, 30000.0, -30000.0]]).to(dtype)
    de = T.ops.glu_backward(torch.ones(1, 4).to(dtype).to(cuda), xe.to(cuda), name).cpu()
    assert bool(torch.isfinite(de.float()).all())


def test_mirror_modules_train_through_the_kernels(cuda):
    """The mirror modules above their kernel thresholds: loss.backward() reaches the parameters
    and the input through the backward kernels and matches the PyTorch backend of the same module."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 6, 4104, generator=g)
    dy = torch.randn(2, 6, 4104, generator=g)
    for make in (lambda: T.FastRMSNorm(4104, eps=1e-6), lambda: T.FastLayerNorm(4104, eps=1e-5)):
        m = make().to(cuda)
        assert m._check_triton_availability()
        with torch.no_grad():
            m.weight.copy_(1 + 0.1 * torch.randn(4104, generator=g))
        xl = x.to(cuda).requires_grad_(True)
        m(xl).backward(dy.to(cuda))
        ref = make()
        ref.load_state_dict({k: v.cpu() for k, v in m.state_dict().items()})
        xr = x.clone().requires_grad_(True)
        ref._pytorch_forward(xr).backward(dy)
        assert rel_err(xl.grad.cpu(), xr.grad) <= 2e-5
        for (n1, p1), (_, p2) in zip(m.named_parameters(), ref.named_parameters()):
            assert rel_err(p1.grad.cpu(), p2.grad) <= 1e-4, n1  # fp32 sums over the rows
    for make in (lambda: T.FastFusedResidualRMSNorm(4104, eps=1e-6),
                 lambda: T.FastFusedResidualLayerNorm(4104, eps=1e-5)):
        m = make().to(cuda)
        assert m._check_triton_availability()
        with torch.no_grad():
            m.weight.copy_(1 + 0.1 * torch.randn(4104, generator=g))
        res = torch.randn(2, 6, 4104, generator=g)
        xl, rl = x.to(cuda).requires_grad_(True), res.to(cuda).requires_grad_(True)
        m(xl, rl).backward(dy.to(cuda))
        ref = make()
        ref.load_state_dict({k: v.cpu() for k, v in m.state_dict().items()})
        xr, rr = x.clone().requires_grad_(True), res.clone().requires_grad_(True)
        ref._pytorch_forward(xr, rr).backward(dy)
        # both sides are fp32 here (the reference module on the CPU is the yardstick)
        assert rel_err(xl.grad.cpu(), xr.grad) <= 5e-5, rel_err(xl.grad.cpu(), xr.grad)
        assert rel_err(rl.grad.cpu(), rr.grad) <= 5e-5
        for (n1, p1), (_, p2) in zip(m.named_parameters(), ref.named_parameters()):
            assert rel_err(p1.grad.cpu(), p2.grad) <= 1e-4, n1
    xg = torch.randn(3, 5, 2 * 640, generator=g)
    dyg = torch.randn(3, 5, 640, generator=g)
    for cls in (T.FastSwiGLU, T.FastGeGLU, T.FastReGLU):
        xl = xg.to(cuda).requires_grad_(True)
        cls(640)(xl).backward(dyg.to(cuda))
        xr = xg.clone().requires_grad_(True)
        cls(640, use_triton=False)(xr).backward(dyg)
        # ATen's fp32 GELU-tanh backward carries a cancellation error of about 1e-4 of its own
        assert rel_err(xl.grad.cpu(), xr.grad) <= (2e-4 if cls is T.FastGeGLU else 2e-5)


def test_broadcast_gradients_are_materialised(cuda):
    """y.sum().backward() hands the backward a gradient expanded from one scalar (all strides 0)."""
    x = torch.randn(6, 4104, device=cuda, requires_grad=True)
    w = torch.ones(4104, device=cuda, requires_grad=True)
    T.TritonRMSNormKernel.apply(x, w, 1e-6).sum().backward()
    xr, wr = x.detach().cpu().requires_grad_(True), w.detach().cpu().requires_grad_(True)
    R.rmsnorm_ref(xr, wr, 1e-6).sum().backward()
    assert rel_err(x.grad.cpu(), xr.grad) <= 1e-4 and rel_err(w.grad.cpu(), wr.grad) <= 1e-4
    xg = torch.randn(5, 2 * 640, device=cuda, requires_grad=True)
    T.TritonSwiGLUKernel.apply(xg).sum().backward()
    xgr = xg.detach().cpu().requires_grad_(True)
    R.swiglu_ref(xgr).sum().backward()
    assert rel_err(xg.grad.cpu(), xgr.grad) <= 2e-5


def test_forward_only_ops_still_refuse_backward(cuda):
    q = torch.randn(1, 128, 2, 128, device=cuda, dtype=torch.bfloat16, requires_grad=True)
    out = T.TritonAttentionKernel.apply(q, q, q, causal=True)
    with pytest.raises(NotImplementedError):
        out.float().sum().backward()


def test_empty_and_invalid_backward_inputs(cuda):
    w = torch.ones(512, device=cuda, dtype=torch.bfloat16)
    x0 = torch.empty(0, 512, device=cuda, dtype=torch.bfloat16)
    dx, dw = T.ops.rmsnorm_backward(x0, x0, w, 1e-6)
    assert dx.shape == (0, 512) and bool((dw == 0).all())
    dx, dw, db = T.ops.layernorm_backward(x0, x0, w, 1e-5)
    assert dx.shape == (0, 512) and bool((dw == 0).all()) and bool((db == 0).all())
    assert T.ops.glu_backward(torch.empty(0, 256, device=cuda, dtype=torch.bfloat16),
                              x0, "swiglu").shape == (0, 512)
    x = torch.randn(4, 512, device=cuda, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        T.ops.rmsnorm_backward(x[:, :8], x, w, 1e-6)
    with pytest.raises(ValueError):
        T.ops.glu_backward(x, x, "swiglu")
    with pytest.raises(ValueError):
        T.ops.rmsnorm_backward(x.cpu(), x.cpu(), w.cpu(), 1e-6)
