"""The hand-written derivatives of the RMSNorm and SwiGLU backwards (``ops.kernels.rms_norm_bwd2 / swiglu_bwd2``) against
autograd differentiating the plain statements twice (reference src/ttt/model.py:123-134 and its SwiGLU)."""
import pytest
import torch

from dttt_b200.ops import kernels


def _rms_oracle(x, w, g, c, e, eps):
    x, w, g = (t.detach().double().clone().requires_grad_(True) for t in (x, w, g))
    y = w * x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    dx, dw = torch.autograd.grad(y, (x, w), g, create_graph=True)
    L = (c.double() * dx).sum() + ((e.double() * dw).sum() if e is not None else 0.0)
    return torch.autograd.grad(L, (g, x, w))


@pytest.mark.parametrize("with_e", [False, True])
def test_rmsnorm_second_order_formulas(with_e):
    gen = torch.Generator().manual_seed(0)
    rows, D, eps = 6, 16, 1e-5
    x, g, c = (torch.randn(rows, D, generator=gen) for _ in range(3))
    w = torch.rand(D, generator=gen) + 0.5
    e = torch.randn(D, generator=gen) if with_e else None
    want = _rms_oracle(x, w, g, c, e, eps)
    rstd = torch.rsqrt(x.pow(2).mean(-1) + eps)
    got = kernels.rms_norm_bwd2(c, e, g, x, w, rstd)
    for name, a, b in zip(("g", "x", "w"), got, want):
        assert (a.double() - b).abs().max().item() < 1e-4 * (b.abs().max().item() + 1e-9), name


def _swiglu_oracle(g, u, dy, cg, cu):
    g, u, dy = (t.detach().double().clone().requires_grad_(True) for t in (g, u, dy))
    y = torch.nn.functional.silu(g) * u
    dg, du = torch.autograd.grad(y, (g, u), dy, create_graph=True)
    L = (cg.double() * dg).sum() + (cu.double() * du).sum()
    return torch.autograd.grad(L, (dy, g, u))


def test_swiglu_second_order_formulas():
    gen = torch.Generator().manual_seed(1)
    g, u, dy, cg, cu = (torch.randn(4, 24, generator=gen) for _ in range(5))
    want = _swiglu_oracle(g, u, dy, cg, cu)
    got = kernels.swiglu_bwd2(cg, cu, dy, g, u)
    for name, a, b in zip(("dy", "g", "u"), got, want):
        assert (a.double() - b).abs().max().item() < 1e-5 * (b.abs().max().item() + 1e-9), name


@pytest.mark.gpu
@pytest.mark.parametrize("rows,D", [(64, 2048), (1000, 64), (16, 4096), (8, 256)])
@pytest.mark.parametrize("with_e", [False, True])
def test_rmsnorm_second_order_kernel(rows, D, with_e):
    from dttt_b200.ops import _lib
    assert kernels.available("elementwise_bwd2"), "the second-order elementwise kernels are not in the loaded library"
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(rows)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    x, g, c = (bf(torch.randn(rows, D, generator=gen)) for _ in range(3))
    w = (torch.rand(D, generator=gen) + 0.5).to(dev)
    e = torch.randn(D, generator=gen).to(dev) if with_e else None
    eps = 1e-5
    up = lambda t: None if t is None else t.float().cpu()
    want = _rms_oracle(up(x), up(w), up(g), up(c), up(e), eps)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + eps)
    got = kernels.rms_norm_bwd2(c, e, g, x, w, rstd)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, a, b in zip(("g", "x", "w"), got, want):
        rel = (a.double().cpu() - b).norm().item() / (b.norm().item() + 1e-30)
        assert rel < 1e-2, (name, rel)


@pytest.mark.gpu
def test_swiglu_second_order_kernel_and_staged_ops_under_a_recorded_backward():
    from dttt_b200.ops import _lib, functional as Fn
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(5)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    g, u, dy, cg, cu = (bf(torch.randn(64, 512, generator=gen)) for _ in range(5))
    want = _swiglu_oracle(*(t.float().cpu() for t in (g, u, dy, cg, cu)))
    got = kernels.swiglu_bwd2(cg, cu, dy, g, u)
    torch.cuda.synchronize()
    for name, a, b in zip(("dy", "g", "u"), got, want):
        rel = (a.double().cpu() - b).norm().item() / (b.norm().item() + 1e-30)
        assert rel < 1e-2, (name, rel)
    # the staged ops differentiated twice: kernel derivatives against the reference statements
    w = (torch.rand(512, generator=gen) + 0.5).to(dev).to(torch.bfloat16)

    def run(flag):
        kernels.SECOND_ORDER_ELEMENTWISE = flag
        try:
            gg, uu = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
            ww = w.clone().requires_grad_(True)
            y = Fn.rms_norm(Fn.glu(gg, uu, "silu"), ww, 1e-5)
            first = torch.autograd.grad((y.float() * dy.float()).sum(), (gg, uu), create_graph=True)
            L = (first[0].float() * cg.float()).sum() + (first[1].float() * cu.float()).sum()
            return torch.autograd.grad(L, (gg, uu, ww))
        finally:
            kernels.SECOND_ORDER_ELEMENTWISE = True

    a, b = run(True), run(False)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, x1, x0 in zip(("g", "u", "w"), a, b):
        rel = (x1.double() - x0.double()).norm().item() / (x0.double().norm().item() + 1e-30)
        assert rel < 3e-2, (name, rel)
