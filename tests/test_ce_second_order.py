"""The hand-written derivative of the cross-entropy backward (``ops.ce.second_order``) against autograd differentiating the
dense statement twice (the reference differentiates its fused cross-entropy's VJP, reference src/ttt/fused_ce.py:84-121)."""
import pytest
import torch

from dttt_b200.ops import ce


def _oracle(g, h, E, y, w, c):
    g, h, E, w = (t.detach().double().clone().requires_grad_(True) for t in (g, h, E, w))
    z = h @ E.t()
    loss = (w * (torch.logsumexp(z, -1) - z.gather(-1, y[:, None]).squeeze(-1))).sum()
    (g_h,) = torch.autograd.grad(loss, h, g, create_graph=True)
    L = (c.double() * g_h).sum()
    return torch.autograd.grad(L, (g, h, E, w)), torch.logsumexp(z, -1).detach(), g_h.detach()


def _case(N, H, V, seed=0):
    gen = torch.Generator().manual_seed(seed)
    h = torch.randn(N, H, generator=gen)
    E = torch.randn(V, H, generator=gen) * 0.3
    y = torch.randint(0, V, (N,), generator=gen)
    w = torch.rand(N, generator=gen)
    c = torch.randn(N, H, generator=gen)
    g = torch.tensor(0.7)
    return g, h, E, y, w, c


def test_ce_second_order_formulas_match_autograd_of_autograd():
    g, h, E, y, w, c = _case(12, 8, 20)
    (wg, wh, wE, ww), logZ, _ = _oracle(g, h, E, y, w, c)
    g_g, g_h, r, d, g_w = ce.second_order(c, g, h, E, y, w, logZ.float())
    g_E = r.t() @ h + d.t() @ c
    for name, got, want in (("g", g_g, wg), ("h", g_h, wh), ("E", g_E, wE), ("w", g_w, ww)):
        err = (got.double() - want).abs().max().item() / (want.abs().max().item() + 1e-12)
        assert err < 1e-5, (name, err)


@pytest.mark.gpu
def test_ce_row_kernels_and_second_order_on_the_gpu():
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("linear_ce_bwd2"), "the second-order cross-entropy kernels are not in the loaded library"
    dev = torch.device("cuda", 0)
    N, H, V = 256, 128, 1000
    g, h, E, y, w, c = _case(N, H, V, seed=2)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    hb, Eb, cb = bf(h), bf(E), bf(c)
    (wg, wh, wE, ww), logZ, _ = _oracle(g, hb.float().cpu(), Eb.float().cpu(), y, w, cb.float().cpu())
    g_g, g_h, r, d, g_w = ce.second_order(cb, g.to(dev), hb, Eb, y.to(dev), w.to(dev), logZ.float().to(dev))
    g_E = r.float().t() @ hb.float() + d.float().t() @ cb.float()
    torch.cuda.synchronize()
    _lib.check_status()
    rel = lambda a, b: (a.double().cpu() - b).norm().item() / (b.norm().item() + 1e-30)
    assert rel(g_g, wg) < 1e-2 and rel(g_h, wh) < 2e-2 and rel(g_E, wE) < 2e-2 and rel(g_w, ww) < 1e-2, \
        (rel(g_g, wg), rel(g_h, wh), rel(g_E, wE), rel(g_w, ww))


@pytest.mark.gpu
def test_weighted_ce_meta_gradient_with_the_differentiable_backward():
    """``weighted_ce`` differentiated twice in the inner-pass setting: kernel path against the dense statement."""
    from dttt_b200.ops import _lib, functional as Fn
    dev = torch.device("cuda", 0)
    N, H, V = 256, 128, 1024
    g, h, E, y, w, c = _case(N, H, V, seed=4)
    hb = h.to(dev).to(torch.bfloat16)
    Eb = E.to(dev).to(torch.bfloat16)
    yd, wd, cd = y.to(dev), w.to(dev), c.to(dev).to(torch.bfloat16)

    def run(flag):
        ce.SECOND_ORDER_KERNEL = flag
        try:
            hh = hb.clone().requires_grad_(True)
            EE = Eb.clone().requires_grad_(True)
            loss = ce.weighted_ce(hh, EE, yd, wd, block=512)
            with Fn.inner_backward():
                (g_h,) = torch.autograd.grad(loss, hh, create_graph=True)
            L = (cd.float() * g_h.float()).sum()
            return g_h.detach(), torch.autograd.grad(L, (hh, EE))
        finally:
            ce.SECOND_ORDER_KERNEL = True

    f1, s1 = run(True)
    f0, s0 = run(False)
    torch.cuda.synchronize()
    _lib.check_status()
    rel = lambda a, b: (a.double() - b.double()).norm().item() / (b.double().norm().item() + 1e-30)
    assert rel(f1, f0) < 2e-2
    assert rel(s1[0], s0[0]) < 3e-2 and rel(s1[1], s0[1]) < 3e-2, (rel(s1[0], s0[0]), rel(s1[1], s0[1]))
