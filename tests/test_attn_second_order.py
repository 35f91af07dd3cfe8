"""The hand-written derivative of the attention backward (``ops.attn_second``) against autograd differentiating
the plain statement twice (the reference differentiates ``attend_xla`` twice, reference src/ttt/attention.py:181-201)."""
import math

import pytest
import torch

from dttt_b200.ops import attn_second


def _statement(q, K, V, scale, causal):
    n, C, nh, d = q.shape
    Kn, nkv = K.shape[1], K.shape[2]
    G = nh // nkv
    Kh = K.repeat_interleave(G, dim=2)
    Vh = V.repeat_interleave(G, dim=2)
    s = torch.einsum("nchd,nkhd->nhck", q, Kh) * scale
    if causal:
        i = torch.arange(C)[:, None]
        j = torch.arange(Kn)[None, :]
        s = s.masked_fill(j > i + (Kn - C), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("nhck,nkhd->nchd", torch.softmax(s, -1), Vh)
    return o, lse


def _case(n, C, Kn, nh, nkv, d, causal, dtype=torch.float64, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=dtype)
    q, K, V, dO = r(n, C, nh, d), r(n, Kn, nkv, d), r(n, Kn, nkv, d), r(n, C, nh, d)
    cots = r(n, C, nh, d), r(n, Kn, nkv, d), r(n, Kn, nkv, d)
    return q, K, V, dO, cots


def _autograd_twice(q, K, V, dO, cots, scale, causal):
    q, K, V, dO = (t.detach().clone().requires_grad_(True) for t in (q, K, V, dO))
    o, lse = _statement(q, K, V, scale, causal)
    first = torch.autograd.grad(o, (q, K, V), dO, create_graph=True)
    L = sum((c * f).sum() for c, f in zip(cots, first))
    return torch.autograd.grad(L, (dO, q, K, V)), o.detach(), lse.detach()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 8, 24, 4, 2, 8), (1, 4, 4, 2, 2, 4), (1, 16, 48, 4, 1, 8)])
def test_second_order_formulas_match_autograd_of_autograd(shape, causal):
    n, C, Kn, nh, nkv, d = shape
    scale = 1.0 / math.sqrt(d)
    q, K, V, dO, cots = _case(*shape, causal)
    want, o, lse = _autograd_twice(q, K, V, dO, cots, scale, causal)
    got = attn_second.second_order(*(c.float() for c in cots), dO.float(), q.float(), K.float(), V.float(), o.float(), lse.float(),
                                   scale, causal)
    for name, w, g in zip(("dO", "q", "K", "V"), want, got):
        err = (g.double() - w).abs().max().item() / (w.abs().max().item() + 1e-12)
        assert err < 2e-5, (name, err)


def test_missing_cotangents_count_as_zero():
    shape = (1, 8, 16, 2, 1, 8)
    scale = 0.3
    q, K, V, dO, cots = _case(*shape, True)
    zero = (cots[0], torch.zeros_like(cots[1]), torch.zeros_like(cots[2]))
    want, o, lse = _autograd_twice(q, K, V, dO, zero, scale, True)
    got = attn_second.second_order(cots[0].float(), None, None, dO.float(), q.float(), K.float(), V.float(), o.float(), lse.float(), scale, True)
    for w, g in zip(want, got):
        assert (g.double() - w).abs().max().item() <= 2e-5 * (w.abs().max().item() + 1e-12) + 1e-9


# ------------------------------------------------------------------------------------------------ on the GPU
def _f64_oracle(q, K, V, dO, cots, scale, causal):
    up = lambda t: t.detach().double().cpu()
    want, o, lse = _autograd_twice(up(q), up(K), up(V), up(dO), tuple(up(c) for c in cots), scale, causal)
    return want, o, lse


def _rel(got, want):
    return (got.double().cpu() - want).norm().item() / (want.norm().item() + 1e-30)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,Kn,C,causal", [(64, 1024, 32, True), (48, 2052, 16, False), (16, 9216, 8, True), (8, 10240, 8, True), (32, 36, 16, True)])
def test_row_kernel_matches_the_row_statement(rows, Kn, C, causal):
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("attention_bwd2"), "the second-order row kernel is not in the loaded library"
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(Kn)
    r = lambda *s: torch.randn(*s, generator=g).to(dev)
    S, dP, gdS, X = r(rows, Kn) * 3, r(rows, Kn), r(rows, Kn), r(rows, Kn)
    scale = 0.37
    s = S * scale
    if causal:
        c = torch.arange(rows, device=dev) % C
        j = torch.arange(Kn, device=dev)
        s = s.masked_fill(j[None, :] > c[:, None] + (Kn - C), float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.softmax(s, -1)
    delta = (p * dP).sum(-1)
    want = attn_second._rows_torch(S.double(), dP.double(), gdS.double(), X.double(), lse.double(), delta.double(), C, causal, scale)
    got = kernels.attention_bwd2_rows(S, dP, gdS, X, lse, delta, C, causal, scale)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, w, gt in zip(("P", "dS", "gdP", "gS"), want, got):
        assert (gt.double() - w).abs().max().item() <= 1e-2 * w.abs().max().item() + 1e-6, name
        assert (gt.double() - w).norm().item() <= 4e-3 * w.norm().item(), name


@pytest.mark.gpu
@pytest.mark.parametrize("n,C,Kn,nh,nkv,causal", [(1, 128, 384, 4, 2, True), (2, 256, 256, 8, 2, True), (1, 128, 640, 4, 1, False), (1, 256, 1088, 2, 1, True)])
def test_score_kernel_matches_the_row_statement(n, C, Kn, nh, nkv, causal):
    """The tcgen05 score stage against the f64 row statement applied to f64 score products."""
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("attention_bwd2_scores"), "the second-order score kernel is not in the loaded library"
    d = 64
    dev = torch.device("cuda", 0)
    scale = 1.0 / math.sqrt(d)
    q, K, V, dO, cots = _case(n, C, Kn, nh, nkv, d, causal, dtype=torch.float32, seed=5)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    q, K, V, dO = bf(q), bf(K), bf(V), bf(dO)
    gQ, gK, gV = (bf(c) for c in cots)
    up = lambda t: t.double().cpu()
    o, lse = _statement(up(q), up(K), up(V), scale, causal)
    delta = (up(dO) * o).sum(-1).permute(0, 2, 1).contiguous()                        # [n, nh, C]
    got = kernels.attention_bwd2_scores(q, dO, gQ, K, V, gK, gV, lse.float().to(dev), delta.float().to(dev), scale, causal)
    torch.cuda.synchronize()
    _lib.check_status()
    T = lambda t: t.transpose(-1, -2)
    qg, dOg, gQg = (attn_second._rows(up(t), nkv) for t in (q, dO, gQ))
    kg, vg, gKg, gVg = (attn_second._keys(up(t)) for t in (K, V, gK, gV))
    G = nh // nkv
    want = attn_second._rows_torch(qg @ T(kg), dOg @ T(vg), gQg @ T(kg) + qg @ T(gKg), dOg @ T(gVg), lse.reshape(n * nkv, G * C),
                                   delta.reshape(n * nkv, G * C), C, causal, scale)
    for name, w, gt in zip(("P", "dS", "gdP", "gS"), want, got):
        assert gt.shape == w.shape, name
        assert _rel(gt, w) < 6e-3, (name, _rel(gt, w))


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("n,C,Kn,nh,nkv,causal", [(1, 128, 384, 4, 2, True), (2, 256, 256, 8, 2, True), (1, 128, 640, 4, 1, False)])
def test_second_order_on_the_gpu_matches_f64_autograd(n, C, Kn, nh, nkv, causal, fused, monkeypatch):
    from dttt_b200.ops import _lib
    monkeypatch.setattr(attn_second, "FUSED_SCORES", fused)
    d = 64
    dev = torch.device("cuda", 0)
    scale = 1.0 / math.sqrt(d)
    q, K, V, dO, cots = _case(n, C, Kn, nh, nkv, d, causal, dtype=torch.float32)
    bf = lambda t: t.to(dev).to(torch.bfloat16)
    q, K, V, dO = bf(q), bf(K), bf(V), bf(dO)
    cots = tuple(bf(c) for c in cots)
    want, o, lse = _f64_oracle(q, K, V, dO, cots, scale, causal)
    got = attn_second.second_order(*cots, dO, q, K, V, o.to(dev).to(torch.bfloat16), lse.to(dev).float(), scale, causal)
    torch.cuda.synchronize()
    _lib.check_status()
    for name, w, gt in zip(("dO", "q", "K", "V"), want, got):
        assert _rel(gt, w) < 2e-2, (name, _rel(gt, w))


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [True, False])
def test_window_attention_meta_gradient_with_the_differentiable_backward(causal):
    """``attend_window`` differentiated twice: the kernel path (flash backward + hand-written derivative) against the
    reference statement differentiated twice by autograd."""
    from dttt_b200.ops import _lib, attention
    dev = torch.device("cuda", 0)
    n, C, nh, nkv, d, W = 2, 128, 8, 2, 64, 3
    g = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=g).to(dev).to(torch.bfloat16)
    base = [mk(n, C, nh, d), mk(n, C, nkv, d), mk(n, C, nkv, d), mk(n, W * C, nkv, d), mk(n, W * C, nkv, d)]
    w_out = mk(n, C, nh, d)
    cot = [mk(n, C, nh, d), mk(n, C, nkv, d), mk(n, C, nkv, d), mk(n, W * C, nkv, d), mk(n, W * C, nkv, d)]

    def run(flag):
        attention.SECOND_ORDER_KERNEL = flag
        try:
            ins = [t.clone().requires_grad_(True) for t in base]
            o = attention.attend_window(ins[0], ins[1], ins[2], ins[3], ins[4], 2, C, 0.125, own="causal" if causal else "full", inner=True)
            first = torch.autograd.grad((o.float() * w_out.float()).sum(), ins, create_graph=True)
            L = sum((c.float() * f.float()).sum() for c, f in zip(cot, first))
            second = torch.autograd.grad(L, ins, allow_unused=True)
            return [f.detach() for f in first], second
        finally:
            attention.SECOND_ORDER_KERNEL = True

    f1, s1 = run(True)
    f0, s0 = run(False)
    torch.cuda.synchronize()
    _lib.check_status()
    for a, b in zip(f1, f0):
        assert _rel(a, b.double().cpu()) < 2e-2
    for i, (a, b) in enumerate(zip(s1, s0)):
        if b is None:
            continue
        b = b.double().cpu()
        assert _rel(a, b) < 3e-2, (i, _rel(a, b))
