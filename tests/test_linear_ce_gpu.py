"""The cross-entropy epilogues of the tcgen05 GEMM against dense f32 statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K,V", [(256, 256, 1024), (300, 512, 5000), (2048, 2048, 128256), (100, 128, 300)])
def test_linear_ce_fwd(N, K, V):
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("linear_ce")
    torch.manual_seed(0)
    h = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    E = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.randint(0, V, (N,), device="cuda")
    lse, nll = kernels.linear_ce_fwd(h, E, y)
    torch.cuda.synchronize()
    _lib.check_status()
    logits = h.float() @ E.float().t()
    lref = torch.logsumexp(logits, -1)
    nref = lref - logits.gather(1, y[:, None]).squeeze(1)
    assert (lse - lref).abs().max().item() < 2e-3
    assert (nll - nref).abs().max().item() < 2e-3


@pytest.mark.parametrize("N,K,V,s,e", [(256, 256, 1024, 0, 1024), (300, 512, 5000, 2048, 5000), (1024, 2048, 20000, 8192, 16384)])
def test_linear_ce_dlogits(N, K, V, s, e):
    from dttt_b200.ops import _lib, kernels
    torch.manual_seed(1)
    h = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    E = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.randint(0, V, (N,), device="cuda")
    coef = torch.randn(N, device="cuda")
    logits = h.float() @ E.float().t()
    lse = torch.logsumexp(logits, -1)
    D = kernels.linear_ce_dlogits(h, E[s:e], y.to(torch.int32), coef, lse, s)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = torch.softmax(logits, -1)
    ref[torch.arange(N), y] -= 1.0
    ref = (ref * coef[:, None])[:, s:e]
    assert (D.float() - ref).abs().max().item() < 1e-2 * ref.abs().max().item() + 1e-6


def test_weighted_ce_uses_fused_path_and_matches():
    from dttt_b200.ops import ce as CE, kernels
    torch.manual_seed(2)
    N, K, V = 512, 256, 20000
    h = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    E = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    y = torch.randint(0, V, (N,), device="cuda")
    w = torch.rand(N, device="cuda")
    before = kernels.LAUNCHES
    loss = CE.weighted_ce(h, E, y, w, 8192)
    gh, gE = torch.autograd.grad(loss, (h, E))
    assert kernels.LAUNCHES > before, "the fused kernels did not run"
    h32, E32 = h.detach().float().requires_grad_(), E.detach().float().requires_grad_()
    logits = h32 @ E32.t()
    lr = (w * (torch.logsumexp(logits, -1) - logits.gather(1, y[:, None]).squeeze(1))).sum()
    ghr, gEr = torch.autograd.grad(lr, (h32, E32))
    rel = lambda a, b: (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-12)
    assert abs(loss.item() - lr.item()) / lr.item() < 2e-3
    assert rel(gh, ghr) < 3e-2 and rel(gE, gEr) < 3e-2
