"""Fast-weight gradients summed in one f32 buffer by the products that use the bf16 copy (``ops.gemm.cast_acc``), on the
CPU with the kernels replaced by their PyTorch statements: same gradients as the chain of bf16 tensors that autograd adds
up, through a read, a recorded inner gradient and a second chunk's copy whose only consumer reports through the buffer."""
import pytest
import torch

from dttt_b200.ops import functional as Fn
from dttt_b200.ops import gemm


def _rel(u, v):
    return float((u.double() - v.double()).norm() / (v.double().norm() + 1e-30))


def _chain(acc: bool, monkeypatch):
    monkeypatch.setattr(gemm, "EMULATE", True)
    monkeypatch.setattr(gemm, "CAST_ACC", acc)
    torch.manual_seed(3)
    B, C, H, I = 2, 16, 32, 64
    W = (torch.randn(B, H, I) * 0.1).requires_grad_(True)
    x1 = torch.randn(B, C, H).bfloat16().requires_grad_(True)
    x2 = torch.randn(B, C, H).bfloat16()
    hits = [0]
    orig = gemm._acc_into

    def spy(*a):
        r = orig(*a)
        hits[0] += bool(r)
        return r
    monkeypatch.setattr(gemm, "_acc_into", spy)
    cast = gemm.cast_acc if acc else (lambda t: t.to(torch.bfloat16))
    Wc = cast(W)
    read = gemm.mm(x1, Wc)
    inner = (gemm.mm(x2, Wc).float().tanh() ** 2).sum()
    with Fn.inner_backward():
        (g,) = torch.autograd.grad(inner, [Wc], create_graph=True)
    assert g.dtype == torch.bfloat16 and g.requires_grad                 # the recorded pass returns ordinary gradients
    W2c = cast(W - 0.1 * g.float())
    out = gemm.mm(x1, W2c).float().sum() + read.float().pow(2).sum()
    out.backward()
    return W.grad, x1.grad, hits[0]


def test_buffer_sums_match_autograd_sums(monkeypatch):
    gw0, gx0, h0 = _chain(False, monkeypatch)
    gw1, gx1, h1 = _chain(True, monkeypatch)
    assert h0 == 0 and h1 == 3                                            # the read, the inner forward, the next chunk's product
    assert gw1.dtype == torch.float32 and _rel(gw1, gw0) < 1e-2           # f32 sums against bf16 sums
    assert _rel(gx1.float(), gx0.float()) < 1e-6


def test_cast_fast_uses_the_buffer_only_when_a_gradient_is_wanted(monkeypatch):
    from dttt_b200.ttt import inner as IN
    monkeypatch.setattr(gemm, "EMULATE", True)
    W = [(torch.randn(2, 8, 16), torch.randn(2, 8, 16), torch.randn(2, 16, 8))]
    plain = IN.cast_fast(W, torch.bfloat16)
    assert all(not hasattr(t, "grad_acc") and t.dtype == torch.bfloat16 for t in plain[0])
    Wg = [tuple(t.clone().requires_grad_(True) for t in W[0])]
    tracked = IN.cast_fast(Wg, torch.bfloat16)
    assert all(hasattr(t, "grad_acc") for t in tracked[0])
    with torch.no_grad():
        assert all(not hasattr(t, "grad_acc") for t in IN.cast_fast(Wg, torch.bfloat16)[0])
    monkeypatch.setattr(gemm, "CAST_ACC", False)
    assert all(not hasattr(t, "grad_acc") for t in IN.cast_fast(Wg, torch.bfloat16)[0])


def test_no_contribution_and_direct_gradient(monkeypatch):
    """A copy that also receives an ordinary gradient (a consumer outside the GEMM) adds it to the buffer; one that
    receives nothing returns nothing."""
    monkeypatch.setattr(gemm, "EMULATE", True)
    W = torch.randn(2, 8, 16).requires_grad_(True)
    x = torch.randn(2, 4, 8).bfloat16()
    Wc = gemm.cast_acc(W)
    (gemm.mm(x, Wc).float().sum() + Wc.float().sum()).backward()
    ref = torch.matmul(x.float().transpose(1, 2), torch.ones(2, 4, 16)) + 1.0
    assert _rel(W.grad, ref) < 1e-2
    W2 = torch.randn(2, 8, 16).requires_grad_(True)
    c2 = gemm.cast_acc(W2)
    (c2.float().sum() * 0.0 + W2.sum()).backward()
    assert torch.allclose(W2.grad, torch.ones_like(W2.grad))


def test_copy_written_by_the_step_kernel_is_used_once(monkeypatch):
    """``lo_copy`` (the bf16 copy a fused step wrote beside its f32 result) replaces the cast: with a gradient wanted it
    becomes the tracked copy, without one it is returned as it is; a second cast of the same tensor makes its own copy."""
    from dttt_b200.ttt import inner as IN
    monkeypatch.setattr(gemm, "EMULATE", True)
    w = torch.randn(2, 8, 16)
    marker = w.to(torch.bfloat16) + 1.0                                  # recognisably not w.to(bf16)
    w.lo_copy = marker
    got = IN.cast_fast([(w, w.clone(), w.clone())], torch.bfloat16)[0]
    assert got[0] is marker and w.lo_copy is None
    assert torch.equal(IN.cast_fast([(w, w, w)], torch.bfloat16)[0][0], w.to(torch.bfloat16))
    wg = torch.randn(2, 8, 16).requires_grad_(True)
    wg.lo_copy = marker
    c = IN.cast_fast([(wg, wg, wg)], torch.bfloat16)[0][0]
    assert torch.equal(c, marker) and c.requires_grad and hasattr(c, "grad_acc") and wg.lo_copy is None
    x = torch.randn(2, 4, 8).bfloat16()
    gemm.mm(x, c).float().sum().backward()
    assert wg.grad is not None and wg.grad.dtype == torch.float32


def test_a_partial_backward_leaves_nothing_behind(monkeypatch):
    """A gradient taken w.r.t. an activation only runs the products' backward, not the copy's own node; what those products
    put into the buffer must not be counted again by a later full backward over the same graph."""
    monkeypatch.setattr(gemm, "EMULATE", True)
    W = torch.randn(2, 8, 16).requires_grad_(True)
    x = torch.randn(2, 4, 8).bfloat16().requires_grad_(True)
    y = gemm.mm(x, gemm.cast_acc(W)).float().sum()
    torch.autograd.grad(y, [x], retain_graph=True)
    y.backward()
    ref = torch.matmul(x.detach().float().transpose(1, 2), torch.ones(2, 4, 16))
    assert _rel(W.grad, ref) < 1e-2
