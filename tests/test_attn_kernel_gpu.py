"""The tcgen05 flash-attention forward kernel against an f32 softmax(QK^T)V."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, scale, causal):
    n, Cq, nh, d = q.shape
    Kn, nkv = k.shape[1], k.shape[2]
    rep = nh // nkv
    q32 = q.float().permute(0, 2, 1, 3)                                   # [n, nh, Cq, d]
    k32 = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    v32 = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = q32 @ k32.transpose(-1, -2) * scale
    if causal:
        i = torch.arange(Cq, device=q.device)[:, None]
        j = torch.arange(Kn, device=q.device)[None, :]
        s = s.masked_fill(j > i + (Kn - Cq), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v32
    return o.permute(0, 2, 1, 3), lse


@pytest.mark.parametrize("n,Cq,Kn,nh,nkv,d,causal", [
    (2, 128, 128, 4, 2, 64, True),
    (2, 128, 128, 4, 2, 64, False),
    (1, 256, 1280, 8, 2, 64, True),
    (1, 256, 1280, 8, 2, 64, False),
    (2, 200, 333, 4, 4, 128, False),
    (1, 100, 100, 2, 1, 64, True),
    (1, 384, 640, 4, 1, 128, True),
    (1, 1024, 9216, 8, 2, 64, True),
    (2, 640, 1664, 4, 2, 64, True),
    (1, 512, 512, 4, 2, 128, True),
])
@pytest.mark.parametrize("variant", [0, 1])
def test_attn_fwd(n, Cq, Kn, nh, nkv, d, causal, variant):
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("attention"), "the attention kernel is not in the loaded library"
    torch.manual_seed(3)
    q = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    o, lse = kernels.attention_fwd(q, k, v, scale, causal, variant)
    torch.cuda.synchronize()
    _lib.check_status()
    oref, lref = _ref(q, k, v, scale, causal)
    err = (o.float() - oref).abs().max().item()
    assert err < 2e-2, err
    assert (lse - lref).abs().max().item() < 2e-3


@pytest.mark.parametrize("variant", [0, 1])
def test_attn_fwd_large_magnitude(variant):
    """Scores far from zero: the running-max rescale has to carry the sum across key blocks."""
    from dttt_b200.ops import kernels
    torch.manual_seed(4)
    n, Cq, Kn, nh, nkv, d = 1, 128, 512, 2, 2, 64
    q = 4.0 * torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    k = 4.0 * torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    o, lse = kernels.attention_fwd(q, k, v, d ** -0.5, False, variant)
    oref, lref = _ref(q, k, v, d ** -0.5, False)
    assert (o.float() - oref).abs().max().item() < 3e-2
    assert ((lse - lref).abs() / lref.abs().clamp_min(1.0)).max().item() < 2e-3


@pytest.mark.parametrize("n,Cq,Kn,nh,nkv,causal", [
    (1, 128, 128, 1, 1, False),
    (1, 128, 128, 2, 1, True),
    (2, 256, 640, 4, 2, True),
    (2, 256, 640, 4, 2, False),
    (1, 200, 333, 4, 4, False),
    (1, 100, 100, 2, 1, True),
    (1, 1024, 3072, 8, 2, True),
])
@pytest.mark.parametrize("d", [64, 128])
def test_attn_bwd(n, Cq, Kn, nh, nkv, causal, d):
    from dttt_b200.ops import _lib, kernels
    assert kernels.available("attention_bwd")
    torch.manual_seed(5)
    q = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    o, lse = kernels.attention_fwd(q, k, v, scale, causal)
    dq, dk, dv = kernels.attention_bwd(g, q, k, v, o, lse, scale, causal)
    torch.cuda.synchronize()
    _lib.check_status()
    q32, k32, v32 = (t.float().requires_grad_() for t in (q, k, v))
    oref, _ = _ref(q32, k32, v32, scale, causal)
    dqr, dkr, dvr = torch.autograd.grad(oref, (q32, k32, v32), g.float())
    rel = lambda a, b: (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-12)
    assert rel(dv, dvr) < 2e-2, ("dv", rel(dv, dvr))
    assert rel(dk, dkr) < 2e-2, ("dk", rel(dk, dkr))
    assert rel(dq, dqr) < 2e-2, ("dq", rel(dq, dqr))


@pytest.mark.parametrize("n,Cq,Kw,nh,nkv,causal", [(2, 256, 512, 4, 2, True), (2, 256, 512, 4, 2, False), (1, 1024, 2048, 8, 2, True), (3, 128, 128, 2, 1, True)])
@pytest.mark.parametrize("d", [64, 128])
def test_two_segment_keys_equal_the_concatenation(n, Cq, Kw, nh, nkv, causal, d):
    """Window keys (a strided slice of a longer window buffer) and own keys passed as separate tensors: forward and backward
    must equal the single-tensor call on their concatenation."""
    from dttt_b200.ops import _lib, kernels
    torch.manual_seed(6)
    q = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    win_k = torch.randn(n, Kw + 256, nkv, d, device="cuda", dtype=torch.bfloat16)
    win_v = torch.randn(n, Kw + 256, nkv, d, device="cuda", dtype=torch.bfloat16)
    kw, vw = win_k[:, 256:], win_v[:, 256:]                                   # not contiguous across sequences
    ko = torch.randn(n, Cq, nkv, d, device="cuda", dtype=torch.bfloat16)
    vo = torch.randn(n, Cq, nkv, d, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    scale = d ** -0.5
    o2, lse2 = kernels.attention_fwd(q, kw, vw, scale, causal, k2=ko, v2=vo)
    K, V = torch.cat([kw, ko], 1), torch.cat([vw, vo], 1)
    o1, lse1 = kernels.attention_fwd(q, K, V, scale, causal)
    assert torch.equal(o1, o2) and torch.equal(lse1, lse2)
    dq2, dkw, dvw, dko, dvo = kernels.attention_bwd(g, q, kw, vw, o2, lse2, scale, causal, k2=ko, v2=vo)
    dq1, dk1, dv1 = kernels.attention_bwd(g, q, K, V, o1, lse1, scale, causal)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(torch.cat([dkw, dko], 1), dk1) and torch.equal(torch.cat([dvw, dvo], 1), dv1)
    assert (dq2.float() - dq1.float()).abs().max().item() < 2e-2 * dq1.float().abs().max().item()      # bulk reductions add in any order
