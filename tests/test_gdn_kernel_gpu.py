"""The blocked gated-delta-rule kernel (forward and backward) against the token-sequential f32 / f64 recurrence and its
autograd (reference src/ttt/gdn.py:125-136 is the oracle)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, C, nh, D, seed, scale_v=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    k = torch.nn.functional.normalize(r(B, C, nh, D), dim=-1)
    v = scale_v * r(B, C, nh, D)
    beta = torch.sigmoid(r(B, C, nh))
    log_alpha = -0.1 * torch.rand(B, C, nh, device="cuda", generator=g)
    S0 = 0.1 * r(B, nh, D, D)
    return k, v, beta, log_alpha, S0


def _rel(a, b):
    return float((a.double() - b.double()).norm() / (b.double().norm() + 1e-30))


@pytest.mark.parametrize("D,C", [(64, 64), (128, 256), (128, 1024), (64, 1024)])
def test_forward_matches_the_token_recurrence(D, C):
    from dttt_b200.ops import kernels, reference as ref
    k, v, beta, la, S0 = _inputs(2, C, 3, D, 5)
    out = kernels.gdn_chunk_fwd(k, v, beta, la, S0)
    want = ref.gdn_update_sequential(k.double(), v.double(), beta.double(), torch.exp(la.double()), S0.double())
    assert torch.isfinite(out).all()
    assert _rel(out, want) < 1e-4


@pytest.mark.parametrize("D,C", [(64, 64), (64, 192), (128, 128), (128, 1024)])
def test_backward_matches_autograd_of_the_recurrence(D, C):
    from dttt_b200.ops import gdn_scan, reference as ref
    B, nh = 2, 2
    k, v, beta, la, S0 = _inputs(B, C, nh, D, 9)
    leaves = [t.clone().requires_grad_(True) for t in (k, v, beta, la, S0)]
    out = gdn_scan.delta_rule_chunked(*leaves, 64)
    probe = torch.randn(out.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    got = torch.autograd.grad((out * probe).sum(), leaves)
    ref_leaves = [t.double().clone().requires_grad_(True) for t in (k, v, beta, la, S0)]
    rk, rv, rb, rla, rS = ref_leaves
    want_out = ref.gdn_update_sequential(rk, rv, rb, torch.exp(rla), rS)
    want = torch.autograd.grad((want_out * probe.double()).sum(), ref_leaves)
    assert _rel(out, want_out) < 1e-4
    for name, a, b in zip(("dk", "dv", "dbeta", "dlog_alpha", "dS0"), got, want):
        assert torch.isfinite(a).all(), name
        assert _rel(a, b) < 1e-3, (name, _rel(a, b))


def test_model_shape_stays_finite():
    """The hybrid's own shape (one sequence, 1024 tokens, 16 heads of 128) with inputs as the model produces them: keys
    normalised in bf16 (norms slightly off one), gates close to one."""
    from dttt_b200.ops import kernels
    k, v, beta, la, S0 = _inputs(1, 1024, 16, 128, 3, scale_v=0.3)
    k = k.to(torch.bfloat16).float()
    out = kernels.gdn_chunk_fwd(k, v, beta, 0.01 * la, torch.zeros_like(S0))
    assert torch.isfinite(out).all()
