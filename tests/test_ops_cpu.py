import math

import pytest
import torch

from dttt_b200.ops import attention as A
from dttt_b200.ops import ce as CE
from dttt_b200.ops import gdn_scan
from dttt_b200.ops import reference as ref


def test_streamed_ce_equals_dense():
    torch.manual_seed(0)
    h, E = torch.randn(50, 16), torch.randn(37, 16)
    y, w = torch.randint(0, 37, (50,)), torch.rand(50)
    assert torch.allclose(CE.per_token_ce(h, E, y, 8), ref.per_token_ce_dense(h, E, y), atol=1e-5)
    ids, lp = CE.topk_logprobs(h, E, 5, 8)
    full = torch.log_softmax(h @ E.t(), -1)
    v, i = full.topk(5, -1)
    assert torch.equal(ids, i) and torch.allclose(lp, v, atol=1e-5)
    q = torch.softmax(v, -1)
    a = ref.soft_ce_dense(h, E, i, q, w)
    assert torch.isfinite(a)


def test_rope_llama3_scaling_and_pos_q():
    inv = ref.rope_inv_freq(64, 500000.0)
    sc = (("factor", 16.0), ("high_freq_factor", 4.0), ("low_freq_factor", 1.0), ("original_max_position_embeddings", 8192), ("rope_type", "llama3"))
    inv_s = ref.rope_inv_freq(64, 500000.0, sc)
    wl = 2 * math.pi / inv
    assert torch.allclose(inv_s[wl < 8192 / 4], inv[wl < 8192 / 4])                  # short wavelengths keep their frequency
    assert torch.allclose(inv_s[wl > 8192], inv[wl > 8192] / 16.0)                   # long ones are slowed by the factor
    x = torch.randn(2, 5, 3, 64)
    cos, sin = ref.rope_cos_sin(torch.arange(5)[None].expand(2, 5), 64, 1e4)
    y = ref.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)                 # a rotation
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)                               # position 0 is the identity


def test_window_geometry():
    x = torch.arange(2 * 24).reshape(2, 24, 1).float()
    g = A.window_gather(x, 4, 2)
    assert g.shape == (2, 6, 8, 1) and (g[:, 0] == 0).all() and torch.equal(g[0, 3, :, 0], torch.arange(4, 12).float())
    prev = torch.full((2, 8, 1), -1.0)
    assert (A.window_gather(x, 4, 2, prev)[:, 0] == -1).all()
    kv = A.key_validity(1, 4, 3)
    assert kv.tolist() == [False] * 8 + [True] * 8
    assert A.key_validity(5, 4, 3, reach=1).tolist() == [False] * 8 + [True] * 8
    assert A.valid_window_chunks(5, 3, 1) == 1 and A.valid_window_chunks(1, 3, None) == 1
    m = A.own_mask_matrix(6, "split:3")
    assert m[0].tolist() == [True] * 3 + [False] * 3 and m[4].tolist() == [True] * 5 + [False]
    assert A.own_mask_matrix(4, "block:2")[1].tolist() == [True, True, False, False]
    r = A.read_mask_matrix(4, 2)
    assert r[2].tolist() == [True, True, False, False, False, False, True, True]


def test_attend_window_equals_explicit_validity():
    torch.manual_seed(1)
    n, C, nh, nkv, d, W = 2, 4, 4, 2, 8, 3
    q, k, v = torch.randn(n, C, nh, d), torch.randn(n, C, nkv, d), torch.randn(n, C, nkv, d)
    kw, vw = torch.randn(n, W * C, nkv, d), torch.randn(n, W * C, nkv, d)
    for nv, own in ((0, "full"), (2, "causal"), (3, "split:2")):
        o = A.attend_window(q, k, v, kw, vw, nv, C, d ** -0.5, own=own)
        valid = A.key_validity(nv, C, W)[None].expand(n, -1)
        o_ref = ref.attend(q, torch.cat([kw, k], 1), torch.cat([vw, v], 1), valid, d ** -0.5, A.own_mask_matrix(C, own))
        assert torch.allclose(o, o_ref, atol=1e-5), (nv, own)


@pytest.mark.parametrize("block", [8, 16, 64])
def test_chunked_delta_rule_equals_token_recurrence(block):
    torch.manual_seed(2)
    B, C, nh, d = 2, 64, 3, 8
    k = torch.nn.functional.normalize(torch.randn(B, C, nh, d), dim=-1)
    v, beta = torch.randn(B, C, nh, d), torch.sigmoid(torch.randn(B, C, nh))
    la = -torch.rand(B, C, nh) * 0.2
    S0 = torch.randn(B, nh, d, d) * 0.1
    a = gdn_scan.delta_rule_chunked(k, v, beta, la, S0, block)
    b = ref.gdn_update_sequential(k, v, beta, torch.exp(la), S0)
    assert torch.allclose(a, b, atol=2e-5)
    S0.requires_grad_(True)
    gdn_scan.delta_rule_chunked(k, v, beta, la, S0, block).sum().backward()        # differentiable
    assert S0.grad is not None
