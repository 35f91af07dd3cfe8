"""Own-chunk patterns (full, causal, split:K, block:b, sub-block read) and the one-launch segment form of the attention
kernels against the f32 statement (``ops.reference.attend``) and its autograd."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(n, Cq, Kw, nh, nkv, d, seed, extra=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    return r(n, Cq, nh, d), r(n, Kw + extra, nkv, d), r(n, Kw + extra, nkv, d), r(n, Cq, nkv, d), r(n, Cq, nkv, d), r(n, Cq, nh, d)


def _own_mask(pattern, C, dev):
    from dttt_b200.ops import attention as A
    return A._own_part_mask(pattern, C, dev)


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-12)


@pytest.mark.parametrize("pattern", ["full", "causal", "split:96", "split:128", "block:32", "block:128", "block:256", "read:64", "read:128"])
@pytest.mark.parametrize("Cq,Kw,d", [(256, 512, 64), (512, 0, 64), (256, 256, 128), (384, 0, 128)])
def test_patterns_forward_and_backward(pattern, Cq, Kw, d):
    from dttt_b200.ops import _lib, kernels, reference as ref
    n, nh, nkv = 2, 4, 2
    read = pattern.startswith("read")
    q, kw, vw, ko, vo, g = _mk(n, Cq, Kw, nh, nkv, d, 11, extra=Cq if read else 0)       # read: the clean own chunk follows the window
    scale = d ** -0.5
    K, V = torch.cat([kw, ko], 1), torch.cat([vw, vo], 1)
    mask = _own_mask(pattern, Cq, q.device)
    q32, K32, V32 = (t.float().requires_grad_() for t in (q, K, V))
    want = ref.attend(q32, K32, V32, None, scale, mask)
    if kw.shape[1]:
        o, lse = kernels.attention_fwd(q, kw, vw, scale, pattern, k2=ko, v2=vo)
    else:
        o, lse = kernels.attention_fwd(q, ko, vo, scale, pattern)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.isfinite(o.float()).all()
    assert (o.float() - want).abs().max().item() < 2e-2, pattern
    dqr, dKr, dVr = torch.autograd.grad(want, (q32, K32, V32), g.float())
    if kw.shape[1]:
        dq, dkw, dvw, dko, dvo = kernels.attention_bwd(g, q, kw, vw, o, lse, scale, pattern, k2=ko, v2=vo)
        dk, dv = torch.cat([dkw, dko], 1), torch.cat([dvw, dvo], 1)
    else:
        dq, dk, dv = kernels.attention_bwd(g, q, ko, vo, o, lse, scale, pattern)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(dq, dqr) < 2e-2 and _rel(dk, dKr) < 2e-2 and _rel(dv, dVr) < 2e-2, (pattern, _rel(dq, dqr), _rel(dk, dKr), _rel(dv, dVr))


def _segment_reference(q, k, v, kp, vp, C, W, first, reach, patterns, scale):
    """Chunk by chunk with the f32 statement: ``q [B, S, T, nh, d]`` etc.  Returns ``o`` like ``q``."""
    from dttt_b200.ops import attention as A, reference as ref
    B, S, T = q.shape[:3]
    WC = W * C
    pad = lambda own, prev: torch.cat([own.new_zeros((B, WC) + tuple(own.shape[2:])) if prev is None else prev, own], 1)
    kc, vc = pad(k[:, 1], kp), pad(v[:, 1], vp)
    outs = []
    for s in range(S):
        row = []
        for c in range(T // C):
            nv = A.valid_window_chunks(first + c, W, reach)
            sl = slice(c * C, (c + 1) * C)
            Kc = torch.cat([kc[:, WC + (c - nv) * C:WC + c * C], k[:, s, sl]], 1)
            Vc = torch.cat([vc[:, WC + (c - nv) * C:WC + c * C], v[:, s, sl]], 1)
            row.append(ref.attend(q[:, s, sl], Kc, Vc, None, scale, A._own_part_mask(patterns[s], C, q.device)))
        outs.append(torch.cat(row, 1))
    return torch.stack(outs, 1)


@pytest.mark.parametrize("B,S,chunks,C,W,first,reach,with_prev,patterns", [
    (2, 3, 4, 128, 2, 0, None, False, ("full", "full", "causal")),
    (1, 3, 3, 256, 2, 4, None, True, ("full", "full", "causal")),
    (2, 2, 5, 128, 3, 2, 2, True, ("full", "full")),
    (1, 4, 2, 128, 4, 0, None, False, ("full", "block:64", "split:32", "causal")),
    (1, 3, 8, 128, 8, 8, None, True, ("full", "full", "causal")),
    # the suffix's use: the read and the clean pass of ONE chunk, `first` = number of valid window chunks
    (2, 2, 1, 128, 2, 1, None, True, ("full", "full")),
    (2, 2, 1, 256, 2, 0, None, True, ("full", "full")),
    (1, 3, 1, 128, 4, 4, None, True, ("full", "full", "full")),
])
@pytest.mark.parametrize("d", [64, 128])
def test_segment_form_matches_chunk_by_chunk(B, S, chunks, C, W, first, reach, with_prev, patterns, d):
    from dttt_b200.ops import _lib, attention as A
    nh, nkv = 4, 2
    T = chunks * C
    g = torch.Generator(device="cuda").manual_seed(21)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v, go = r(B, S, T, nh, d), r(B, S, T, nkv, d), r(B, S, T, nkv, d), r(B, S, T, nh, d)
    kp, vp = (r(B, W * C, nkv, d), r(B, W * C, nkv, d)) if with_prev else (None, None)
    gtk, gtv = r(B, W * C, nkv, d), r(B, W * C, nkv, d)
    scale = d ** -0.5
    assert A.segment_attention_ok(q, C, W, patterns)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)] + ([t.clone().requires_grad_(True) for t in (kp, vp)] if with_prev else [])
    o, tk, tv = A.segment_attention(leaves[0], leaves[1], leaves[2], (leaves[3], leaves[4]) if with_prev else None, C, W, first, reach, patterns, scale)
    got = torch.autograd.grad([o, tk, tv], leaves, [go, gtk, gtv])
    torch.cuda.synchronize()
    _lib.check_status()
    f = [t.float().clone().requires_grad_(True) for t in (q, k, v)] + ([t.float().clone().requires_grad_(True) for t in (kp, vp)] if with_prev else [])
    want_o = _segment_reference(f[0], f[1], f[2], f[3] if with_prev else None, f[4] if with_prev else None, C, W, first, reach, patterns, scale)
    WC = W * C
    pad = lambda own, prev: torch.cat([own.new_zeros((B, WC) + tuple(own.shape[2:])) if prev is None else prev, own], 1)
    want_tk, want_tv = pad(f[1][:, 1], f[3] if with_prev else None)[:, T:], pad(f[2][:, 1], f[4] if with_prev else None)[:, T:]
    want = torch.autograd.grad([want_o, want_tk, want_tv], f, [go.float(), gtk.float(), gtv.float()])
    assert (o.float() - want_o).abs().max().item() < 2e-2
    assert torch.equal(tk.float(), want_tk.detach()) and torch.equal(tv.float(), want_tv.detach())
    for name, a, b in zip(("dq", "dk", "dv", "dk_prev", "dv_prev"), got, want):
        assert _rel(a, b) < 3e-2, (name, _rel(a, b))
