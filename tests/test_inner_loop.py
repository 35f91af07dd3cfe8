"""The write: batched inner gradient == per-sequence gradients of an unrolled statement; clipping; lr ramp."""
import pytest
import torch

from util import loss_config, make_engine, tiny_model
from dttt_b200.ops import reference as ref
from dttt_b200.ttt import inner as IN


def _setup(B=3):
    eng = make_engine()
    net = eng.net(train=False)
    mc = eng.mc
    C, S = mc.chunk_size, mc.suffix_len
    g = torch.Generator().manual_seed(0)
    h = torch.randn(B, C, mc.hidden_size, generator=g) * 0.5
    toks = torch.randint(0, 120, (B, C), generator=g)
    mask = torch.ones(B, C); mask[:, -1] = 0
    kv = [(torch.randn(B, mc.window_chunks * C, mc.num_key_value_heads, mc.head_dim, generator=g),
           torch.randn(B, mc.window_chunks * C, mc.num_key_value_heads, mc.head_dim, generator=g)) for _ in range(S)]
    pos = torch.arange(2 * C, 3 * C)[None].expand(B, C)
    W = [tuple(t.clone() for t in w) for w in net.template_fast(B)]
    return eng, net, h, toks, mask, kv, pos, W


def test_batched_inner_grad_equals_per_sequence_unrolled():
    eng, net, h, toks, mask, kv, pos, W = _setup()
    g, terms = IN.inner_grad(W, net, h, toks, mask, kv, pos, 2, 0, create_graph=False, pos_q=pos + 1, own="causal")
    mc = eng.mc
    for b in range(h.shape[0]):
        Wb = [tuple(t[b:b + 1].clone().requires_grad_(True) for t in w) for w in W]
        # unrolled: every suffix layer written out with plain reference ops
        x = h[b:b + 1]
        f = 0
        for i in range(mc.suffix_len):
            xn = ref.rms_norm(x, net.p("suffix.attn_norm.weight", i), mc.rms_norm_eps)
            q = (xn @ net.p("suffix.attn.q.weight", i)).unflatten(-1, (mc.num_attention_heads, mc.head_dim))
            k = (xn @ net.p("suffix.attn.k.weight", i)).unflatten(-1, (mc.num_key_value_heads, mc.head_dim))
            v = (xn @ net.p("suffix.attn.v.weight", i)).unflatten(-1, (mc.num_key_value_heads, mc.head_dim))
            q = ref.rms_norm(q, net.p("suffix.attn.q_norm.weight", i), mc.rms_norm_eps)
            k = ref.rms_norm(k, net.p("suffix.attn.k_norm.weight", i), mc.rms_norm_eps)
            cq, sq = ref.rope_cos_sin(pos[b:b + 1] + 1, mc.head_dim, mc.rope_theta)
            ck, sk = ref.rope_cos_sin(pos[b:b + 1], mc.head_dim, mc.rope_theta)
            q, k = ref.apply_rope(q, cq, sq), ref.apply_rope(k, ck, sk)
            K = torch.cat([kv[i][0][b:b + 1], k], 1)
            V = torch.cat([kv[i][1][b:b + 1], v], 1)
            C = mc.chunk_size
            own = torch.tril(torch.ones(C, C, dtype=torch.bool))
            a = ref.attend(q, K, V, None, mc.head_dim ** -0.5, own)
            x = x + a.flatten(-2) @ net.p("suffix.attn.o.weight", i)
            gw, uw, dw = Wb[f]
            xp = ref.rms_norm(x, net.p("prime_norm.weight", f), mc.rms_norm_eps)
            y = (torch.nn.functional.silu(xp @ gw[0]) * (xp @ uw[0])) @ dw[0]
            x = x + ref.rms_norm(y, net.p("prime_post_norm.weight", f), mc.rms_norm_eps)
            f += 1
            xm = ref.rms_norm(x, net.p("suffix.mlp_norm.weight", i), mc.rms_norm_eps)
            x = x + (torch.nn.functional.silu(xm @ net.p("suffix.mlp.gate.weight", i)) * (xm @ net.p("suffix.mlp.up.weight", i))) @ net.p("suffix.mlp.down.weight", i)
        hn = ref.rms_norm(x, net.p("final_norm.weight"), mc.rms_norm_eps)
        w = mask[b] / (mask[b].sum() + 1e-6)
        loss = ref.weighted_ce_dense(hn[0], net.p("embed"), toks[b], w)
        gb = torch.autograd.grad(loss, [t for w_ in Wb for t in w_])
        for a_, b_ in zip(g, gb):
            assert torch.allclose(a_[b], b_[0], atol=2e-6), float((a_[b] - b_[0]).abs().max())


def test_clip_is_one_global_norm_per_sequence_and_update_is_f32():
    eng, net, h, toks, mask, kv, pos, W = _setup()
    g, _ = IN.inner_grad(W, net, h, toks, mask, kv, pos, 2, 0, create_graph=False, pos_q=pos + 1, own="causal")
    norm = IN.seq_norm(g)
    clip = float(norm.min()) * 0.5
    Wn, n2 = IN.inner_apply(W, g, net, 1.0, clip)
    assert torch.allclose(norm, n2)
    delta = IN.seq_norm([a - b for a, b in zip(IN.flat(Wn), IN.flat(W))])
    assert torch.allclose(delta, torch.full_like(delta, clip), rtol=1e-4)       # every sequence is clipped to the same norm
    Wn2, _ = IN.inner_apply(W, g, net, 0.5, 0.0)                                  # clip <= 0 disables
    d2 = IN.seq_norm([a - b for a, b in zip(IN.flat(Wn2), IN.flat(W))])
    assert torch.allclose(d2, 0.5 * norm, rtol=1e-4) and all(t.dtype == torch.float32 for t in IN.flat(Wn2))


def test_directions_keep_the_gradient_norm():
    eng, net, h, toks, mask, kv, pos, W = _setup(2)
    g, _ = IN.inner_grad(W, net, h, toks, mask, kv, pos, 2, 0, create_graph=False, pos_q=pos + 1, own="causal")
    for rule in ("sign", "muon2"):
        u = IN.direction([x.float() for x in g], rule)
        assert torch.allclose(IN.seq_norm(u), IN.seq_norm(g), rtol=1e-3)


def test_inner_lr_ramp():
    assert abs(IN.inner_lr(0, 1.0, 100) - 0.1) < 1e-9 and abs(IN.inner_lr(50, 1.0, 100) - 0.55) < 1e-9
    assert IN.inner_lr(100, 1.0, 100) == 1.0 and IN.inner_lr(3, 0.7, 0) == 0.7


@pytest.mark.parametrize("clip", [0.5, 100.0, 0.0])
def test_fused_plain_step_node_matches_autograd(clip):
    """The one-node form of the default write (fused passes, hand-written meta-gradient) against the chain of torch ops."""
    from dttt_b200.ttt import inner
    torch.manual_seed(0)
    B, F = 3, 2
    W = [torch.randn(B, 8, 16, requires_grad=True) for _ in range(3 * F)]
    g = [(torch.randn(B, 8, 16) * s).requires_grad_() for s in (0.1, 0.2, 0.3, 0.05, 0.4, 0.1)]
    eta = torch.tensor([0.5, 0.7], requires_grad=True)
    norm = inner.seq_norm(g)
    s = torch.clamp(clip / norm, max=1.0) if clip > 0 else torch.ones_like(norm)
    new_r = [W[i] - (s * eta[i // 3]).view(B, 1, 1) * g[i] for i in range(6)]
    out = inner._PlainStep.apply(clip, eta, 6, *W, *g)
    ws, wn = [torch.randn_like(x) for x in new_r], torch.randn(B)
    L_r = sum((a * b).sum() for a, b in zip(new_r, ws)) + (norm * wn).sum()
    L_f = sum((a * b).sum() for a, b in zip(out[:6], ws)) + (out[6] * wn).sum()
    gr = torch.autograd.grad(L_r, [eta] + W + g)
    gf = torch.autograd.grad(L_f, [eta] + W + g)
    assert abs(L_r.item() - L_f.item()) < 1e-4
    for a, b in zip(gr, gf):
        assert torch.allclose(a, b, atol=1e-5, rtol=1e-4)


def test_inner_gradient_taken_through_the_compute_dtype_copies_is_the_same_gradient():
    """bf16 compute, f32 fast weights: differentiating the inner loss w.r.t. the bf16 copies (the default) and w.r.t. the f32
    weights gives the same write and the same meta-gradient (the cast's backward only changes the dtype)."""
    from util import loss_and_grads, tiny_train
    from dttt_b200.ttt import inner
    ids = torch.randint(0, 120, (2, 32), generator=torch.Generator().manual_seed(3))
    res = {}
    for flag in (True, False):
        inner.GRAD_VIA_CAST[0] = flag
        try:
            eng = make_engine(tc=tiny_train(compute_dtype="bfloat16"))
            res[flag] = loss_and_grads(eng, ids, loss_config(eng.tc))
        finally:
            inner.GRAD_VIA_CAST[0] = True
    assert abs(res[True][0] - res[False][0]) < 1e-6
    for k in res[True][1]:
        a, b = res[True][1][k], res[False][1][k]
        # bf16 rounding noise only: the shared copy sums its three uses' gradients in bf16 before the cast back
        assert (a - b).abs().max().item() <= 5e-2 * (b.abs().max().item() + 1e-8), k
        assert (a - b).norm().item() <= 2e-2 * (b.norm().item() + 1e-8), k
