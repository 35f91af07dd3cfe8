"""The write: one clipped gradient step on the per-sequence fast weight per chunk.

    g      = grad_W  mean_{i in targets} CE( suffix(h_inner; W)_i , target_i )     per sequence
    u      = direction(g)                     sgd | sign | muon2, rescaled to ||g||
    u     <- u * min(1, clip / ||u||)         ONE norm over all 3 F matrices of a sequence
    W_l   <- W_l - eta_l u_l - lambda_l (W_l - W0_l)                                 in f32

(reference ``src/ttt/inner_loop.py:1-26``; ``inner_objective`` ``:193-312``, ``clip_global`` ``:332-342``,
``direction`` ``:350-397``, ``inner_apply`` ``:435-481``, ``norm_scales`` ``:556-576``, ``write_chunk``
``:588-719``).  Everything here is batched over sequences: the fast weight is a list over fast layers
of ``(gate [B,H,I], up [B,H,I], down [B,I,H])`` f32 tensors, the sequences never mix, so the gradient
of the *sum* of the per-sequence objectives with respect to the batched weight is the stack of the
per-sequence gradients and one backward pass serves the whole batch.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, NamedTuple, Optional, Sequence, Tuple

import torch

from ..ops import ce as CE
from ..ops import functional as Fn
from ..ops.attention import own_mask_matrix

FastW = List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]

STAT_NAMES = ("loss", "grad_norm", "clipped", "feat", "distill", "mtp", "kvb")


def zero_stats(device) -> torch.Tensor:
    return torch.zeros(len(STAT_NAMES), dtype=torch.float32, device=device)


@dataclass(frozen=True)
class WriteConfig:
    """Write schemes beyond one whole-chunk step (reference inner_loop.py:53-122)."""
    subchunks: int = 1
    subchunk_scale: float = 1.0
    surprise_gamma: float = 0.0
    kvb_weight: float = 0.0
    kvb_value: str = "self"
    fast_frac: float = 0.0
    fast_lr_scale: float = 1.0
    fast_decay: float = 0.0
    steps: int = 1
    norm_alpha: float = 0.0
    norm_cap: float = 1.0

    @property
    def normalised(self) -> bool:
        return self.norm_alpha > 0

    @property
    def plain(self) -> bool:
        return self == WriteConfig()

    def problems(self, chunk: int) -> List[str]:
        """Every rule this combination of write options breaks (empty: fine).  One rule per line: the range of a single
        option first, then which schemes exclude one another."""
        sub, fast, many = self.subchunks > 1, self.fast_frac > 0, self.steps > 1
        table = [
            (self.subchunks < 1 or chunk % max(self.subchunks, 1) != 0, f"inner_subchunks = {self.subchunks} does not divide the chunk of {chunk} tokens"),
            (not 0.0 < self.subchunk_scale <= 1.0, f"inner_subchunk_scale = {self.subchunk_scale} is outside (0, 1]"),
            (self.surprise_gamma < 0, "inner_surprise_gamma is negative"),
            (self.kvb_weight < 0, "inner_kvb_weight is negative"),
            (self.kvb_value not in ("self", "clean"), f"inner_kvb_value = {self.kvb_value!r} is neither 'self' nor 'clean'"),
            (not 0.0 <= self.fast_frac < 1.0, f"inner_fast_frac = {self.fast_frac} is outside [0, 1)"),
            (not 0.0 <= self.fast_decay <= 1.0, f"inner_fast_decay = {self.fast_decay} is outside [0, 1]"),
            (self.fast_lr_scale < 0, "inner_fast_lr_scale is negative"),
            (self.steps < 1, "inner_write_steps is below 1"),
            (self.norm_alpha < 0, "inner_norm_alpha is negative"),
            (self.norm_cap < 1.0, "inner_norm_cap is below 1"),
            (fast and self.subchunks < 2, "inner_fast_frac splits the units by time scale and the fast ones are written per sub-chunk: set inner_subchunks >= 2"),
            (many and (sub or fast), "inner_write_steps > 1 repeats the whole-chunk step: not together with sub-chunks or fast units"),
            (self.normalised and (sub or fast or many), "the normalised step (inner_norm_alpha > 0) is one whole-chunk step: not together with "
                                                        "sub-chunks, fast units or repeated steps"),
        ]
        return [why for broken, why in table if broken]

    def check(self, chunk: int) -> None:
        found = self.problems(chunk)
        if found:
            raise ValueError("write options: " + "; ".join(found))


class InnerExtras(NamedTuple):
    """Side inputs of the optional terms, batched ``[B, C, ...]`` (reference inner_loop.py:125-137)."""
    soft_ids: Optional[torch.Tensor] = None
    soft_q: Optional[torch.Tensor] = None
    soft_mask: Optional[torch.Tensor] = None
    mtp_tgt: Optional[torch.Tensor] = None
    mtp_mask: Optional[torch.Tensor] = None


def inner_lr(step: int, lr: float, warmup_steps: int) -> float:
    """``0.1 lr -> lr`` linearly over ``warmup_steps`` outer steps, then flat (inner_loop.py:140-152)."""
    if warmup_steps <= 0 or step >= warmup_steps:
        return float(lr)
    return 0.1 * lr + (lr - 0.1 * lr) * (step / warmup_steps)


def cast_fast(W: FastW, dtype: torch.dtype) -> FastW:
    """The compute-dtype copies of the fast weights.  f32 -> bf16 copies whose gradient will be wanted go through
    ``ops.gemm.cast_acc``: the products that use them then sum their gradient contributions in one f32 buffer."""
    from ..ops import gemm

    def one(t):
        if t.dtype == dtype:
            return t
        lo = getattr(t, "lo_copy", None)               # written by the step kernel that produced t (one use only)
        if lo is not None:
            t.lo_copy = None
            lo = lo if dtype == torch.bfloat16 and lo.shape == t.shape else None
        if (gemm.CAST_ACC and dtype == torch.bfloat16 and t.dtype == torch.float32 and t.dim() == 3 and t.requires_grad
                and torch.is_grad_enabled() and (t.is_cuda or gemm.EMULATE) and not gemm._FORCE_TORCH):
            return gemm.cast_acc(t, lo)
        return t.to(dtype) if lo is None or (t.requires_grad and torch.is_grad_enabled()) else lo
    return [tuple(one(t) for t in w) for w in W]


def flat(W: FastW) -> List[torch.Tensor]:
    return [t for w in W for t in w]


def unflat(ts: Sequence[torch.Tensor]) -> FastW:
    return [tuple(ts[i:i + 3]) for i in range(0, len(ts), 3)]


def seq_norm(ts: Sequence[torch.Tensor]) -> torch.Tensor:
    """Per-sequence global norm ``[B]`` over a list of ``[B, ...]`` tensors: ``sqrt(sum sq + 1e-8)``."""
    from ..ops import kernels
    if ts[0].is_cuda and not torch.is_grad_enabled() and kernels.available("seq"):
        return torch.sqrt(kernels.seq_sumsq(list(ts)) + 1e-8)
    sq = sum(torch.linalg.vector_norm(t.flatten(1), dim=1, dtype=torch.float32).pow(2) for t in ts)
    return torch.sqrt(sq + 1e-8)


_FRAC_MASKS = {}


def _update_frac_mask(i: int, shape, frac: float, device) -> torch.Tensor:
    """The bool mask of leaf ``i`` kept by ``inner_update_frac``: ``uniform(key(7919 + i), shape) < frac`` on the threefry
    generator, cached (it does not depend on the step or the data)."""
    k = (i, shape, frac, str(device))
    m = _FRAC_MASKS.get(k)
    if m is None:
        from ..utils import rng as _rng
        m = _FRAC_MASKS[k] = _rng.bernoulli(_rng.key(7919 + i), frac, shape).to(device)
    return m


def _bcast(v: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
    return v.reshape(v.shape + (1,) * (t.dim() - v.dim()))


# ---------------------------------------------------------------------------- objective
def inner_objective(W: FastW, model, h_inner: torch.Tensor, tokens: torch.Tensor, inner_mask: torch.Tensor, kv, pos,
                    n_valid: int, fused_block: int, *, tok_w=None, pos_q=None, own: str = "full", feat_tgt=None,
                    feat_mode: str = "off", feat_weight: float = 1.0, extras: Optional[InnerExtras] = None,
                    distill_weight: float = 1.0, mtp_weight: float = 1.0, soft_only: bool = False,
                    surprise_gamma: float = 0.0, kvb_weight: float = 0.0, kvb_src=None, score_from: int = 0,
                    own_mask=None, W_cast: Optional[FastW] = None):
    """Sum over sequences of the per-sequence inner objective, and its terms ``[5]`` (batch-summed
    ``ce, feat, distill, mtp, kvb``).  ``h_inner [B, C, H]`` (or ``[B, V, C, H]`` for V views, averaged),
    ``tokens / inner_mask [B, C]`` (``[B, V, C]``).  Each term is a weighted mean over its own slots of
    one sequence; see the reference docstring (inner_loop.py:201-230) for the terms."""
    net = model
    Wc = W_cast if W_cast is not None else cast_fast(W, net.dtype)       # ``W_cast``: the compute-dtype copies, made by the caller
    lm_w = net.lm_weight()
    has_temp = net.cw.has("inner_temp_log")

    def one(h_in, m):
        res = net.suffix_forward(h_in, pos, kv, Wc, n_valid, inner=True, pos_q=pos_q, own=own, own_mask=own_mask,
                                 return_prime=kvb_weight > 0)
        h = res[0]
        x_l = res[2][0] if kvb_weight > 0 else None                      # [F][B, C, H]
        toks, tw, ks, mm_ = tokens, tok_w, kvb_src, m
        if score_from:
            h, mm_, toks = h[:, score_from:], mm_[:, score_from:], toks[:, score_from:]
            tw = None if tw is None else tw[:, score_from:]
            if x_l is not None:
                x_l = [x[:, score_from:] for x in x_l]
                ks = None if ks is None else [k[:, score_from:] for k in ks]
        w = mm_.float() if tw is None else mm_.float() * tw
        B, Cs = w.shape
        hf = h.reshape(B * Cs, -1)
        if surprise_gamma > 0:
            ce_i = CE.per_token_ce(hf.detach(), lm_w.detach(), toks.reshape(-1), fused_block).view(B, Cs)
            w0 = w.sum(1, keepdim=True) + 1e-6
            rel = ce_i / ((w * ce_i).sum(1, keepdim=True) / w0 + 1e-6)
            w = w * torch.clamp(rel, min=1e-6).pow(surprise_gamma)
            w = w * (w0 / (w.sum(1, keepdim=True) + 1e-6))
        wsum = w.sum(1, keepdim=True) + 1e-6
        wn = w / wsum                                                     # per-sequence mean weights
        zero = torch.zeros((), dtype=torch.float32, device=h.device)
        feat = zero
        if feat_mode != "off":
            pred = Fn.linear(h, net.p("inner_feat_head.weight")).float()
            feat = (wn * (pred - feat_tgt.float()).pow(2).mean(-1)).sum()
        h_mtp = Fn.linear(h, net.p("mtp_head.weight")) if extras is not None and extras.mtp_tgt is not None else None
        if has_temp:
            tau = torch.exp(-net.p("inner_temp_log")).to(h.dtype)
            hf = hf * tau
            h_mtp = None if h_mtp is None else h_mtp * tau
        ce = CE.weighted_ce(hf, lm_w, toks.reshape(-1), wn.reshape(-1), fused_block)
        obj = ce if feat_mode == "off" else (feat if feat_mode == "only" else ce + feat_weight * feat)
        distill = mtp = kvb = zero
        soft = zero
        if extras is not None and extras.soft_ids is not None:
            wd = extras.soft_mask.float() if tok_w is None else extras.soft_mask.float() * tok_w
            wdn = wd / (wd.sum(1, keepdim=True) + 1e-6)
            soft = CE.soft_weighted_ce(hf, lm_w, extras.soft_ids.flatten(0, 1), extras.soft_q.flatten(0, 1),
                                       wdn.reshape(-1), fused_block)
            obj = obj + distill_weight * soft
            q = extras.soft_q.float()
            ent = -(q * torch.log(torch.clamp(q, min=1e-30))).sum(-1)
            distill = soft - (wdn * ent).sum()
        if h_mtp is not None:
            wm = extras.mtp_mask.float() if tok_w is None else extras.mtp_mask.float() * tok_w
            wmn = wm / (wm.sum(1, keepdim=True) + 1e-6)
            mtp = CE.weighted_ce(h_mtp.reshape(B * Cs, -1), lm_w, extras.mtp_tgt.reshape(-1), wmn.reshape(-1), fused_block)
            obj = obj + mtp_weight * mtp
        if kvb_weight > 0:
            errs = []
            for f, x in enumerate(x_l):
                src = x if ks is None else ks[f].detach()
                val = Fn.linear(src.to(x.dtype), net.p("inner_kvb_value.weight", f))
                errs.append(_bind_err(net, f, Wc[f], x, val))
            err = torch.stack(errs).mean(0)                               # [B, Cs]
            kvb = (wn * err).sum()
            obj = obj + kvb_weight * kvb
        if soft_only:
            obj = distill_weight * soft
        return obj, torch.stack([ce.detach().float(), feat.detach().float(), distill.detach().float(),
                                 mtp.detach().float(), kvb.detach().float()])

    if h_inner.dim() == 3:
        return one(h_inner, inner_mask)
    V = h_inner.shape[1]
    parts = [one(h_inner[:, v], inner_mask[:, v]) for v in range(V)]
    return sum(p[0] for p in parts) / V, sum(p[1] for p in parts) / V


class _BindErr(torch.autograd.Function):
    """Key-value-binding error of one layer with a layer-local inner gradient: only ``W_l`` receives a
    first-order gradient; key ``x`` and value ``v`` are inputs of the inner problem (zero cotangent), while
    the *recorded* backward still depends on them, so the meta-gradient reaches them through the write
    (reference inner_loop.py:163-190)."""

    @staticmethod
    def forward(ctx, fn, x, v, *W):
        ctx.fn = fn
        ctx.save_for_backward(x, v, *W)
        with torch.no_grad():
            return fn(W, x, v)

    @staticmethod
    def backward(ctx, g):
        x, v, *W = ctx.saved_tensors
        with torch.enable_grad():
            Wl = [w if w.requires_grad else w.detach().requires_grad_(True) for w in W]
            e = ctx.fn(Wl, x, v)
            gw = torch.autograd.grad(e, Wl, g, create_graph=torch.is_grad_enabled())
        return (None, None, None, *gw)


def _bind_err(net, f: int, Wl, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    def fn(W, xx, vv):
        y = net.norm("prime_post_norm.weight", f, net.fast_mlp(tuple(W), xx))
        return (y.float() - vv.float()).pow(2).mean(-1)
    if torch.is_grad_enabled() and any(w.requires_grad for w in Wl):
        return _BindErr.apply(fn, x, v, *Wl)
    return fn(Wl, x, v)


def token_weights(net, h_clean: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """``[B, C]`` per-token weights ``2 sigmoid(u . h_clean)`` (None without a token gate)."""
    if not net.cw.has("inner_token_gate.weight") or h_clean is None:
        return None
    z = h_clean.float() @ net.p("inner_token_gate.weight").float() + net.p("inner_token_gate.bias").float()
    return 2.0 * torch.sigmoid(z[..., 0])


# ---------------------------------------------------------------------------- the step
_NS = (3.4445, -4.7750, 2.0315)


def orthogonalise(g: torch.Tensor, iters: int = 2) -> torch.Tensor:
    """Newton-Schulz iterations toward the orthogonal factor of ``g [..., m, n]`` as a linear map of ``g``
    whose matrix is held constant for the meta-gradient (reference inner_loop.py:359-382)."""
    a, b, c = _NS
    tr = g.shape[-2] > g.shape[-1]
    x = g.transpose(-1, -2) if tr else g
    with torch.no_grad():
        xn = x / (torch.linalg.matrix_norm(x.float(), dim=(-2, -1), keepdim=True) + 1e-7)
        m = xn.shape[-2]
        eye = torch.eye(m, dtype=torch.float32, device=g.device)
        P = eye.expand(*xn.shape[:-2], m, m)
        xk = xn.float()
        for _ in range(iters):
            xb = xk.to(torch.bfloat16)
            Amat = (xb @ xb.transpose(-1, -2)).float() if xb.is_cuda else (xb.float() @ xb.float().transpose(-1, -2))
            Ab = Amat.to(torch.bfloat16)
            A2 = (Ab @ Ab).float() if Ab.is_cuda else (Ab.float() @ Ab.float())
            Pk = a * eye + b * Amat + c * A2
            xk = (Pk.to(torch.bfloat16).float() @ xb.float())
            P = Pk.to(torch.bfloat16).float() @ P.to(torch.bfloat16).float()
    y = P.to(torch.bfloat16).float() @ x.to(torch.bfloat16).float()
    return y.transpose(-1, -2) if tr else y


def direction(g: List[torch.Tensor], rule: str) -> List[torch.Tensor]:
    if rule == "sgd":
        return g
    if rule == "sign":
        u = [x * torch.rsqrt(x.pow(2) + 1e-12) for x in g]
    elif rule == "muon2":
        u = [orthogonalise(x, 2) for x in g]
    else:
        raise ValueError(f"inner_update {rule!r}")
    ratio = seq_norm(g) / seq_norm(u)
    return [x * _bcast(ratio, x) for x in u]


def mask_units(ts: List[torch.Tensor], unit_mask: torch.Tensor) -> List[torch.Tensor]:
    """Zero everything outside the hidden units ``unit_mask [I]`` (gate/up columns, down rows)."""
    m = unit_mask.float()
    out = []
    for i in range(0, len(ts), 3):
        g, u, d = ts[i:i + 3]
        out += [g * m.to(g.dtype), u * m.to(u.dtype), d * m[:, None].to(d.dtype)]
    return out


def unit_scale(ts: List[torch.Tensor], scale) -> List[torch.Tensor]:
    """Normalised step: ``scale = (f_units [B,F,I], f_dims [B,F,H])``; down rows x f_units, gate/up x min(f_dims, f_units)."""
    fu, fd = scale
    out = []
    for f in range(len(ts) // 3):
        g, u, d = ts[3 * f:3 * f + 3]
        f_gu = torch.minimum(fd[:, f, :, None], fu[:, f, None, :])
        out += [g * f_gu, u * f_gu, d * fu[:, f, :, None]]
    return out


def inner_grad(W: FastW, model, h_inner, tokens, inner_mask, kv, pos, n_valid, fused_block, *, create_graph: bool,
               h_clean=None, distill_meta: bool = True, **kw):
    """Per-sequence gradients of the inner objective w.r.t. ``W`` (a flat list like ``flat(W)``) and the terms."""
    tok_w = token_weights(model, h_clean)
    extras = kw.get("extras")
    soft_first_order = extras is not None and extras.soft_ids is not None and not distill_meta
    Wl = flat(W)
    kw = dict(kw)
    W_cast = kw.pop("W_cast", None)
    # The objective sees W only through its compute-dtype copy, so the gradient is taken w.r.t. that copy (same values as
    # the gradient w.r.t. W, without the cast's backward and, under the meta-gradient, that backward's derivative).
    via_cast = (GRAD_VIA_CAST[0] and Wl[0].dtype != model.dtype and not soft_first_order and not kw.get("kvb_weight", 0.0))
    if not create_graph:
        # a first-order write: nothing outside this call may see the graph built here
        h_inner = h_inner.detach()
        kv = [(a.detach(), b.detach()) for a, b in kv]
        h_clean = None if h_clean is None else h_clean.detach()
        tok_w = None if tok_w is None else tok_w.detach()
    with torch.enable_grad():
        if not create_graph:
            Wl = [w.detach().requires_grad_(True) for w in Wl]
        elif not all(w.requires_grad for w in Wl):
            Wl = [w if w.requires_grad else w.detach().requires_grad_(True) for w in Wl]
        kw2 = dict(kw)
        if soft_first_order:
            kw2["distill_weight"] = 0.0
        wrt = Wl
        if via_cast:
            if not create_graph:
                src = flat(W_cast) if W_cast is not None else flat(cast_fast(unflat(Wl), model.dtype))
                wrt = [c.detach().requires_grad_(True) for c in src]
            else:
                wrt = flat(W_cast) if W_cast is not None and all(c.requires_grad for c in flat(W_cast)) \
                    else flat(cast_fast(unflat(Wl), model.dtype))
            kw2["W_cast"] = unflat(wrt)
        obj, terms = inner_objective(unflat(Wl), model, h_inner, tokens, inner_mask, kv, pos, n_valid, fused_block,
                                     tok_w=tok_w, **kw2)
        with Fn.inner_backward():
            g = torch.autograd.grad(obj, wrt, create_graph=create_graph)
        if soft_first_order:
            Wd = [w.detach().requires_grad_(True) for w in Wl]
            obj2, terms2 = inner_objective(unflat(Wd), model, h_inner, tokens, inner_mask, kv, pos, n_valid, fused_block,
                                           tok_w=tok_w, **dict(kw, soft_only=True))
            with Fn.inner_backward():
                g2 = torch.autograd.grad(obj2, Wd)
            g = [a + b.detach() for a, b in zip(g, g2)]
            terms = terms.clone()
            terms[2] = terms2[2]
    if not create_graph:
        g = [x.detach() for x in g]
    return list(g), terms


# The inner gradient is taken w.r.t. the compute-dtype copies of the fast weights (False: w.r.t. the f32 weights themselves).
GRAD_VIA_CAST = [True]

# The plain step as one autograd node with fused kernels (False: the chain of differentiable torch ops; "force": also
# for CPU tensors, where the node's pieces are torch statements -- used by the tests).
FUSED_PLAIN_STEP = [True]
# The fused step also writes the bf16 copy of the new weights (False: the next chunk casts them in a pass of its own).
LO_COPY = [os.environ.get("DTTT_LO_COPY", "1") == "1"]


def _seq_ops(t: torch.Tensor):
    """(sumsq, axpy, dot, lincomb) per sequence: the CUDA kernels, or torch statements of the same on the CPU."""
    from ..ops import kernels
    if t.is_cuda and kernels.available("seq"):
        return kernels.seq_sumsq, kernels.seq_axpy, kernels.seq_dot, kernels.seq_lincomb
    B = t.shape[0]
    sumsq = lambda ts: sum(x.float().flatten(1).pow(2).sum(1) for x in ts)
    axpy = lambda w, g, c: w - c.view(B, *([1] * (w.dim() - 1))) * g.float()
    dot = lambda a_, g_: sum((x.float() * y.float()).flatten(1).sum(1) for x, y in zip(a_, g_))
    lincomb = lambda a, g, al, be: (al.view(B, *([1] * (a.dim() - 1))) * a + be.view(B, *([1] * (a.dim() - 1))) * g.float()).to(g.dtype)
    return sumsq, axpy, dot, lincomb


class _PlainStep(torch.autograd.Function):
    """``W'_i = W_i - eta_f s_b g_i`` with ``s_b = min(1, clip / ||g||_b)`` over every matrix of a sequence (reference
    inner_loop.py:435-481, the default rule), forward and first-order backward each a handful of fused passes:

        dW_i  = dW'_i
        dg_i  = -eta_f s_b dW'_i + [clipped_b] (clip / ||g||_b^3) (sum_j eta_fj <dW'_j, g_j>_b) g_i + (dnorm_b / ||g||_b) g_i
        deta_f = -sum_b s_b sum_{i in f} <dW'_i, g_i>_b

    The backward is the meta-gradient's path through the write (reference chunk_scan.py:604-625); nothing
    differentiates it again."""

    @staticmethod
    def forward(ctx, clip, eta, n, *Wg):
        from ..ops import kernels
        ctx.set_materialize_grads(False)               # the bf16 copies below never receive a gradient: no zeros for them
        W, g = Wg[:n], Wg[n:]
        sumsq, axpy, _, _ = _seq_ops(W[0])
        norm = torch.sqrt(sumsq(list(g)) + 1e-8)
        s = torch.clamp(clip / norm, max=1.0) if clip > 0 else torch.ones_like(norm)
        los = []
        if axpy is kernels.seq_axpy and LO_COPY[0] and all(w.dtype == torch.float32 for w in W):
            # the kernel writes the bf16 copy of W' in the same pass: the next chunk's cast has nothing left to do
            pairs = [axpy(W[i], g[i], s * eta[i // 3], want_lo=True) for i in range(n)]
            new, los = [p_[0] for p_ in pairs], [p_[1] for p_ in pairs]
            ctx.mark_non_differentiable(*los)
        else:
            new = [axpy(W[i], g[i], s * eta[i // 3]) for i in range(n)]
        ctx.save_for_backward(eta, norm, s, *g)
        ctx.clip, ctx.n = clip, n
        return (*new, norm, *los)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *grads):
        n, clip = ctx.n, ctx.clip
        eta, norm, s, *g = ctx.saved_tensors
        dnew, dnorm = list(grads[:n]), grads[n]
        _, _, dot, lincomb = _seq_ops(g[0])
        dnew = [torch.zeros_like(gi, dtype=torch.float32) if d is None else d.float() for d, gi in zip(dnew, g)]
        F_ = n // 3
        dots = [dot(dnew[3 * f:3 * f + 3], g[3 * f:3 * f + 3]) for f in range(F_)]          # [F] x [B]
        wdot = sum(eta[f] * dots[f] for f in range(F_))
        beta = torch.zeros_like(norm)
        if clip > 0:
            beta = torch.where(norm > clip, wdot * clip / norm.pow(3), beta)
        if dnorm is not None:
            beta = beta + dnorm / norm
        dg = [lincomb(dnew[i], g[i], -eta[i // 3] * s, beta) for i in range(n)] if any(ctx.needs_input_grad[3 + n:]) else [None] * n
        deta = torch.stack([-(s * dots[f]).sum() for f in range(F_)]) if ctx.needs_input_grad[1] else None
        return (None, deta, None, *dnew, *dg)


def inner_apply(W: FastW, g: List[torch.Tensor], model, lr: float, clip: float, rule: str = "sgd", *, inner_mask=None,
                h_clean=None, loss=None, frac: float = 1.0, unit_mask=None, scale=None, W0: Optional[FastW] = None):
    """The step of gradient ``g``: ``(W', pre-clip norm [B])`` (reference inner_loop.py:435-481)."""
    net = model
    Wl = flat(W)
    plain = (rule == "sgd" and unit_mask is None and frac >= 1.0 and scale is None
             and not net.cw.has("inner_precond.0.gate.weight") and not net.cw.has("inner_gate.weight")
             and not net.cw.has("inner_decay_logit"))
    if plain:
        # the main line: one norm, one fused multiply-add per matrix
        eta = torch.full((len(W),), float(lr), dtype=torch.float32, device=Wl[0].device)
        if net.cw.has("inner_step_log"):
            eta = eta * torch.exp(net.p("inner_step_log").float())
        if FUSED_PLAIN_STEP[0] and (Wl[0].is_cuda or FUSED_PLAIN_STEP[0] == "force"):
            out = _PlainStep.apply(float(clip), eta, len(Wl), *Wl, *g)           # the kernels read bf16 or f32 gradients
            n = len(Wl)
            for t, lo in zip(out[:n], out[n + 1:]):
                t.lo_copy = lo
            return unflat(list(out[:n])), out[n]
        g = [x.float() for x in g]
        norm = seq_norm(g)
        s = torch.clamp(clip / norm, max=1.0) if clip > 0 else torch.ones_like(norm)
        B = Wl[0].shape[0]
        coef = s[:, None] * eta[None, :]                                    # [B, F]
        new = []
        for f in range(len(W)):
            for j in range(3):
                p, d = Wl[3 * f + j], g[3 * f + j]
                new.append(torch.addcmul(p, coef[:, f].view(B, 1, 1), d, value=-1.0))
        return unflat(new), norm
    g = [x.float() for x in g]
    if unit_mask is not None:
        g = mask_units(g, unit_mask)
    u = direction(g, rule)
    F_ = len(W)
    if net.cw.has("inner_precond.0.gate.weight"):
        names = ("gate", "up", "down")
        out = []
        for f in range(F_):
            for j, nm in enumerate(names):
                a = net.p(f"inner_precond.0.{nm}.weight", f).float()
                b = net.p(f"inner_precond.1.{nm}.weight", f).float()
                out.append(u[3 * f + j] * torch.exp(a)[None, :, None] * torch.exp(b)[None, None, :])
        u = out
    if frac < 1.0:
        # fixed write dimensions, one draw per leaf from the counter generator (reference inner_loop.py: bernoulli(PRNGKey(7919 + i)))
        masks = [_update_frac_mask(i, tuple(x.shape[1:]), float(frac), x.device).to(x.dtype) for i, x in enumerate(u)]
        um = [x * m for x, m in zip(u, masks)]
        ratio = seq_norm(u) / seq_norm(um)
        u = [x * _bcast(ratio, x) for x in um]
    norm = seq_norm(u)
    if clip > 0:
        s = torch.clamp(clip / norm, max=1.0)
        u = [x * _bcast(s, x) for x in u]
    if scale is not None:
        u = unit_scale(u, scale)
    B = Wl[0].shape[0]
    eta = torch.full((B, F_), float(lr), dtype=torch.float32, device=Wl[0].device)
    if net.cw.has("inner_step_log"):
        eta = eta * torch.exp(net.p("inner_step_log").float())[None, :]
    if net.cw.has("inner_gate.weight"):
        m = inner_mask.reshape(B, -1, inner_mask.shape[-1])[:, 0]
        ratio = (m > 0).float().mean(-1)
        feats = torch.cat([h_clean.float().mean(1), torch.stack([loss.detach() / 8.0, ratio], dim=-1)], dim=-1)   # [B, H+2]
        gw, gb = net.p("inner_gate.weight").float(), net.p("inner_gate.bias").float()               # [F, H+2, 1], [F, 1]
        gate = torch.einsum("bh,fh->bf", feats, gw[..., 0]) + gb[:, 0][None]
        eta = float(lr) * 2.0 * torch.sigmoid(gate)
    new = []
    lam = 0.1 * torch.sigmoid(net.p("inner_decay_logit").float()) if net.cw.has("inner_decay_logit") else None
    for f in range(F_):
        for j in range(3):
            p, d = Wl[3 * f + j], u[3 * f + j]
            nw = p - eta[:, f, None, None] * d
            if lam is not None:
                p0 = net.p(("fast_weight.gate.weight", "fast_weight.up.weight", "fast_weight.down.weight")[j], f).float()
                nw = nw - lam[f] * (p - p0[None])
            new.append(nw.float())
    return unflat(new), norm


def inner_update(W: FastW, model, h_inner, tokens, inner_mask, kv, pos, n_valid, lr: float, clip: float, fused_block: int,
                 rule: str = "sgd", *, create_graph: bool, h_clean=None, frac: float = 1.0, unit_mask=None, scale=None,
                 **kw):
    """Batched inner step: ``(W', stats [7])`` with stats batch-summed in the order ``STAT_NAMES``."""
    g, terms = inner_grad(W, model, h_inner, tokens, inner_mask, kv, pos, n_valid, fused_block,
                          create_graph=create_graph, h_clean=h_clean, **kw)
    loss_seq = None
    if model.cw.has("inner_gate.weight"):
        B = tokens.shape[0]
        loss_seq = terms[0].expand(B) / B              # the gate's surprise feature: the batch mean stands in per sequence
    Wn, norm = inner_apply(W, g, model, lr, clip, rule, inner_mask=inner_mask, h_clean=h_clean, loss=loss_seq,
                           frac=frac, unit_mask=unit_mask, scale=scale)
    clipped = (norm > clip).float().sum() if clip > 0 else torch.zeros((), device=norm.device)
    stats = torch.stack([terms[0], norm.detach().sum(), clipped.detach(), terms[1], terms[2], terms[3], terms[4]])
    return Wn, stats


def norm_scales(model, W: FastW, h_inner, kv, pos, n_valid, pos_q, own, inner_mask, alpha: float, cap: float):
    """``(f_units [B,F,I], f_dims [B,F,H])`` of the normalised step, constants for the meta-gradient
    (reference inner_loop.py:556-576): per fast layer the RMS over the written slots of the hidden units'
    activations and of the inputs, ``f = min(cap, (max r / r)^alpha)``."""
    net = model
    with torch.no_grad():
        Wc = cast_fast([tuple(t.detach() for t in w) for w in W], net.dtype)
        _, _, (xs, _) = net.suffix_forward(h_inner, pos, kv, Wc, n_valid, pos_q=pos_q, own=own, return_prime=True)
        mw = inner_mask.float() / (inner_mask.float().sum(1, keepdim=True) + 1e-6)           # [B, C]
        fu, fd = [], []
        for f, x in enumerate(xs):
            _, a = net.fast_mlp(Wc[f], x, return_hidden=True)
            ru = torch.sqrt(torch.einsum("bc,bci->bi", mw, a.float().pow(2)))
            rd = torch.sqrt(torch.einsum("bc,bch->bh", mw, x.float().pow(2)))
            fn = lambda r: torch.clamp((r.max(-1, keepdim=True).values / (r + 1e-12)).pow(alpha), max=cap)
            fu.append(fn(ru))
            fd.append(fn(rd))
        return torch.stack(fu, 1), torch.stack(fd, 1)


def fast_unit_mask(inter: int, frac: float, device=None) -> torch.Tensor:
    return torch.arange(inter, device=device) < int(round(frac * inter))


def write_chunk(W: FastW, model, h_inner, tokens, inner_mask, kv, pos, n_valid: int, lr: float, clip: float,
                fused_block: int, rule: str, h_clean, pos_q, own: str, wc: WriteConfig, *, create_graph: bool,
                W0: Optional[FastW] = None, kvb_src=None, W_cast: Optional[FastW] = None):
    """The causal write of one chunk under ``wc`` (reference inner_loop.py:588-719); a plain ``wc`` is one
    ``inner_update``.  Shared by training and decoding.  ``W_cast``: the caller's compute-dtype copies of ``W``
    (differentiable functions of it), reused by the plain write instead of casting again."""
    net = model
    base = dict(rule=rule, h_clean=h_clean, own=own, create_graph=create_graph)
    if wc.plain:
        return inner_update(W, net, h_inner, tokens, inner_mask, kv, pos, n_valid, lr, clip, fused_block,
                            pos_q=pos_q, W_cast=W_cast, **base)
    if net.cw.has("inner_gate.weight") or net.cw.has("inner_decay_logit"):
        raise ValueError("the write schemes are defined for the plain step: no write gate / learned decay")
    ks_all = kvb_src if wc.kvb_weight > 0 else None
    if wc.normalised:
        scale = norm_scales(net, W, h_inner, kv, pos, n_valid, pos_q, own, inner_mask, wc.norm_alpha, wc.norm_cap)
        return inner_update(W, net, h_inner, tokens, inner_mask, kv, pos, n_valid, lr, clip, fused_block, pos_q=pos_q,
                            kvb_weight=wc.kvb_weight, kvb_src=ks_all, surprise_gamma=wc.surprise_gamma, scale=scale, **base)
    B, C = tokens.shape
    n = wc.subchunks
    wkw = dict(surprise_gamma=wc.surprise_gamma, kvb_weight=wc.kvb_weight)
    own_full = own_mask_matrix(C, own, tokens.device)

    def full_step(w):
        return inner_update(w, net, h_inner, tokens, inner_mask, kv, pos, n_valid, lr, clip, fused_block, pos_q=pos_q,
                            kvb_src=ks_all, **base, **wkw)

    def sub_args(k):
        s, e = k * C // n, (k + 1) * C // n
        sel = (torch.arange(e, device=tokens.device) >= s).float()
        m_k = inner_mask[:, :e].float() * sel[None]
        ks = None if ks_all is None else [x[:, :e] for x in ks_all]
        om = None if own_full is None else own_full[:e, :e]
        return s, e, m_k, ks, om

    if wc.fast_frac > 0:
        fast = fast_unit_mask(W[0][0].shape[-1], wc.fast_frac, tokens.device)
        mf = inner_mask.float()
        wtot = mf.sum(1) + 1e-6
        acc, sts, w = None, [], W
        for k in range(n):
            s, e, m_k, ks, om = sub_args(k)
            g, terms = inner_grad(w, net, h_inner[:, :e], tokens[:, :e], m_k, kv, pos[:, :e], n_valid, fused_block,
                                  create_graph=create_graph, h_clean=h_clean, pos_q=None if pos_q is None else pos_q[:, :e],
                                  own="full" if om is None else own, own_mask=om, kvb_src=ks, score_from=s, **wkw)
            w, norm = inner_apply(w, g, net, lr * wc.fast_lr_scale, clip * wc.subchunk_scale, rule, unit_mask=fast)
            share = m_k.sum(1) / wtot
            g_slow = [x * _bcast(share, x) for x in mask_units([x.float() for x in g], ~fast)]
            acc = g_slow if acc is None else [a + b for a, b in zip(acc, g_slow)]
            sts.append((terms, norm, (norm > clip * wc.subchunk_scale).float()))
        loss = sum(t[0] for t, _, _ in sts) / n
        w, norm_s = inner_apply(w, acc, net, lr, clip, rule, unit_mask=~fast)
        norm_f = sum(x for _, x, _ in sts) / n
        clip_f = sum(x for _, _, x in sts) / n
        zero = torch.zeros((), device=tokens.device)
        stats = torch.stack([loss, ((norm_f + norm_s) / 2).detach().sum(),
                             ((clip_f + (norm_s > clip).float()) / 2).detach().sum(), zero, zero, zero,
                             sum(t[4] for t, _, _ in sts) / n])
        if wc.fast_decay > 0:
            if W0 is None:
                raise ValueError("inner_fast_decay needs W0")
            keep = fast.float()
            new = []
            for f in range(len(w)):
                trip = []
                for j in range(3):
                    cur, w0 = w[f][j], W0[f][j].float()
                    relaxed = w0 + (1.0 - wc.fast_decay) * (cur - w0)
                    km = keep[None, None, :] if j < 2 else keep[None, :, None]
                    trip.append(cur * (1 - km) + relaxed * km)
                new.append(tuple(trip))
            w = new
        return w, stats
    if n == 1 and wc.steps > 1:
        w, sts = W, []
        for _ in range(wc.steps):
            w, st = full_step(w)
            sts.append(st)
        return w, torch.stack(sts).mean(0)
    if n == 1:
        return full_step(W)
    w, sts = W, []
    for k in range(n):
        s, e, m_k, ks, om = sub_args(k)
        w, st = inner_update(w, net, h_inner[:, :e], tokens[:, :e], m_k, kv, pos[:, :e], n_valid, lr,
                             clip * wc.subchunk_scale, fused_block, rule=rule, h_clean=h_clean,
                             pos_q=None if pos_q is None else pos_q[:, :e], own="full" if om is None else own, own_mask=om,
                             kvb_src=ks, score_from=s, create_graph=create_graph, **wkw)
        sts.append(st)
    return w, torch.stack(sts).mean(0)


def drift_stats(W_final: FastW, W0: FastW) -> dict:
    """``||W - W0|| / ||W0||`` over all leaves and sequences (reference inner_loop.py:722-732)."""
    # one reduction pass per leaf; a W0 leaf that is one template broadcast over the batch is reduced once and scaled
    def sq(t):
        if t.dim() == 3 and t.stride(0) == 0 and t.shape[0] > 1:
            return torch.linalg.vector_norm(t[0].float()).pow(2) * t.shape[0]
        return torch.linalg.vector_norm(t.float()).pow(2)
    d = torch.sqrt(sum(sq(a.float() - b.float()) for a, b in zip(flat(W_final), flat(W0))))
    i = torch.sqrt(sum(sq(b) for b in flat(W0)))
    return {"ttt_drift_rel": d / (i + 1e-12), "ttt_delta_norm": d, "ttt_init_norm": i}
