"""Jacobian lens and memory read-out for the chunked test-time-training model.

    lens_l(h) = unembed(J_l h),   unembed = lm_head . final_norm,   J_l = E[ d h_L / d h_l ]

with ``h_L`` the last layer's residual BEFORE the final norm (so ``J = I`` at the last layer and the lens there is the
model's own output).  The lens is fitted in the READ condition of the outer stream: a chunk after the window has filled,
the memory written from the previous chunks, a mask on the chunk, query positions ``pos + 1`` under the outer shift.
Injection points: ``("out", l)`` is the residual after layer ``l`` (prefix layers first, then suffix); ``("mem", s)`` is, in
suffix layer ``s``, the residual right after the memory's read is added and before that layer's base MLP.

The memory's own part in suffix layer ``s`` is ``m_s = p_s(W) - p_s(W_0)`` on the same input, with
``p_s = post_norm_s(W_s(pre_norm_s(h)))``.  Its effect on the logits is read three ways: the exact first-order effect in
context (``direct_effect``, a JVP of the network above the injection point), the lens (``decode_delta``) and the exact
non-linear total (``Reader.read`` with the memory on and off).  Options of the read used by the probes: ``transplant``
(the memory queried at the write's inputs of chosen source slots) and ``den_W`` (a fast branch normalised by the RMS of
another memory's output).  Role and definitions: reference ``tools/j_lens/core.py:1-486``.

Everything here runs the model's plain PyTorch statements (f32 tensors take the reference path of every op), so the
forward is differentiable to any order and in forward mode.  Only the fast-weight memory is supported, as in generation.
"""
from __future__ import annotations

import dataclasses as dc
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ... import generate as G
from ...models.blocks import Net
from ...ops import attention as A
from ...ops import functional as Fn
from ...ttt import inner as IN
from ...utils import rng

Point = Tuple[str, int]


@dc.dataclass
class Transplant:
    """At the slots ``dst [B, n]`` of the read chunk use the memory's contribution computed at the inputs ``x_src`` (per fast
    layer ``[B, n, H]``: the write's inputs of the source slots holding the same tokens)."""
    dst: torch.Tensor
    x_src: List[torch.Tensor]


class Reader:
    """A model opened for reading and writing chunk by chunk with a run's own write."""

    def __init__(self, engine, cfg, step: int, inner_lr: Optional[float] = None, inner_task: Optional[str] = None):
        self.eng, self.cfg = engine, cfg
        self.net: Net = engine.net(train=False)
        self.mc = self.net.cfg
        if self.mc.memory != "ttt":
            raise NotImplementedError("the probes read the fast-weight memory; the gdn arm has no decoding path here")
        self.C, self.Wn = self.mc.chunk_size, self.mc.window_chunks
        self.outer_shift = bool(cfg.outer_shift)
        self.task = inner_task or cfg.inner_task
        self.lr = IN.inner_lr(step, cfg.inner_lr, cfg.inner_lr_warmup_steps) if inner_lr is None else inner_lr
        self.wc = engine.lcfg.write
        self.dev = self.net.p("final_norm.weight").device

    # ---- state
    def fresh(self, B: int) -> G.DecodeState:
        return G.init_state(self.net, B)

    def positions(self, B: int, chunk: int) -> torch.Tensor:
        return (chunk * self.C + torch.arange(self.C, device=self.dev))[None].expand(B, self.C)

    def write(self, state: G.DecodeState, ids: torch.Tensor, key=None) -> G.DecodeState:
        """The chunk ``ids [B, C]`` becomes context: its K/V enter the windows and the fast weight takes the run's write."""
        cfg = self.cfg
        key = rng.fold_in(rng.key(cfg.seed), state.chunk) if key is None else key
        ratio = cfg.inner_mask_ratio if cfg.inner_mask_ratio > 0 else 0.5 * (cfg.inner_mask_range[0] + cfg.inner_mask_range[1])
        with torch.no_grad():
            return G.commit_block(self.net, ids.to(self.dev), self.positions(ids.shape[0], state.chunk), state, key.to(self.dev), self.lr,
                                  cfg.inner_clip, ratio, cfg.fused_ce_block, inner_task=self.task, wc=self.wc)

    def write_pass(self, ids: torch.Tensor, upto: int, keep: Sequence[int] = ()) -> Tuple[G.DecodeState, Dict[int, G.DecodeState]]:
        """Write chunks ``0 .. upto - 1`` of ``ids [B, T]``; ``keep``: chunk indices whose PRE-write state is returned too."""
        st = self.fresh(ids.shape[0])
        snaps = {}
        for c in range(upto):
            if c in keep:
                snaps[c] = st
            st = self.write(st, ids[:, c * self.C:(c + 1) * self.C])
        if upto in keep:
            snaps[upto] = st
        return st, snaps

    def with_memory(self, state: G.DecodeState, W) -> G.DecodeState:
        return G.DecodeState(state.kv, W, state.chunk)

    def reset_memory(self, state: G.DecodeState) -> G.DecodeState:
        B = state.kv[0][0].shape[0]
        return self.with_memory(state, [tuple(t.detach().clone() for t in w) for w in self.net.template_fast(B)])

    # ---- the read
    def forward(self, x: torch.Tensor, state: G.DecodeState, *, inject: Optional[Dict[Point, torch.Tensor]] = None,
                capture: Sequence[Point] = (), leaves: Optional[Dict[Point, torch.Tensor]] = None, own: str = "full",
                shift: Optional[bool] = None, transplant: Optional[Transplant] = None, den_W=None, start: Optional[Point] = None):
        """Token ids ``x [B, C]`` through every layer against ``state``.  Returns ``(h_L [B, C, H] before the final norm,
        captures)``; ``captures`` maps the requested points to residuals, ``("mem_part", s)`` to the memory's own part
        ``m_s`` and ``("mem_in", s)`` to the fast branch's input.  ``leaves[point]``: replace the residual at ``point`` by
        this tensor (a leaf to differentiate from); ``inject[point]`` is added there."""
        net, mc = self.net, self.mc
        B = x.shape[0]
        pos = self.positions(B, state.chunk)
        shift = self.outer_shift if shift is None else shift
        pos_q = pos + 1 if shift else None
        nv = A.valid_window_chunks(state.chunk, self.Wn, mc.reach)
        inject, leaves, cap = inject or {}, leaves or {}, {}
        Wc = IN.cast_fast(state.W, net.dtype)
        W0 = IN.cast_fast(net.template_fast(B), net.dtype)
        Wden = None if den_W is None else IN.cast_fast(den_W, net.dtype)

        def at(point, h):
            if point in leaves:
                h = leaves[point]
            if point in inject:
                h = h + inject[point].to(h.dtype)
            if point in capture:
                cap[point] = h
            return h
        h = net.embed_tokens(x.to(self.dev))
        Lp, f = mc.prefix_len, 0
        for l in range(mc.num_hidden_layers):
            stack, i = ("prefix", l) if l < Lp else ("suffix", l - Lp)
            q, k, v = net.qkv(stack, i, net.norm(f"{stack}.attn_norm.weight", i, h), pos, pos_q)
            a = A.attend_window(q, k, v, state.kv[l][0], state.kv[l][1], nv, self.C, net.scale, own=own)
            h = h + Fn.linear(a.flatten(-2), net.p(f"{stack}.attn.o.weight", i))
            if stack == "suffix" and mc.fast_mask[i]:
                xin = net.norm("prime_norm.weight", f, h)
                post = lambda y, ref=None: self._post_norm(f, y, ref)
                y = net.fast_mlp(Wc[f], xin)
                p = post(y, None if Wden is None else net.fast_mlp(Wden[f], xin))
                if transplant is not None:
                    xs = transplant.x_src[f].to(xin.dtype)
                    m_src = post(net.fast_mlp(Wc[f], xs)) - post(net.fast_mlp(W0[f], xs))
                    m_here = p - post(net.fast_mlp(W0[f], xin))
                    idx = transplant.dst.to(self.dev)[..., None].expand(-1, -1, h.shape[-1])
                    p = p + torch.zeros_like(p).scatter(1, idx, m_src - torch.gather(m_here, 1, idx))
                if ("mem_part", i) in capture or ("mem_in", i) in capture:
                    cap[("mem_part", i)] = p - post(net.fast_mlp(W0[f], xin))
                    cap[("mem_in", i)] = xin
                h = at(("mem", i), h + p)
                f += 1
            h = h + net.mlp(stack, i, net.norm(f"{stack}.mlp_norm.weight", i, h))
            h = at(("out", l), h)
        return h, cap

    def _post_norm(self, f: int, y: torch.Tensor, ref: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``prime_post_norm`` of ``y``; with ``ref`` the RMS in the denominator is that of ``ref`` (``den_W``)."""
        w = self.net.p("prime_post_norm.weight", f).float()
        src = (y if ref is None else ref).float()
        r = torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + self.mc.rms_norm_eps)
        return (w * y.float() * r).to(y.dtype)

    def unembed(self, h_L: torch.Tensor) -> torch.Tensor:
        return self.net.logits(self.net.norm("final_norm.weight", None, h_L)).float()

    def read(self, ids: torch.Tensor, masked: torch.Tensor, state: G.DecodeState, **kw) -> torch.Tensor:
        """Logits ``[B, C, V]`` of the outer read of chunk ``ids`` with the tokens at ``masked`` replaced by the mask id."""
        x = torch.where(masked.to(ids.device), torch.full_like(ids, self.mc.mask_token_id), ids)
        with torch.no_grad():
            h_L, _ = self.forward(x, state, **kw)
            return self.unembed(h_L)

    def slot_ce(self, logits: torch.Tensor, ids: torch.Tensor, masked: torch.Tensor, next_first: Optional[torch.Tensor] = None):
        """Per-slot CE of the scored tokens and the scored-slot mask ``[B, C]``.  Under the outer shift slot ``i`` predicts token
        ``i + 1`` (the last slot predicts ``next_first``, scored only when given)."""
        ids, masked = ids.to(logits.device), masked.to(logits.device)
        if self.outer_shift:
            nxt = ids[:, -1:] if next_first is None else next_first.to(ids.device).view(-1, 1)
            tgt = torch.cat([ids[:, 1:], nxt], 1)
            sc = torch.cat([masked[:, 1:], torch.zeros_like(masked[:, :1])], 1)
        else:
            tgt, sc = ids, masked
        ce = torch.nn.functional.cross_entropy(logits.flatten(0, 1), tgt.flatten().long(), reduction="none").view(ids.shape)
        return ce * sc, sc

    def valid_slots(self, masked: torch.Tensor) -> torch.Tensor:
        """The slots the training loss scores: those whose target is masked (shifted by one under the outer shift)."""
        if self.outer_shift:
            return torch.cat([masked[:, 1:], torch.zeros_like(masked[:, :1])], 1)
        return masked

    def mean_ce(self, logits, ids, masked) -> torch.Tensor:
        ce, sc = self.slot_ce(logits, ids, masked)
        return ce.sum(1) / sc.sum(1).clamp_min(1)


# ---------------------------------------------------------------------------------------------------- the lens
def fit_lens(reader: Reader, reads: Sequence[Tuple[torch.Tensor, torch.Tensor, G.DecodeState]], point: Point, block: int = 64) -> torch.Tensor:
    """``J [H, H]`` at ``point`` by the "sum" estimator: one-hot cotangents on every valid target slot at once, the gradient at
    a source slot summed over the targets, averaged over the valid source slots of every read ``(ids, masked, state)``."""
    H = reader.mc.hidden_size
    J = torch.zeros(H, H, dtype=torch.float64, device=reader.dev)
    n = 0
    for ids, masked, state in reads:
        x = torch.where(masked, torch.full_like(ids, reader.mc.mask_token_id), ids)
        with torch.enable_grad():
            h0, cap = reader.forward(x, state, capture=(point,))
            leaf = cap[point].detach().float().requires_grad_(True)
            h_L, _ = reader.forward(x, state, leaves={point: leaf})
            valid = reader.valid_slots(masked.to(reader.dev))
            vm = valid.to(h_L.dtype)[..., None]
            for a in range(0, H, block):
                eye = torch.zeros(min(block, H - a), *h_L.shape, dtype=h_L.dtype, device=reader.dev)
                for j in range(eye.shape[0]):
                    eye[j, ..., a + j] = 1.0
                (g,) = torch.autograd.grad(h_L, leaf, eye * vm, retain_graph=True, is_grads_batched=True)     # [blk, B, C, H]
                J[a:a + eye.shape[0]] += (g * vm).sum((1, 2)).double()
        n += int(valid.sum())
    return (J / max(n, 1)).float()


def decode_delta(reader: Reader, J: torch.Tensor, h_L: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    """Logit change the lens assigns to a residual contribution ``m [.., H]`` at the point ``J`` was fitted:
    ``lm_head . J_norm(h_L) . J m`` (the final norm linearised at ``h_L``)."""
    dm = (m.float() @ J.t().to(m.device))
    h = h_L.detach().float().requires_grad_(True)
    with torch.enable_grad():
        _, d = torch.autograd.functional.jvp(lambda t: reader.unembed(t), (h,), (dm,))
    return d


def direct_effect(reader: Reader, x: torch.Tensor, state: G.DecodeState, point: Point, m: torch.Tensor) -> torch.Tensor:
    """Exact first-order effect on the logits of adding ``m [B, C, H]`` at ``point``, all positions at once (a JVP of the
    network above the injection point, in context)."""
    zero = torch.zeros_like(m, dtype=torch.float32)

    def f(delta):
        h_L, _ = reader.forward(x, state, inject={point: delta})
        return reader.unembed(h_L)
    with torch.enable_grad():
        _, d = torch.autograd.functional.jvp(f, (zero,), (m.float(),))
    return d
