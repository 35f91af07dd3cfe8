"""Linear + cross-entropy over the (tied) embedding without a resident ``[N, V]`` tensor.

``weighted_ce(h, E, y, w) = sum_i w_i (logsumexp_v(h_i . E_v) - h_i . E_{y_i})`` — the reference's
``fused_weighted_ce`` (``src/ttt/fused_ce.py:28-121``): the forward streams the vocabulary in blocks
carrying a running (max, sum-exp); the backward recomputes each block's logits and forms
``d = g w (softmax - onehot)``, ``g_h += d E_b``, ``g_E_b = d^T h``.  ``E``'s gradient goes straight into
its f32 master buffer when the leaf carries ``grad_target`` (the GEMM epilogue accumulates), which is
also what keeps the tied embedding's gradient in f32 (reference model.py:534-542).

When the backward is recorded (inner loss under the meta-gradient) the dense statement is
differentiated instead, with the ``[N, V]`` logits produced in f32 by the bf16 tensor-core GEMM.

Also here: ``per_token_ce`` (``fused_ce.py:76-81``), ``soft_weighted_ce`` against a sparse top-k
teacher distribution (``:151-213``) and the streaming ``topk_logprobs`` (``:224-259``).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import gemm as _gemm
from . import reference as ref
from .functional import mm, staged, use_kernels, _INNER_BACKWARD


def _blocks(V: int, block: int):
    block = block if block > 0 else V
    return [(s, min(V, s + block)) for s in range(0, V, block)]


def _stream_lse(h: torch.Tensor, E: torch.Tensor, block: int) -> torch.Tensor:
    """``logZ [N]`` (f32) of ``h @ E^T``, one vocabulary block at a time."""
    N = h.shape[0]
    if _fused(h, E):
        from . import kernels
        return kernels.linear_ce_fwd(h, E, torch.zeros(N, dtype=torch.int32, device=h.device))[0]
    run_max = torch.full((N,), float("-inf"), dtype=torch.float32, device=h.device)
    run_sum = torch.zeros(N, dtype=torch.float32, device=h.device)
    for s, e in _blocks(E.shape[0], block):
        logits = _block_logits(h, E[s:e])
        bmax = logits.max(dim=-1).values
        new_max = torch.maximum(run_max, bmax)
        run_sum = run_sum * torch.exp(run_max - new_max) + torch.exp(logits - new_max[:, None]).sum(-1)
        run_max = new_max
    return run_max + torch.log(run_sum)


def _fused(h: torch.Tensor, E: torch.Tensor) -> bool:
    """Whether the GEMM-epilogue kernels (``csrc/gemm_tcgen05.cu``, the cross-entropy epilogues) take this call."""
    if not (use_kernels(h) and h.is_cuda):
        return False
    from . import kernels
    return kernels.available("linear_ce") and kernels.linear_ce_supported(h, E)


def _block_logits(h: torch.Tensor, Eb: torch.Tensor) -> torch.Tensor:
    if use_kernels(h) and Eb.dtype == torch.bfloat16:
        return _gemm.gemm_raw(h, Eb, False, True, torch.float32)
    return h.float() @ Eb.float().t()


def _target_logit(h: torch.Tensor, E: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    return (h.float() * E[targets.long()].float()).sum(-1)


# ---- staged pieces
def _ce_ref(h, E, targets, weights, block, target=None):
    """Dense, differentiable to any order; the logits come from the tensor-core GEMM on the GPU."""
    logits = mm(h, E if E.dtype == h.dtype else E.to(h.dtype), False, True, out_dtype=torch.float32) \
        if use_kernels(h) else h.float() @ E.float().t()
    lse = torch.logsumexp(logits, dim=-1)
    tgt = logits.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)
    return (weights.float() * (lse - tgt)).sum()


def _ce_fwd(h, E, targets, weights, block, target=None):
    with torch.no_grad():
        if _fused(h, E):
            from . import kernels
            logZ, nll = kernels.linear_ce_fwd(h, E, targets)
            return (weights.float() * nll).sum(), (logZ,)
        logZ = _stream_lse(h, E, block)
        loss = (weights.float() * (logZ - _target_logit(h, E, targets))).sum()
    return loss, (logZ,)


def _ce_bwd(g, tensors, saved, needs, block, target=None):
    h, E, targets, weights = tensors
    (logZ,) = saved
    need_h, need_E = needs[0], needs[1] and not _INNER_BACKWARD[0]
    gw = (g.float() * weights.float())
    g_h = torch.zeros(h.shape, dtype=torch.float32, device=h.device) if need_h else None
    kern = use_kernels(h) and E.dtype == torch.bfloat16
    g_E = None
    if need_E and not (kern and target is not None):
        g_E = torch.zeros(E.shape, dtype=torch.float32, device=E.device)
    if need_E and kern and target is not None:
        gfull, layer = target
        gbuf = gfull if layer is None else gfull[layer]
    tl = targets.long()
    fused = _fused(h, E)
    if fused:
        from . import kernels
        ti, gwc = targets.to(torch.int32).contiguous(), gw.contiguous()
    for s, e in _blocks(E.shape[0], block):
        if fused:
            db = kernels.linear_ce_dlogits(h, E[s:e], ti, gwc, logZ, s)
        else:
            logits = _block_logits(h, E[s:e])
            d = torch.exp(logits - logZ[:, None])
            inb = (tl >= s) & (tl < e)
            d.scatter_add_(1, (tl - s).clamp(0, e - s - 1).unsqueeze(1), -inb.to(d.dtype).unsqueeze(1))
            d = d * gw[:, None]
        if kern:
            if not fused:
                db = d.to(torch.bfloat16)
            if need_h:
                _gemm.gemm_raw(db, E[s:e], False, False, torch.float32, out=g_h, accumulate=True)
            if need_E:
                if target is not None:
                    _gemm.gemm_raw(db, h, True, False, torch.float32, out=gbuf[s:e], accumulate=True)
                else:
                    _gemm.gemm_raw(db, h, True, False, torch.float32, out=g_E[s:e], accumulate=False)
        else:
            if need_h:
                g_h += d @ E[s:e].float()
            if need_E:
                g_E[s:e] = d.t() @ h.float()
    return (g_h.to(h.dtype) if need_h else None, g_E.to(E.dtype) if g_E is not None else None, None, None)


# ---- the backward as a differentiable operation (recorded inner pass)
SECOND_ORDER_KERNEL = True


def second_order(c, g, h, E, targets, weights, logZ):
    """Derivative of ``g_h = g w (p E - E_y)`` (the cross-entropy backward w.r.t. ``h``) contracted with the cotangent
    ``c [N, H]``: returns ``(grad g, grad h [N, H] f32, r, d, grad w)`` where E's gradient is ``r^T h + d^T c``
    (left to the caller, who may accumulate it in place).  With ``u = c E^T`` and ``ubar = rowsum(p o u)``:
    ``r = gw p o (u - ubar)``, ``d = gw (p - onehot)``, ``grad h = r E``, ``grad g = sum_i w_i (ubar_i - u_iy)``."""
    gw = g.float() * weights.float()
    tl = targets.long()
    if h.is_cuda:
        from . import kernels
        Eb = E if E.dtype == torch.bfloat16 else E.to(torch.bfloat16)
        hb, cb = h.to(torch.bfloat16), c.to(torch.bfloat16)
        z = _gemm.gemm_raw(hb, Eb, False, True, torch.float32)
        u = _gemm.gemm_raw(cb, Eb, False, True, torch.float32)
        ubar = kernels.ce_bwd2_rowdot(z, u, logZ)
        r, d = kernels.ce_bwd2_make(z, u, logZ, ubar, gw, targets)
        del z, u
        g_h = _gemm.gemm_raw(r, Eb, False, False, torch.float32)
    else:
        z = h.float() @ E.float().t()
        u = c.float() @ E.float().t()
        p = torch.exp(z - logZ[:, None])
        ubar = (p * u).sum(-1)
        r = gw[:, None] * p * (u - ubar[:, None])
        d = gw[:, None] * p
        d[torch.arange(d.shape[0]), tl] -= gw
        g_h = r @ E.float()
    u_y = (c.float() * E[tl].float()).sum(-1)
    diff = ubar - u_y
    return (weights.float() * diff).sum(), g_h, r, d, g.float() * diff


class _CEBwd(torch.autograd.Function):
    """``(g, h, E, targets, weights, logZ) -> g_h`` by the streaming first-order backward; differentiable once more by
    ``second_order``.  ``logZ`` is a cache of the forward, not an independent input."""

    @staticmethod
    def forward(ctx, g, h, E, targets, weights, logZ, block, target):
        ctx.save_for_backward(g, h, E, targets, weights, logZ)
        ctx.target = target
        return _ce_bwd(g, (h, E, targets, weights), (logZ,), (True, False, False, False), block, target)[0]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, c):
        g, h, E, targets, weights, logZ = ctx.saved_tensors
        g_g, g_h, r, d, g_w = second_order(c, g, h, E, targets, weights, logZ)
        g_E = None
        if ctx.needs_input_grad[2]:
            if h.is_cuda:
                hb, cb = h.to(torch.bfloat16), c.to(torch.bfloat16)
                if ctx.target is not None:
                    gfull, layer = ctx.target
                    gbuf = gfull if layer is None else gfull[layer]
                    _gemm.gemm_raw(r, hb, True, False, torch.float32, out=gbuf, accumulate=True)
                    _gemm.gemm_raw(d, cb, True, False, torch.float32, out=gbuf, accumulate=True)
                else:
                    acc = _gemm.gemm_raw(r, hb, True, False, torch.float32)
                    _gemm.gemm_raw(d, cb, True, False, torch.float32, out=acc, accumulate=True)
                    g_E = acc.to(E.dtype)
            else:
                g_E = (r.t() @ h.float() + d.t() @ c.float()).to(E.dtype)
        return (g_g if ctx.needs_input_grad[0] else None, g_h.to(h.dtype) if ctx.needs_input_grad[1] else None, g_E, None,
                g_w.to(weights.dtype) if ctx.needs_input_grad[4] else None, None, None, None)


def _ce_diff_bwd(g, tensors, saved, needs, block, target=None):
    """The recorded backward of the inner loss (only ``h``'s gradient is wanted there), or ``None`` to decline."""
    h, E, targets, weights = tensors
    if not SECOND_ORDER_KERNEL or not needs[0] or (needs[1] and not _INNER_BACKWARD[0]) or not _fused(h, E) or E.shape[0] % 4:
        return None
    from . import kernels
    if not kernels.available("linear_ce_bwd2"):
        return None
    return (_CEBwd.apply(g, h, E, targets, weights, saved[0], block, target), None, None, None)


_SPEC = (_ce_fwd, _ce_bwd, _ce_ref, _ce_diff_bwd)


def weighted_ce(h: torch.Tensor, E: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor, block: int = 8192) -> torch.Tensor:
    """``sum_i w_i CE_i`` (f32 scalar).  ``block == 0``: the dense reference (tests)."""
    if block <= 0:
        return ref.weighted_ce_dense(h, E, targets, weights)
    if not h.is_cuda and not _gemm.EMULATE:
        # CPU: the streamed forward is only a memory device; autograd through the dense statement is exact
        return ref.weighted_ce_dense(h, E, targets, weights)
    return staged(_SPEC, (h, E, targets, weights), (block, getattr(E, "grad_target", None)))


@torch.no_grad()
def per_token_ce(h: torch.Tensor, E: torch.Tensor, targets: torch.Tensor, block: int = 8192) -> torch.Tensor:
    """``[N]`` cross-entropy of every row, forward only."""
    if block <= 0:
        return ref.per_token_ce_dense(h, E, targets)
    if _fused(h, E):
        from . import kernels
        return kernels.linear_ce_fwd(h, E, targets)[1]
    return _stream_lse(h, E, block) - _target_logit(h, E, targets)


def soft_weighted_ce(h: torch.Tensor, E: torch.Tensor, ids: torch.Tensor, probs: torch.Tensor, weights: torch.Tensor,
                     block: int = 8192) -> torch.Tensor:
    """``sum_i w_i sum_k q_ik CE(logits_i, id_ik)``: ``= sum_i w_i (sum_k q_ik) logZ_i - sum_i w_i sum_k q_ik h_i.E_id``.
    Built from differentiable pieces (the log-partition term reuses ``weighted_ce``'s machinery through a
    zero-target trick is not needed: logZ is taken from the dense / streamed logits directly)."""
    if block <= 0 or not h.is_cuda:
        return ref.soft_ce_dense(h, E, ids, probs, weights)
    logits = mm(h, E if E.dtype == h.dtype else E.to(h.dtype), False, True, out_dtype=torch.float32)
    lse = torch.logsumexp(logits, dim=-1)
    picked = logits.gather(-1, ids.long())
    q = probs.float()
    return (weights.float() * (q.sum(-1) * lse - (q * picked).sum(-1))).sum()


@torch.no_grad()
def topk_logprobs(h: torch.Tensor, E: torch.Tensor, k: int, block: int = 8192) -> Tuple[torch.Tensor, torch.Tensor]:
    """Streaming top-k over the vocabulary with exact log-probabilities: ``(ids [N, k], logp [N, k])``."""
    N, V = h.shape[0], E.shape[0]
    logZ = _stream_lse(h, E, block)
    best_v = torch.full((N, k), float("-inf"), dtype=torch.float32, device=h.device)
    best_i = torch.zeros((N, k), dtype=torch.long, device=h.device)
    for s, e in _blocks(V, block):
        logits = _block_logits(h, E[s:e])
        kk = min(k, e - s)
        v, i = logits.topk(kk, dim=-1)
        cat_v = torch.cat([best_v, v], dim=-1)
        cat_i = torch.cat([best_i, i + s], dim=-1)
        best_v, sel = cat_v.topk(k, dim=-1)
        best_i = cat_i.gather(-1, sel)
    return best_i, best_v - logZ[:, None]
