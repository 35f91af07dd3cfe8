"""The attention backward as a differentiable operation: forward = the flash backward kernel, backward = its
derivative written out by hand (the "second order" of attention, which the outer gradient of the training objective
needs through every inner write; the reference obtains it from JAX differentiating ``attend_xla``,
reference src/ttt/attention.py:181-201, inside ``chunk_scan``'s ``jax.grad`` of the inner loss).

With ``P = softmax(scale Q K^T)``, ``dP = dO V^T``, ``D = rowsum(P o dP)`` the first backward is

    dS = P o (dP - D)        dQ = scale dS K        dK = scale dS^T Q        dV = P^T dO

and for cotangents ``(gQ, gK, gV)`` of ``(dQ, dK, dV)``

    gdS = scale (gQ K^T + Q gK^T)        X = dO gV^T
    E   = rowsum(P o gdS)                F = rowsum(P o X) + rowsum(gdS o dS) - E D
    gdP = P o (gdS - E)                  gS = P o X + gdS o dS - E (P o dP) - F P
    grad dO = P gV + gdP V               grad V = gdP^T dO
    grad Q  = scale (gS K + dS gK)       grad K = scale (gS^T Q + dS^T gQ)

On the GPU the score stage (the four score-shaped products, the row sums, the four bf16 operand matrices
``P, scale dS, gdP, scale gS``) is one tcgen05 kernel that keeps the scores in tensor memory
(``csrc/attn_bwd2_tcgen05.cu``; head dimension 64, chunk a multiple of 128, keys a multiple of 64); other shapes
form the score products with the tensor-core GEMM in f32 and run ``csrc/attn_bwd2_rows.cu`` over them.  The seven
output products run on the tcgen05 GEMM, batched over (sequence, KV head) with the query heads of a group folded
into the rows.  ``second_order`` is also stated in plain PyTorch
(f32) for CPU tensors; the tests compare both against autograd differentiating the reference statement twice.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.autograd.function import once_differentiable


# the score stage runs on the tcgen05 kernel where its shape limits hold (False: f32 score GEMMs + the row kernel)
FUSED_SCORES = True


def _rows(t: torch.Tensor, nkv: int) -> torch.Tensor:
    """``[n, C, nh, d] -> [n * nkv, G * C, d]`` (head ``h = kv * G + g``, row ``g * C + c``)."""
    n, C, nh, d = t.shape
    G = nh // nkv
    return t.reshape(n, C, nkv, G, d).permute(0, 2, 3, 1, 4).reshape(n * nkv, G * C, d)


def _unrows(t: torch.Tensor, n: int, C: int, nh: int) -> torch.Tensor:
    B, R, d = t.shape
    nkv = B // n
    G = nh // nkv
    return t.reshape(n, nkv, G, C, d).permute(0, 3, 1, 2, 4).reshape(n, C, nh, d)


def _keys(t: torch.Tensor) -> torch.Tensor:
    """``[n, Kn, nkv, d] -> [n * nkv, Kn, d]``."""
    n, Kn, nkv, d = t.shape
    return t.permute(0, 2, 1, 3).reshape(n * nkv, Kn, d)


def _unkeys(t: torch.Tensor, n: int) -> torch.Tensor:
    B, Kn, d = t.shape
    return t.reshape(n, B // n, Kn, d).permute(0, 2, 1, 3)


def _rows_torch(S, dP, gdS, X, lse, delta, chunk, causal, scale):
    """The row stage in PyTorch (f32): same inputs and outputs as ``kernels.attention_bwd2_rows`` (outputs f32)."""
    Kn = S.shape[-1]
    p = torch.exp(S * scale - lse[..., None])
    if causal:
        c = torch.arange(S.shape[-2], device=S.device) % chunk
        j = torch.arange(Kn, device=S.device)
        p = p * (j[None, :] <= (c[:, None] + (Kn - chunk))).to(p.dtype)
    gds = gdS * scale
    D = delta[..., None]
    E = (p * gds).sum(-1, keepdim=True)
    dS = p * (dP - D)
    F = (p * X).sum(-1, keepdim=True) + (gds * dS).sum(-1, keepdim=True) - E * D
    gdP = p * (gds - E)
    gS = p * X + gds * dS - E * p * dP - F * p
    return p, dS * scale, gdP, gS * scale


def _fused_ok(q: torch.Tensor, Kn: int) -> bool:
    from . import kernels
    return (FUSED_SCORES and kernels.available("attention_bwd2_scores") and q.shape[-1] == 64 and q.shape[1] % 128 == 0
            and Kn % 64 == 0)


def supported(q: torch.Tensor, Kn: int) -> bool:
    """Whether ``second_order`` has a kernel path for this call: the tcgen05 score stage (any number of keys), or the row kernel
    over f32 score products (up to ``kernels.ATTN_BWD2_MAX_KEYS`` keys, a multiple of 4)."""
    from . import kernels
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] % 8 == 0):
        return False
    return _fused_ok(q, Kn) or (kernels.available("attention_bwd2") and Kn % 4 == 0 and Kn <= kernels.ATTN_BWD2_MAX_KEYS)


def second_order(gQ: Optional[torch.Tensor], gK: Optional[torch.Tensor], gV: Optional[torch.Tensor], dO: torch.Tensor,
                 q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, o: torch.Tensor, lse: torch.Tensor, scale: float,
                 causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of ``<gQ, dQ> + <gK, dK> + <gV, dV>`` w.r.t. ``(dO, q, K, V)`` where ``(dQ, dK, dV)`` is the attention
    backward at ``(q, K, V, dO)``.  ``q, dO, o, gQ [n, C, nh, d]``; ``K, V, gK, gV [n, Kn, nkv, d]``; ``lse [n, nh, C]`` (natural
    log-sum-exp of the scaled scores); ``causal`` aligned to the end of the key axis.  A ``None`` cotangent counts as zero."""
    n, C, nh, d = q.shape
    Kn, nkv = K.shape[1], K.shape[2]
    G = nh // nkv
    gQ = torch.zeros_like(q) if gQ is None else gQ
    gK = torch.zeros_like(K) if gK is None else gK
    gV = torch.zeros_like(V) if gV is None else gV
    delta_h = (dO.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()                  # [n, nh, C]
    delta = delta_h.reshape(n * nkv, G * C)
    lse_r = lse.reshape(n * nkv, G * C).contiguous().float()
    if q.is_cuda:
        from . import kernels
        from .gemm import gemm_raw
        bf = torch.bfloat16
        qg, dOg, gQg = (_rows(t.to(bf), nkv).contiguous() for t in (q, dO, gQ))
        kg, vg, gKg, gVg = (_keys(t.to(bf)).contiguous() for t in (K, V, gK, gV))
        f32 = torch.float32
        if _fused_ok(q, Kn) and kernels.attention_bwd2_scores_supported(q, K):
            # scores in tensor memory, never in global memory
            P, dS, gdP, gS = kernels.attention_bwd2_scores(q, dO.to(bf), gQ.to(bf), K, V.to(bf), gK.to(bf), gV.to(bf),
                                                           lse.float(), delta_h, scale, causal)
        else:
            S = gemm_raw(qg, kg, False, True, f32)
            dP = gemm_raw(dOg, vg, False, True, f32)
            gdS = gemm_raw(torch.cat([gQg, qg], -1), torch.cat([kg, gKg], -1), False, True, f32)
            X = gemm_raw(dOg, gVg, False, True, f32)
            P, dS, gdP, gS = kernels.attention_bwd2_rows(S, dP, gdS, X, lse_r, delta, C, causal, scale)
            del S, dP, gdS, X
        g_dO = gemm_raw(P, gVg, False, False, f32)
        gemm_raw(gdP, vg, False, False, f32, out=g_dO, accumulate=True)
        g_V = gemm_raw(gdP, dOg, True, False)
        g_q = gemm_raw(gS, kg, False, False, f32)
        gemm_raw(dS, gKg, False, False, f32, out=g_q, accumulate=True)
        g_K = gemm_raw(gS, qg, True, False, f32)
        gemm_raw(dS, gQg, True, False, f32, out=g_K, accumulate=True)
    else:
        f = lambda t: t.float()
        qg, dOg, gQg = (_rows(f(t), nkv) for t in (q, dO, gQ))
        kg, vg, gKg, gVg = (_keys(f(t)) for t in (K, V, gK, gV))
        T = lambda t: t.transpose(-1, -2)
        S, dP = qg @ T(kg), dOg @ T(vg)
        gdS = gQg @ T(kg) + qg @ T(gKg)
        X = dOg @ T(gVg)
        P, dS, gdP, gS = _rows_torch(S, dP, gdS, X, lse_r, delta, C, causal, scale)
        g_dO = P @ gVg + gdP @ vg
        g_V = T(gdP) @ dOg
        g_q = gS @ kg + dS @ gKg
        g_K = T(gS) @ qg + T(dS) @ gQg
    return (_unrows(g_dO, n, C, nh).to(dO.dtype), _unrows(g_q, n, C, nh).to(q.dtype), _unkeys(g_K, n).to(K.dtype),
            _unkeys(g_V, n).to(V.dtype))


class _AttnBwd(torch.autograd.Function):
    """``(dO, q, kw, vw, ko, vo, o, lse) -> (dq, dkw, dvw, dko, dvo)`` on the flash backward kernel (``ko / vo`` may be
    ``None``: one key segment, three results); differentiable once more by ``second_order``.  ``o`` and ``lse`` are caches of
    the forward, not independent inputs: the derivative treats ``D`` and ``P`` as functions of ``(q, K, V, dO)``."""

    @staticmethod
    def forward(ctx, g, q, kw, vw, ko, vo, o, lse, scale, causal):
        from . import kernels
        ctx.save_for_backward(g, q, kw, vw, ko, vo, o, lse)
        ctx.scale, ctx.causal = scale, causal
        res = kernels.attention_bwd(g.contiguous(), q, kw, vw, o, lse, scale, causal, k2=ko, v2=vo)
        return tuple(res)

    @staticmethod
    @once_differentiable
    def backward(ctx, *cots):
        g, q, kw, vw, ko, vo, o, lse = ctx.saved_tensors
        two = ko is not None
        if two:
            gq, gkw, gvw, gko, gvo = cots
            z = lambda c, like: torch.zeros_like(like) if c is None else c
            K, V = torch.cat([kw, ko.to(kw.dtype)], 1), torch.cat([vw, vo.to(vw.dtype)], 1)
            if gkw is None and gko is None:
                gK = None
            else:
                gK = torch.cat([z(gkw, kw), z(gko, ko).to(kw.dtype)], 1)
            if gvw is None and gvo is None:
                gV = None
            else:
                gV = torch.cat([z(gvw, vw), z(gvo, vo).to(vw.dtype)], 1)
        else:
            gq, gK, gV = cots
            K, V = kw, vw
        g_dO, g_q, g_K, g_V = second_order(gq, gK, gV, g, q, K, V, o, lse, ctx.scale, ctx.causal)
        Kw = kw.shape[1]
        if two:
            outs = (g_dO, g_q, g_K[:, :Kw], g_V[:, :Kw], g_K[:, Kw:].to(ko.dtype), g_V[:, Kw:].to(vo.dtype))
        else:
            outs = (g_dO, g_q, g_K, g_V, None, None)
        outs = tuple(t if nd else None for t, nd in zip(outs, ctx.needs_input_grad[:6]))
        return (*outs, None, None, None, None)


def attention_bwd_diff(g, q, kw, vw, ko, vo, o, lse, scale, causal):
    """The attention backward with a graph: ``(dq, dkw, dvw[, dko, dvo])``."""
    return _AttnBwd.apply(g, q, kw, vw, ko, vo, o, lse, scale, causal)
