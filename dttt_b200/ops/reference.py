"""Plain-PyTorch statements of every op: the oracle the CUDA kernels are tested against, the path
taken on CPU, and the differentiable form used when a backward pass must itself be differentiated
(the meta-gradient).  All of them are ordinary autograd-traceable torch code.

Reference sites: RMSNorm ``src/ttt/model.py:123-134``; RoPE ``:82-117``; attention
``src/ttt/attention.py:181-201``; dense CE ``src/ttt/fused_ce.py:127-132``; CART kernel and band
correlation ``src/ttt/objective.py:80-109``; the token-sequential gated delta rule
``src/ttt/gdn.py:106-136``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

NEG = -1e30


# ------------------------------------------------------------------ norms / activations
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x32 = x.float()
    var = x32.pow(2).mean(dim=-1, keepdim=True)
    return (weight.float() * (x32 * torch.rsqrt(var + eps))).to(x.dtype)


def act_fn(name: str):
    if name == "silu":
        return F.silu
    if name == "gelu":
        return lambda t: F.gelu(t, approximate="tanh")      # jax.nn.gelu defaults to the tanh form
    raise ValueError(name)


def glu(gate: torch.Tensor, up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    return act_fn(act)(gate) * up


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    x32 = x.float()
    return (x32 * torch.rsqrt(x32.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


# ------------------------------------------------------------------ rotary embedding
def llama3_inv_freq(inv_freq: torch.Tensor, scaling) -> torch.Tensor:
    s = dict(scaling)
    factor, low, high, old = s["factor"], s["low_freq_factor"], s["high_freq_factor"], s["original_max_position_embeddings"]
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > old / low, inv_freq / factor, inv_freq)
    smooth = (old / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < old / high) & ~(wavelen > old / low)
    return torch.where(medium, smoothed, scaled)


def rope_inv_freq(head_dim: int, theta: float, scaling=None, device=None) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    return llama3_inv_freq(inv, scaling) if scaling is not None else inv


def rope_cos_sin(pos: torch.Tensor, head_dim: int, theta: float, scaling=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``pos [...]`` -> ``cos, sin [..., head_dim]`` in f32 (the two halves repeat the same angles)."""
    inv = rope_inv_freq(head_dim, theta, scaling, pos.device)
    ang = pos.float().unsqueeze(-1) * inv
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [..., T, heads, d]`` with ``cos/sin [..., T, d]``; half-rotation layout ``[-x2, x1]``."""
    x32 = x.float()
    half = x32.shape[-1] // 2
    rot = torch.cat([-x32[..., half:], x32[..., :half]], dim=-1)
    return (x32 * cos.unsqueeze(-2) + rot * sin.unsqueeze(-2)).to(x.dtype)


# ------------------------------------------------------------------ attention
def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, key_valid: Optional[torch.Tensor], scale: float,
           own_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact attention.  ``q [n, C, nh, d]``, ``k/v [n, K, nkv, d]``, ``key_valid [n, K]`` bool (None = all),
    ``own_mask [C, M]`` bool restricting each query's view of the LAST ``M`` keys.  f32 scores and softmax,
    additive -1e30 masks.  Returns ``[n, C, nh, d]`` in ``q.dtype``."""
    n, C, nh, d = q.shape
    K, nkv = k.shape[1], k.shape[2]
    rep = nh // nkv
    qg = q.reshape(n, C, nkv, rep, d)
    s = torch.einsum("ncgrd,nkgd->ngrck", qg.float(), k.float()) * scale
    if key_valid is not None:
        s = s + torch.where(key_valid, 0.0, NEG).to(s.dtype)[:, None, None, None, :]
    if own_mask is not None:
        M = own_mask.shape[1]
        bias = torch.zeros(C, K, dtype=s.dtype, device=s.device)
        bias[:, K - M:] = torch.where(own_mask.to(s.device), 0.0, NEG)
        s = s + bias
    p = torch.softmax(s, dim=-1).to(v.dtype)
    o = torch.einsum("ngrck,nkgd->ncgrd", p.float(), v.float())
    return o.reshape(n, C, nh, d).to(q.dtype)


# ------------------------------------------------------------------ cross entropy
def weighted_ce_dense(h: torch.Tensor, emb: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """``sum_i w_i * CE(h_i @ emb^T, target_i)`` with f32 logits."""
    logits = h.float() @ emb.float().t()
    lp = torch.log_softmax(logits, dim=-1)
    return (weights.float() * (-lp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1))).sum()


def per_token_ce_dense(h: torch.Tensor, emb: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    logits = h.float() @ emb.float().t()
    lp = torch.log_softmax(logits, dim=-1)
    return -lp.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1)


def soft_ce_dense(h: torch.Tensor, emb: torch.Tensor, ids: torch.Tensor, probs: torch.Tensor,
                  weights: torch.Tensor) -> torch.Tensor:
    """``sum_i w_i sum_k q_ik CE(logits_i, id_ik)`` against a sparse (top-k) target distribution."""
    logits = h.float() @ emb.float().t()
    lp = torch.log_softmax(logits, dim=-1)
    return (weights.float() * (-(probs.float() * lp.gather(-1, ids.long())).sum(-1))).sum()


# ------------------------------------------------------------------ CART time weights
def cart_kernel(p: float = 0.1, window: int = 512, device=None) -> torch.Tensor:
    """``[2*window+1]``: ``0.5 p (1-p)^(|d|-1)``, zero at ``d = 0``."""
    d = torch.arange(-window, window + 1, device=device).abs().float()
    w = 0.5 * p * torch.pow(torch.tensor(1.0 - p, device=device), torch.clamp(d - 1.0, min=0.0))
    return torch.where(d == 0, torch.zeros_like(w), w)


def band_correlate(x: torch.Tensor, kernel: torch.Tensor) -> torch.Tensor:
    """``out[b, t] = sum_d kernel[d + W] x[b, t + d]`` (zero padded), ``x [B, T]`` f32."""
    W = (kernel.shape[0] - 1) // 2
    return F.conv1d(x.float().unsqueeze(1), kernel.float().view(1, 1, -1), padding=W).squeeze(1)


# ------------------------------------------------------------------ gated delta rule (token sequential)
def gdn_update_sequential(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, alpha: torch.Tensor,
                          S: torch.Tensor) -> torch.Tensor:
    """``S_t = a_t S_{t-1} + b_t (v_t - a_t S_{t-1} k_t) k_t^T`` over the tokens of one chunk.
    ``k [.., C, nh, dk]``, ``v [.., C, nh, dv]``, ``beta/alpha [.., C, nh]``, ``S [.., nh, dv, dk]`` (f32)."""
    S = S.float()
    C = k.shape[-3]
    for t in range(C):
        kt, vt = k[..., t, :, :].float(), v[..., t, :, :].float()
        Sd = alpha[..., t, :, None, None].float() * S
        err = vt - torch.einsum("...hvk,...hk->...hv", Sd, kt)
        S = Sd + beta[..., t, :, None, None].float() * torch.einsum("...hv,...hk->...hvk", err, kt)
    return S
