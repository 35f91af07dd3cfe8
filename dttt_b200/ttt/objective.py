"""Masked-diffusion objective pieces: the outer noising, the CART time weights, the inner masks.

Reference: ``src/ttt/objective.py`` — ``q_sample`` (``:54-77``), ``cart_kernel`` / ``band_correlate``
(``:80-109``), ``time_weights`` (``:112-125``), ``span_mask`` (``:131-142``), ``make_inner_mask``
(``:145-204``).  Keys are the counter-based keys of ``utils.rng`` with the reference's split order, a
single key ``[2]`` for a training batch or row-wise keys ``[B, 2]`` for evaluation draws that must not
depend on the batch shape.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from ..ops import reference as ref
from ..utils import rng


def to_chunks(x: torch.Tensor, chunk: int) -> torch.Tensor:
    """``[B, T, ...]`` -> ``[nc, B, C, ...]``."""
    B, T = x.shape[:2]
    return x.reshape(B, T // chunk, chunk, *x.shape[2:]).transpose(0, 1)


def from_chunks(x: torch.Tensor) -> torch.Tensor:
    nc, B, C = x.shape[:3]
    return x.transpose(0, 1).reshape(B, nc * C, *x.shape[3:])


def q_sample(key: torch.Tensor, ids: torch.Tensor, loss_mask: Optional[torch.Tensor], mask_token_id: int,
             t: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``t ~ U[0,1)`` per sequence, ``u ~ U[0,1)`` per token, ``t_mask = (u < t) & loss_mask``.
    Returns ``(x_t [B,T], t [B], t_mask [B,T])``."""
    B, T = ids.shape
    dev = ids.device
    # keys are derived where the key lives; the per-token draw happens on the tokens' device
    ks = rng.split(key, 2)
    if key.dim() == 2:                              # row-wise keys [B, 2]
        if t is None:
            t = rng.uniform(ks[:, 0], ())
        u = rng.uniform(ks[:, 1].to(dev), (T,))
    else:
        if t is None:
            t = rng.uniform(ks[0], (B,))
        u = rng.uniform(ks[1].to(dev), (B, T))
    t = t.to(dev).float()
    t_mask = u < t[:, None]
    if loss_mask is not None:
        t_mask = t_mask & loss_mask.bool()
    return torch.where(t_mask, torch.full_like(ids, mask_token_id), ids), t, t_mask


def time_weights(mode: str, t: Optional[torch.Tensor], t_mask: torch.Tensor, kernel: Optional[torch.Tensor]) -> torch.Tensor:
    """Per-token outer weights ``[B, T]`` f32 before masking (cart | linear | original | none)."""
    tm = t_mask.float()
    if mode == "cart":
        return cart_weights(1.0 - tm, kernel)
    if mode == "linear":
        return (1.0 - t)[:, None].expand_as(tm)
    if mode == "original":
        return (1.0 / torch.clamp(t, min=1e-6))[:, None].expand_as(tm)
    if mode == "none":
        return torch.ones_like(tm)
    raise ValueError(f"time_reweighting {mode!r}")


def cart_weights(visible: torch.Tensor, kernel: torch.Tensor) -> torch.Tensor:
    """Density of visible neighbours: the band correlation of ``visible [B, T]`` with the CART kernel."""
    from ..ops import kernels
    if visible.is_cuda and kernels.available("cart"):
        return kernels.cart_band(visible, kernel)
    return ref.band_correlate(visible, kernel)


def span_mask(key: torch.Tensor, n: int, ratio: torch.Tensor, span: float) -> torch.Tensor:
    """``[.., n]`` bool: geometric spans (mean ``span``) covering about ``ratio`` of the positions."""
    ks = rng.split(key, 2)
    starts = rng.uniform(ks[..., 0, :], (n,)) < (ratio / span)[..., None]
    lengths = 1 + torch.floor(torch.log(rng.uniform(ks[..., 1, :], (n,), 1e-6, 1.0))
                              / torch.log(torch.tensor(1.0 - 1.0 / span))).to(torch.int64)
    pos = torch.arange(n, device=key.device)
    ends = torch.where(starts, pos + torch.clamp(lengths, max=int(8 * span)), torch.zeros_like(lengths))
    return torch.cummax(ends, dim=-1).values > pos


def inner_masks(keys: torch.Tensor, chunks: torch.Tensor, ratio: float, ratio_range: Tuple[float, float],
                mask_token_id: int, pad_token_id: int, views: int = 1, span: float = 0.0,
                view_mode: str = "complement") -> Tuple[torch.Tensor, torch.Tensor]:
    """Batched inner mask draw: ``keys [..., 2]``, ``chunks [..., C]`` -> ``(x_inner, mask)`` shaped
    ``[..., C]`` for one view and ``[..., V, C]`` for more.  Pinned ratio (``ratio >= 0``): the key is
    the draw key; sampled: ``(k_ratio, k_draw) = split(key)``, ``ratio ~ U(lo, hi)``.  Pads are never masked."""
    lo, hi = float(ratio_range[0]), float(ratio_range[1])
    C = chunks.shape[-1]
    dev = chunks.device
    not_pad = chunks != pad_token_id
    mask_tok = torch.full_like(chunks, mask_token_id)
    if view_mode == "strata":
        ks = rng.split(keys, 3)
        u = rng.uniform(ks[..., 0, :], ())
        order = torch.argsort(rng.uniform(ks[..., 1, :], (views,)), dim=-1).float()
        r = (lo + (hi - lo) * (order + u[..., None]) / views).to(dev)           # [..., V]
        if span > 0:
            vk = rng.split(ks[..., 2, :], views)
            ms = span_mask(vk.to(dev), C, r, span)
        else:
            ms = rng.uniform(ks[..., 2, :].to(dev), (views, C)) < r[..., None]
        ms = ms & not_pad[..., None, :]
        return torch.where(ms, mask_tok[..., None, :], chunks[..., None, :]), ms
    if ratio is not None and ratio >= 0:
        r = torch.full(keys.shape[:-1], float(ratio), device=dev)
        k_draw = keys.to(dev)
    else:
        ks = rng.split(keys, 2)
        r = rng.uniform(ks[..., 0, :], (), lo, hi).to(dev)
        k_draw = ks[..., 1, :].to(dev)
    if span > 0:
        m = span_mask(k_draw, C, r, span) & not_pad
    else:
        m = (rng.uniform(k_draw, (C,)) < r[..., None]) & not_pad
    if views == 1:
        return torch.where(m, mask_tok, chunks), m
    ms = torch.stack([m, ~m & not_pad], dim=-2)
    return torch.where(ms, mask_tok[..., None, :], chunks[..., None, :]), ms
