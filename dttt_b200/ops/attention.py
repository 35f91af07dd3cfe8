"""Chunk-window attention.

Geometry (reference ``src/ttt/attention.py:5-10``): a chunk of ``C`` query slots attends to the clean
keys of the previous ``W`` chunks plus the keys of its own chunk; inside the own chunk the pattern is
``full`` (bidirectional), ``causal``, ``split:K`` or ``block:b``; the sub-block read adds the chunk's
clean keys as a second own-chunk key set (``[C, 2C]`` pattern).  Window slots that precede the sequence
start, or lie beyond ``reach`` chunks, are invalid.  The window is stored oldest chunk first, so the
valid keys are always a *suffix* of the window followed by the own chunk: the fast path slices that
suffix instead of masking, and batches all calls that share a valid length.

``attend`` is the general entry point (explicit key validity, exact semantics of the reference's
``attend_xla``, ``attention.py:181-201``).  ``attend_window`` is what the model calls.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Optional, Tuple

import torch

from . import reference as ref
from .functional import staged, use_kernels


# ------------------------------------------------------------------ geometry
def window_gather(x: torch.Tensor, chunk: int, window: int, prev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [B, T, ...]`` -> ``[B, nc, window*chunk, ...]``: for chunk ``c`` the tokens of chunks
    ``[c-window, c)``; ``prev [B, window*chunk, ...]`` is what precedes ``x`` (zeros when absent)."""
    B, T = x.shape[:2]
    nc, WC = T // chunk, window * chunk
    if WC == 0:
        return x.new_zeros((B, nc, 0) + tuple(x.shape[2:]))
    pad = x.new_zeros((B, WC) + tuple(x.shape[2:])) if prev is None else prev.to(x.dtype)
    xp = torch.cat([pad, x], dim=1)
    idx = (torch.arange(nc, device=x.device)[:, None] * chunk + torch.arange(WC, device=x.device)[None, :])
    return xp[:, idx]


class _WindowGroups(torch.autograd.Function):
    """The KV windows of runs of chunks that see the same number of window chunks, cut out of ``[prev | x]`` in one
    node: ``groups = ((n_valid, first_chunk, count), ...)`` -> one ``[B * count, n_valid * chunk, ...]`` tensor per
    group holding, for every chunk of the run, the newest ``n_valid`` chunks before it.  One node means one gradient
    buffer: the backward adds every window's gradient into a single ``[prev | x]``-shaped tensor instead of
    materialising a full-size zero tensor per slice."""

    @staticmethod
    def forward(ctx, x, prev, chunk, window, groups):
        B, T = x.shape[:2]
        rest = tuple(x.shape[2:])
        WC = window * chunk
        pad = x.new_zeros((B, WC) + rest) if prev is None else prev.to(x.dtype)
        xp = torch.cat([pad, x], dim=1).contiguous()
        sB, sT = xp.stride(0), xp.stride(1)
        outs = []
        for nv, c0, cnt in groups:
            if nv == 0:
                outs.append(x.new_zeros((B * cnt, 0) + rest))
                continue
            v = xp.as_strided((B, cnt, nv * chunk) + rest, (sB, chunk * sT, sT) + tuple(xp.stride()[2:]),
                              xp.storage_offset() + (c0 + window - nv) * chunk * sT)
            outs.append(v.reshape((B * cnt, nv * chunk) + rest))
        ctx.meta = (B, T, rest, chunk, window, tuple(groups), prev is not None)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *gs):
        B, T, rest, chunk, window, groups, has_prev = ctx.meta
        WC = window * chunk
        gxp = None
        for (nv, c0, cnt), g in zip(groups, gs):
            if g is None or nv == 0:
                continue
            if gxp is None:
                gxp = g.new_zeros((B, WC + T) + rest)
            g5 = g.reshape((B, cnt, nv, chunk) + rest)
            for j in range(nv):
                a = (c0 + window - nv + j) * chunk
                gxp[:, a:a + cnt * chunk] += g5[:, :, j].reshape((B, cnt * chunk) + rest)
        if gxp is None:
            return None, None, None, None, None
        return gxp[:, WC:], (gxp[:, :WC] if has_prev else None), None, None, None


def window_groups(x: torch.Tensor, chunk: int, window: int, prev: Optional[torch.Tensor], groups):
    """See ``_WindowGroups``; ``groups`` as ``[(n_valid, first_chunk, count), ...]`` with chunk indices relative to ``x``."""
    return _WindowGroups.apply(x, prev, chunk, window, tuple(groups))


def valid_window_chunks(chunk_idx: int, window: int, reach: Optional[int]) -> int:
    """How many of the newest window chunks chunk ``chunk_idx`` may see."""
    n = min(chunk_idx, window)
    return n if reach is None else min(n, reach)


def key_validity(chunk_idx, chunk: int, window: int, reach=None, device=None) -> torch.Tensor:
    """``[(window+1)*chunk]`` bool, as reference attention.py:109-120."""
    j = torch.arange(window * chunk, device=device)
    win = (chunk_idx - window + j // chunk) >= 0
    if reach is not None:
        win = win & (j // chunk >= window - reach)
    return torch.cat([win, torch.ones(chunk, dtype=torch.bool, device=device)])


def key_validity_all(nc: int, chunk: int, window: int, first: int = 0, reach=None, device=None) -> torch.Tensor:
    return torch.stack([key_validity(first + c, chunk, window, reach, device) for c in range(nc)])


@lru_cache(maxsize=64)
def _own_mask_cpu(chunk: int, own: str) -> Optional[torch.Tensor]:
    if own == "full":
        return None
    i = torch.arange(chunk)[:, None]
    j = torch.arange(chunk)[None, :]
    if own == "causal":
        return j <= i
    if own.startswith("split:"):
        K = int(own.split(":")[1])
        return (j < K) | ((i >= K) & (j <= i))
    if own.startswith("block:"):
        b = int(own.split(":")[1])
        return (j // b) <= (i // b)
    raise ValueError(f"own-chunk mode {own!r}")


_DEV_MASKS = {}


def own_mask_matrix(chunk: int, own: str, device=None) -> Optional[torch.Tensor]:
    """``[C, C]`` bool own-chunk pattern (None for ``full``); reference attention.py:132-150.  Cached per device."""
    m = _own_mask_cpu(chunk, own)
    if m is None or device is None or torch.device(device).type == "cpu":
        return m
    key = (chunk, own, str(device))
    d = _DEV_MASKS.get(key)
    if d is None:
        d = _DEV_MASKS[key] = m.to(device)
    return d


def read_mask_matrix(chunk: int, block: int, device=None) -> torch.Tensor:
    """``[C, 2C]`` bool: the sub-block read over ``[clean own keys, noisy own keys]`` (attention.py:153-159)."""
    i = torch.arange(chunk, device=device)[:, None] // block
    j = torch.arange(chunk, device=device)[None, :] // block
    return torch.cat([j < i, j == i], dim=1)


# ------------------------------------------------------------------ general attention
def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, key_valid: Optional[torch.Tensor], scale: float,
           own_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact masked attention, any order of differentiation (``ops.reference.attend``)."""
    return ref.attend(q, k, v, key_valid, scale, own_mask)


def attend_window(q: torch.Tensor, k_own: torch.Tensor, v_own: torch.Tensor, k_win: torch.Tensor, v_win: torch.Tensor,
                  n_valid: int, chunk: int, scale: float, own: str = "full", inner: bool = False,
                  own_mask: Optional[torch.Tensor] = None,
                  extra_own: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """One batch of chunk calls that all see the newest ``n_valid`` window chunks.

    ``q [n, Cq, nh, d]``; ``k_own/v_own [n, Cq, nkv, d]``; ``k_win/v_win [n, Wc*C, nkv, d]`` (oldest first);
    ``own``: the own-chunk pattern by name, or pass an explicit ``own_mask [Cq, M]``;
    ``extra_own``: the chunk's clean K/V placed between the window and the own keys (sub-block read).
    ``inner``: this call's backward will itself be differentiated.
    """
    WC = k_win.shape[1]
    kw, vw = k_win[:, WC - n_valid * chunk:], v_win[:, WC - n_valid * chunk:]
    named = own_mask is None or extra_own is not None      # the pattern is one the kernels know by name
    pattern = own
    if extra_own is not None:
        # sub-block read: [window | clean own keys | noisy own keys]; its [C, 2C] mask is the "read" pattern of the model's read_block
        if own_mask is None or own_mask.shape[-1] != 2 * q.shape[1]:
            named = False
        else:
            pattern = f"read:{_read_block_of(own_mask)}"
    if named and use_kernels(q) and _pattern_ok(q, kw, k_own, pattern):
        if extra_own is not None:
            kw = torch.cat([kw, extra_own[0].to(kw.dtype)], dim=1)
            vw = torch.cat([vw, extra_own[1].to(vw.dtype)], dim=1)
        if kw.shape[1] > 0 and _two_segment_ok(q, kw, k_own):
            # window and own keys stay separate tensors: the kernels read (and, backward, write) both pairs directly
            return staged((_fast_fwd2, _fast_bwd2, _ref_for_staged2, _diff_bwd2), (q, kw, vw, k_own.to(kw.dtype), v_own.to(vw.dtype)),
                          (scale, pattern))
        K = torch.cat([kw, k_own.to(kw.dtype)], dim=1) if kw.shape[1] else k_own
        V = torch.cat([vw, v_own.to(vw.dtype)], dim=1) if vw.shape[1] else v_own
        return staged((_fast_fwd, _fast_bwd, _ref_for_staged, _diff_bwd), (q, K, V), (scale, pattern))
    parts_k = [kw] + ([extra_own[0].to(k_own.dtype)] if extra_own is not None else []) + [k_own]
    parts_v = [vw] + ([extra_own[1].to(v_own.dtype)] if extra_own is not None else []) + [v_own]
    K = torch.cat(parts_k, dim=1) if len(parts_k) > 1 or n_valid else k_own
    V = torch.cat(parts_v, dim=1) if len(parts_v) > 1 or n_valid else v_own
    if own_mask is None and own != "full":
        own_mask = own_mask_matrix(q.shape[1], own, q.device)
    if use_kernels(q) and own_mask is None:
        return staged((_fast_fwd, _fast_bwd, _ref_for_staged, _diff_bwd), (q, K, V), (scale, "full"))
    return ref.attend(q, K, V, None, scale, own_mask)


def _read_block_of(read_mask: torch.Tensor) -> int:
    """Sub-block length of a ``read_mask_matrix``: the number of own (second-half) keys the first query sees."""
    C = read_mask.shape[0]
    key = (C, read_mask.data_ptr())
    b = _READ_BLOCKS.get(key)
    if b is None:
        b = _READ_BLOCKS[key] = int(read_mask[0, C:].sum().item())
    return b


_READ_BLOCKS = {}


def _pattern_ok(q, kw, k_own, pattern: str) -> bool:
    """Can the kernels run this pattern on these shapes?  ``full`` / ``causal`` always (any chunk length); the others need
    chunks that are multiples of 128 and, for the backward, head dimension 64."""
    from . import kernels
    if not (kernels.available("attention") and kernels.attention_supported(q, k_own)):
        return False
    mode, _ = kernels.parse_pattern(pattern)
    if mode <= 1:
        return True
    return q.is_cuda and q.shape[1] % 128 == 0 and kw.shape[1] % 128 == 0 and kernels.available("attention_segment")


def _own_part_mask(pattern: str, C: int, device) -> Optional[torch.Tensor]:
    """The bool mask of a named pattern over the own-chunk keys: ``[C, C]``, for ``read`` ``[C, 2 C]`` (clean own keys first)."""
    name, _, arg = pattern.partition(":")
    if name == "full":
        return None
    return read_mask_matrix(C, int(arg), device) if name == "read" else own_mask_matrix(C, pattern, device)


# ------------------------------------------------------------------ a whole segment of the prefix in one launch
CLEAN_STREAM = 1


class _SegmentAttention(torch.autograd.Function):
    """Every chunk of every stream of one prefix layer's segment: one forward launch, one backward launch (plus the small
    ``delta`` kernel).  The clean stream's keys and values are laid out once as ``[previous window | segment]``; every chunk
    reads its window from that buffer in place, and the backward accumulates the gradient of a clean key over all the windows
    that held it on chip.  First order only (the prefix is never inside the inner step's recorded backward)."""

    @staticmethod
    def forward(ctx, q, k, v, k_prev, v_prev, C, W, first, reach, patterns, scale):
        from . import kernels
        B, S, T = q.shape[:3]
        WC = W * C

        def lay_out(own, prev):
            buf = own.new_empty((B, WC + T) + tuple(own.shape[3:]))
            if WC:
                if prev is None:
                    buf[:, :WC].zero_()
                else:
                    buf[:, :WC].copy_(prev)
            buf[:, WC:].copy_(own[:, CLEAN_STREAM])
            return buf
        kc, vc = lay_out(k, k_prev), lay_out(v, v_prev)
        o, lse = kernels.attention_fwd_segment(q, kc, vc, k, v, C, W, first, reach, patterns, scale)
        ctx.save_for_backward(q, k, v, kc, vc, o, lse)
        ctx.meta = (C, W, first, reach, tuple(patterns), scale, k_prev is not None)
        return o, kc[:, T:].clone(), vc[:, T:].clone()

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, go, g_tail_k, g_tail_v):
        from . import kernels
        q, k, v, kc, vc, o, lse = ctx.saved_tensors
        C, W, first, reach, patterns, scale, has_prev = ctx.meta
        dq, dk, dv, dk_prev, dv_prev = kernels.attention_bwd_segment(go, q, kc, vc, k, v, o, lse, C, W, first, reach, patterns, scale,
                                                                     g_tail_k, g_tail_v)
        return dq, dk, dv, (dk_prev if has_prev else None), (dv_prev if has_prev else None), None, None, None, None, None, None


def segment_attention_ok(q: torch.Tensor, C: int, W: int, patterns) -> bool:
    from . import kernels
    S = q.shape[1]
    return (use_kernels(q) and q.is_cuda and C % 128 == 0 and S >= 2 and S <= 8 and S * (W + 1) * (C // 128) <= 512
            and kernels.attention_segment_supported(q, W, patterns))


def segment_attention(q, k, v, kv_prev, C: int, W: int, first: int, reach, patterns, scale: float):
    """``q [B, S, T, nh, d]``, ``k / v [B, S, T, nkv, d]`` (stream 1 is the clean one), ``kv_prev``: the clean keys / values of the
    ``W`` chunks before the segment (None at the sequence start) -> ``(o [B, S, T, nh, d], k_tail, v_tail [B, W C, nkv, d])``."""
    kp, vp = (None, None) if kv_prev is None else kv_prev
    return _SegmentAttention.apply(q, k, v, kp, vp, C, W, first, reach, tuple(patterns), scale)


# staged execution: library/hand-written forward + first-order backward, reference for the second order
_BIAS = {}
# the recorded backward runs the flash backward kernel with a hand-written derivative (False: differentiate the reference statement)
SECOND_ORDER_KERNEL = True


def _causal_bias(C: int, Kn: int, device) -> torch.Tensor:
    """``[C, Kn]`` f32 additive mask, causal aligned to the end of the key axis."""
    key = (C, Kn, str(device))
    b = _BIAS.get(key)
    if b is None:
        i = torch.arange(C, device=device)[:, None]
        j = torch.arange(Kn, device=device)[None, :]
        b = _BIAS[key] = torch.where(j <= i + (Kn - C), 0.0, ref.NEG).float()
        if len(_BIAS) > 32:
            _BIAS.pop(next(iter(_BIAS)))
    return b


def _ref_for_staged(q, K, V, scale, pattern):
    """The differentiable-to-any-order statement used when a backward is recorded.  On the GPU the two
    products run on the tensor-core GEMM (batched over sequence x KV head, the query heads of a group folded
    into the rows), scores and softmax in f32 as in the reference (attention.py:181-201)."""
    causal = pattern == "causal"
    if not use_kernels(q) or pattern not in ("full", "causal"):
        return ref.attend(q, K, V, None, scale, _own_part_mask(pattern, q.shape[1], q.device))
    from .gemm import mm
    n, C, nh, d = q.shape
    Kn, nkv = K.shape[1], K.shape[2]
    rep = nh // nkv
    qg = q.reshape(n, C, nkv, rep, d).permute(0, 2, 3, 1, 4).reshape(n * nkv, rep * C, d)
    kg = K.permute(0, 2, 1, 3).reshape(n * nkv, Kn, d)
    vg = V.permute(0, 2, 1, 3).reshape(n * nkv, Kn, d)
    s = mm(qg, kg, False, True, out_dtype=torch.float32) * scale
    if causal:
        s = (s.view(n * nkv, rep, C, Kn) + _causal_bias(C, Kn, q.device)).view(n * nkv, rep * C, Kn)
    p = torch.softmax(s, dim=-1).to(q.dtype)
    o = mm(p, vg)
    return o.view(n, nkv, rep, C, d).permute(0, 3, 1, 2, 4).reshape(n, C, nh, d)


def _two_segment_ok(q, kw, k_own) -> bool:
    from . import kernels
    return (q.is_cuda and kernels.available("attention") and kernels.available("attention_bwd") and kernels.attention_bwd_supported(q, kw)
            and kw.shape[1] % 128 == 0 and kernels.ATTN_VARIANT == 0)


def _ref_for_staged2(q, kw, vw, ko, vo, scale, pattern):
    return _ref_for_staged(q, torch.cat([kw, ko], 1), torch.cat([vw, vo], 1), scale, pattern)


def _fast_fwd2(q, kw, vw, ko, vo, scale, pattern):
    from . import kernels
    o, lse = kernels.attention_fwd(q, kw, vw, scale, pattern, k2=ko, v2=vo)
    return o, (o, lse)


def _fast_bwd2(g, tensors, saved, needs, scale, pattern):
    from . import kernels
    q, kw, vw, ko, vo = tensors
    return kernels.attention_bwd(g, q, kw, vw, saved[0], saved[1], scale, pattern, k2=ko, v2=vo)


def _diff_bwd2(g, tensors, saved, needs, scale, pattern):
    """The backward as an operation with a hand-written derivative (``ops.attn_second``), or ``None`` to decline (then the
    statement is differentiated; the hand-written derivative covers the full and causal patterns)."""
    from . import attn_second
    q, kw, vw, ko, vo = tensors
    if (pattern not in ("full", "causal") or not SECOND_ORDER_KERNEL or not saved
            or not attn_second.supported(q, kw.shape[1] + ko.shape[1])):
        return None
    return attn_second.attention_bwd_diff(g, q, kw, vw, ko, vo, saved[0], saved[1], scale, pattern == "causal")


def _diff_bwd(g, tensors, saved, needs, scale, pattern):
    from . import attn_second, kernels
    q, K, V = tensors
    if (pattern not in ("full", "causal") or not SECOND_ORDER_KERNEL or not saved or not kernels.available("attention_bwd")
            or not kernels.attention_bwd_supported(q, K) or not attn_second.supported(q, K.shape[1])):
        return None
    return attn_second.attention_bwd_diff(g, q, K, V, None, None, saved[0], saved[1], scale, pattern == "causal")


def _fast_fwd(q, K, V, scale, pattern):
    from . import kernels
    if kernels.available("attention") and kernels.attention_supported(q, K):
        o, lse = kernels.attention_fwd(q, K, V, scale, pattern)
        return o, (o, lse)
    with torch.no_grad():
        o = _ref_for_staged(q, K, V, scale, pattern)
    return o, ()


def _fast_bwd(g, tensors, saved, needs, scale, pattern):
    from . import kernels
    q, K, V = tensors
    if saved and kernels.available("attention_bwd") and kernels.attention_bwd_supported(q, K):
        return kernels.attention_bwd(g, q, K, V, saved[0], saved[1], scale, pattern)
    # shapes the kernels do not cover (CPU tensors, f32): differentiate the tensor-core statement
    with torch.enable_grad():
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, K, V))
        o = _ref_for_staged(qq, kk, vv, scale, pattern)
        return torch.autograd.grad(o, (qq, kk, vv), g)
