"""Python front ends of the hand-written CUDA kernels other than the GEMM (``ops.gemm``).

``available(name)`` says whether the named kernel family is compiled into the loaded library; the
dispatchers in ``ops.functional`` ask before using one.  Families are added to ``_FAMILIES`` by the
sections below as their symbols are found.
"""
from __future__ import annotations

import collections
import ctypes
from typing import Dict

import torch

from . import _lib

import os

_FAMILIES: Dict[str, bool] = {}
# DTTT_DISABLE_KERNELS=attention,linear_ce,... switches families off (ablations; the op falls back to its staged statement)
_DISABLED = set(x for x in os.environ.get("DTTT_DISABLE_KERNELS", "").split(",") if x)
LAUNCHES = 0


def available(name: str) -> bool:
    from . import gemm as _g
    if name in _DISABLED:
        return False
    if _g.EMULATE and not torch.cuda.is_available():
        return name in _EMULATED
    if not torch.cuda.is_available():
        return False
    ok = _FAMILIES.get(name)
    if ok is None:
        sym = _SYMBOL.get(name)
        ok = bool(sym) and hasattr(_lib.lib(), sym)
        _FAMILIES[name] = ok
    return ok


def disable(name: str) -> None:
    _DISABLED.add(name)


def enable(name: str) -> None:
    _DISABLED.discard(name)


# family -> a symbol whose presence means the family is built
_SYMBOL: Dict[str, str] = {}
# families whose launchers have a PyTorch stand-in for CPU tensors (DTTT_EMULATE=1, see ops.gemm)
_EMULATED = {"rmsnorm", "rope", "swiglu"}

# =============================================================================== elementwise family
import ctypes as _ct

from . import reference as _ref

_vp, _ll, _i, _f = _ct.c_void_p, _ct.c_longlong, _ct.c_int, _ct.c_float
_lib.register("dttt_rmsnorm_fwd", _i, [_vp, _vp, _vp, _vp, _ll, _i, _f, _vp])
_lib.register("dttt_rmsnorm_bwd", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _vp])
_lib.register("dttt_rope", _i, [_vp, _vp, _vp, _vp, _ll, _i, _i, _f, _vp])
_lib.register("dttt_rope_table", _i, [_vp, _vp, _ll, _i, _vp, _vp])
_lib.register("dttt_rope_apply", _i, [_vp, _vp, _vp, _ll, _i, _i, _f, _vp])
_lib.register("dttt_swiglu_fwd", _i, [_vp, _vp, _vp, _ll, _vp])
_lib.register("dttt_swiglu_bwd", _i, [_vp, _vp, _vp, _vp, _vp, _ll, _vp])
_lib.register("dttt_adamw", _i, [_vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _f, _vp])
_lib.register("dttt_seq_sumsq", _i, [_vp, _vp, _i, _ll, _i, _vp])
_lib.register("dttt_seq_axpy", _i, [_vp, _vp, _vp, _vp, _vp, _i, _ll, _i, _vp])
_lib.register("dttt_seq_dot", _i, [_vp, _vp, _vp, _i, _ll, _i, _vp])
_lib.register("dttt_seq_lincomb", _i, [_vp, _vp, _vp, _vp, _vp, _i, _ll, _i, _vp])
_SYMBOL.update(rmsnorm="dttt_rmsnorm_fwd", rope="dttt_rope", swiglu="dttt_swiglu_fwd", adamw="dttt_adamw",
               seq="dttt_seq_sumsq")


def _p(t):
    return _ct.c_void_p(t.data_ptr()) if t is not None else _ct.c_void_p(0)


def _stream():
    return _ct.c_void_p(_lib.stream_ptr())


def _check(rc, what):
    global LAUNCHES
    if rc != 0:
        raise _lib.KernelError(f"{what} launch failed rc={rc}")
    LAUNCHES += 1


# ---- RMSNorm
def _rms_fwd(x, w, eps):
    xc = x.contiguous()
    D = xc.shape[-1]
    rows = xc.numel() // D
    y = torch.empty_like(xc)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    wf = w.detach().float().contiguous()
    if not x.is_cuda:
        x32 = xc.float()
        r = torch.rsqrt(x32.pow(2).mean(-1) + eps)
        return (wf * x32 * r[..., None]).to(x.dtype), (r.reshape(-1),)
    _check(_lib.lib().dttt_rmsnorm_fwd(_p(xc), _p(wf), _p(y), _p(rstd), rows, D, float(eps), _stream()), "rmsnorm_fwd")
    return y, (rstd,)


def _rms_bwd(g, tensors, saved, needs, eps):
    x, w = tensors
    (rstd,) = saved
    xc, gc = x.contiguous(), g.contiguous()
    D = xc.shape[-1]
    rows = xc.numel() // D
    dx = torch.empty_like(xc)
    dw = torch.zeros(D, dtype=torch.float32, device=x.device) if needs[1] else None
    wf = w.detach().float().contiguous()
    if not x.is_cuda:
        x32, g32, r = xc.float().reshape(rows, D), gc.float().reshape(rows, D), rstd[:, None]
        xh = x32 * r
        dxv = r * (wf * g32 - xh * (wf * g32 * xh).mean(-1, keepdim=True))
        return dxv.to(x.dtype).view(x.shape), ((g32 * xh).sum(0).to(w.dtype) if needs[1] else None)
    _check(_lib.lib().dttt_rmsnorm_bwd(_p(xc), _p(wf), _p(gc), _p(rstd), _p(dx), _p(dw), rows, D, _stream()), "rmsnorm_bwd")
    return dx, (dw.to(w.dtype) if dw is not None else None)


# ---- the RMSNorm backward as a differentiable operation (recorded passes)
_lib.register("dttt_rmsnorm_bwd2", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _vp])
_lib.register("dttt_swiglu_bwd2", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _vp])
_SYMBOL.update(elementwise_bwd2="dttt_rmsnorm_bwd2")
SECOND_ORDER_ELEMENTWISE = True


def rms_norm_bwd2(c, e, g, x, w, rstd):
    """Derivative of the RMSNorm backward ``(g, x, w) -> (dx, dw)`` contracted with the cotangents ``c`` (of ``dx``) and ``e``
    (of ``dw``, may be ``None``): ``(grad g, grad x, grad w)``."""
    D = x.shape[-1]
    rows = x.numel() // D
    wf = w.detach().float().contiguous()
    if not x.is_cuda:
        x32, g32, c32, r = x.float().reshape(rows, D), g.float().reshape(rows, D), c.float().reshape(rows, D), rstd.reshape(rows, 1)
        xh, u = x32 * r, wf * g32
        al, be, ga = (c32 * xh).mean(-1, keepdim=True), (u * xh).mean(-1, keepdim=True), (c32 * u).mean(-1, keepdim=True)
        t = r * (c32 - xh * al)
        gg = wf * t
        gx = r * r * ((3 * al * be - ga) * xh - be * c32 - al * u)
        if e is not None:
            v = e.float() * g32
            gg = gg + e.float() * xh
            gx = gx + r * (v - xh * (v * xh).mean(-1, keepdim=True))
        return gg.to(g.dtype).view(g.shape), gx.to(x.dtype).view(x.shape), (g32 * t).sum(0).to(w.dtype)
    xc, gc, cc = x.contiguous(), g.contiguous(), c.contiguous()
    gg, gx = torch.empty_like(gc), torch.empty_like(xc)
    gwt = torch.zeros(D, dtype=torch.float32, device=x.device)
    ef = None if e is None else e.detach().float().contiguous()
    _check(_lib.lib().dttt_rmsnorm_bwd2(_p(xc), _p(wf), _p(gc), _p(rstd), _p(cc), _p(ef), _p(gg), _p(gx), _p(gwt), rows, D, _stream()),
           "rmsnorm_bwd2")
    return gg, gx, gwt.to(w.dtype)


class _RmsBwd(torch.autograd.Function):
    """``(g, x, w, rstd) -> (dx, dw)`` on the backward kernel; differentiable once more by ``rms_norm_bwd2``.  ``rstd`` is a
    cache of the forward, not an independent input."""

    @staticmethod
    def forward(ctx, g, x, w, rstd, eps):
        ctx.save_for_backward(g, x, w, rstd)
        dx, dw = _rms_bwd(g, (x, w), (rstd,), (True, True), eps)
        return dx, dw

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, c, e):
        g, x, w, rstd = ctx.saved_tensors
        if c is None:
            c = torch.zeros_like(x)
        gg, gx, gw = rms_norm_bwd2(c.to(x.dtype), e, g.to(x.dtype), x, w, rstd)
        return gg.to(g.dtype), gx, gw, None, None


def _rms_diff_bwd(g, tensors, saved, needs, eps):
    x, w = tensors
    if not SECOND_ORDER_ELEMENTWISE or x.dtype != torch.bfloat16 or (x.is_cuda and not available("elementwise_bwd2")):
        return None
    return _RmsBwd.apply(g, x, w, saved[0], eps)


_RMS_SPEC = (_rms_fwd, _rms_bwd, _ref.rms_norm, _rms_diff_bwd)


def rms_norm(x, w, eps):
    from .functional import staged
    if x.shape[-1] % 8:
        return _ref.rms_norm(x, w, eps)
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad):
        return staged(_RMS_SPEC, (x, w), (eps,))
    return _rms_fwd(x, w, eps)[0]


# ---- rotary embedding
# (cos, sin) per (row, frequency) of the positions last seen: one table serves q and k, every head and layer of a chunk and
# the backward (DTTT_ROPE_TABLE=0: every call computes its angles itself).  An entry keeps its position tensor alive, so a
# recycled address cannot pass for it, and the version counter catches in-place edits.
ROPE_TABLE = os.environ.get("DTTT_ROPE_TABLE", "1") == "1"
_ROPE_TABLES: "collections.OrderedDict" = collections.OrderedDict()
_ROPE_TABLES_MAX = 8


def _rope_table(pc, inv_freq, rows, d):
    try:
        key = (pc.data_ptr(), pc.numel(), pc._version, inv_freq.data_ptr(), inv_freq._version, d, _lib.stream_ptr())
    except RuntimeError:                               # inference tensors keep no version counter: nothing to key a cache on
        key = None
    hit = _ROPE_TABLES.get(key) if key is not None else None
    if hit is not None:
        _ROPE_TABLES.move_to_end(key)
        return hit[2]
    tab = torch.empty(rows, d // 2, 2, dtype=torch.float32, device=pc.device)
    _check(_lib.lib().dttt_rope_table(_p(pc), _p(inv_freq), rows, d, _p(tab), _stream()), "rope_table")
    if key is None:
        return tab
    _ROPE_TABLES[key] = (pc, inv_freq, tab)
    while len(_ROPE_TABLES) > _ROPE_TABLES_MAX:
        _ROPE_TABLES.popitem(last=False)
    return tab


def _rope_run(x, pos, inv_freq, sign):
    xc = x.contiguous()
    heads, d = xc.shape[-2], xc.shape[-1]
    rows = xc.numel() // (heads * d)
    out = torch.empty_like(xc)
    pc = pos.contiguous()
    assert pc.numel() == rows and pc.dtype == torch.int64, (pc.shape, rows, pc.dtype)
    if not x.is_cuda:
        ang = pc.float().unsqueeze(-1) * inv_freq
        emb = torch.cat([ang, ang], dim=-1)
        return _ref.apply_rope(xc, emb.cos(), sign * emb.sin())
    if ROPE_TABLE and inv_freq.dtype == torch.float32 and inv_freq.is_contiguous() and inv_freq.numel() == d // 2:
        tab = _rope_table(pc, inv_freq, rows, d)
        _check(_lib.lib().dttt_rope_apply(_p(xc), _p(out), _p(tab), rows, heads, d, float(sign), _stream()), "rope_apply")
        return out
    _check(_lib.lib().dttt_rope(_p(xc), _p(out), _p(pc), _p(inv_freq), rows, heads, d, float(sign), _stream()), "rope")
    return out


def _rope_ref(x, pos, inv_freq):
    ang = pos.float().unsqueeze(-1) * inv_freq
    emb = torch.cat([ang, ang], dim=-1)
    return _ref.apply_rope(x, emb.cos(), emb.sin())


class _Rope(torch.autograd.Function):
    """The rotation is linear in ``x`` and its transpose is the rotation by the opposite angle, so the backward is the same
    operation with the sign flipped: differentiable to any order on the kernel."""

    @staticmethod
    def forward(ctx, x, pos, inv_freq, sign):
        ctx.pos, ctx.inv, ctx.sign = pos, inv_freq, sign
        return _rope_run(x, pos, inv_freq, sign)

    @staticmethod
    def backward(ctx, g):
        if torch.is_grad_enabled():
            return _Rope.apply(g, ctx.pos, ctx.inv, -ctx.sign), None, None, None
        return _rope_run(g, ctx.pos, ctx.inv, -ctx.sign), None, None, None


def rope(x, pos, inv_freq):
    """``x [..., T, heads, d]`` rotated by the angles ``pos [..., T] * inv_freq [d/2]``."""
    from .functional import staged
    if x.shape[-1] % 16:
        return _rope_ref(x, pos, inv_freq)
    if torch.is_grad_enabled() and x.requires_grad:
        return _Rope.apply(x, pos, inv_freq, 1.0)
    return _rope_run(x, pos, inv_freq, 1.0)


# ---- SwiGLU
def _swiglu_fwd(g, u):
    gc, uc = g.contiguous(), u.contiguous()
    if not g.is_cuda:
        return _ref.glu(gc.float(), uc.float()).to(g.dtype), ()
    y = torch.empty_like(gc)
    _check(_lib.lib().dttt_swiglu_fwd(_p(gc), _p(uc), _p(y), gc.numel(), _stream()), "swiglu_fwd")
    return y, ()


def _swiglu_bwd(dy, tensors, saved, needs):
    g, u = tensors
    gc, uc, dc = g.contiguous(), u.contiguous(), dy.contiguous()
    if not g.is_cuda:
        sg = torch.sigmoid(gc.float())
        silu = gc.float() * sg
        return (dc.float() * uc.float() * (sg + silu * (1 - sg))).to(g.dtype), (dc.float() * silu).to(u.dtype)
    dg, du = torch.empty_like(gc), torch.empty_like(uc)
    _check(_lib.lib().dttt_swiglu_bwd(_p(gc), _p(uc), _p(dc), _p(dg), _p(du), gc.numel(), _stream()), "swiglu_bwd")
    return dg, du


def swiglu_bwd2(cg, cu, dy, g, u):
    """Derivative of the SwiGLU backward ``(dy, g, u) -> (dg, du)`` contracted with ``(cg, cu)``: ``(grad dy, grad g, grad u)``."""
    if not g.is_cuda:
        g32, u32, d32, a, b = g.float(), u.float(), dy.float(), cg.float(), cu.float()
        s = torch.sigmoid(g32)
        silu = g32 * s
        s1 = s * (1 + g32 * (1 - s))
        s2 = s * (1 - s) * (2 + g32 * (1 - 2 * s))
        return ((a * u32 * s1 + b * silu).to(dy.dtype), (d32 * (a * u32 * s2 + b * s1)).to(g.dtype), (a * d32 * s1).to(u.dtype))
    gc, uc, dc, ac, bc = (t.contiguous() for t in (g, u, dy, cg, cu))
    og, ou, od = torch.empty_like(gc), torch.empty_like(uc), torch.empty_like(dc)
    _check(_lib.lib().dttt_swiglu_bwd2(_p(gc), _p(uc), _p(dc), _p(ac), _p(bc), _p(og), _p(ou), _p(od), gc.numel(), _stream()), "swiglu_bwd2")
    return od, og, ou


class _SwigluBwd(torch.autograd.Function):
    """``(dy, g, u) -> (dg, du)`` on the backward kernel; differentiable once more by ``swiglu_bwd2``."""

    @staticmethod
    def forward(ctx, dy, g, u):
        ctx.save_for_backward(dy, g, u)
        return _swiglu_bwd(dy, (g, u), (), (True, True))

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, cg, cu):
        dy, g, u = ctx.saved_tensors
        cg = torch.zeros_like(g) if cg is None else cg.to(g.dtype)
        cu = torch.zeros_like(u) if cu is None else cu.to(u.dtype)
        return swiglu_bwd2(cg, cu, dy.to(g.dtype), g, u)


def _swiglu_diff_bwd(dy, tensors, saved, needs):
    g, u = tensors
    if (not SECOND_ORDER_ELEMENTWISE or g.dtype != torch.bfloat16 or u.dtype != torch.bfloat16 or dy.dtype != torch.bfloat16
            or (g.is_cuda and not available("elementwise_bwd2"))):
        return None
    return _SwigluBwd.apply(dy, g, u)


_SWIGLU_SPEC = (_swiglu_fwd, _swiglu_bwd, lambda g, u: _ref.glu(g, u, "silu"), _swiglu_diff_bwd)


def swiglu(g, u):
    from .functional import staged
    if g.numel() % 8:
        return _ref.glu(g, u, "silu")
    if torch.is_grad_enabled() and (g.requires_grad or u.requires_grad):
        return staged(_SWIGLU_SPEC, (g, u), ())
    return _swiglu_fwd(g, u)[0]


# ---- AdamW on a flat f32 range (in place)
def adamw(p, m, v, g, lr, b1, b2, eps, wd, bc1, bc2, gscale):
    _check(_lib.lib().dttt_adamw(_p(p), _p(m), _p(v), _p(g), p.numel(), float(lr), float(b1), float(b2), float(eps), float(wd),
                                 float(bc1), float(bc2), float(gscale), _stream()), "adamw")


# ---- per-sequence pieces of the inner step
def seq_sumsq(ts):
    """``[B]`` f32: sum over a list of ``[B, ...]`` tensors (f32 or bf16) of the squared entries per sequence."""
    B = ts[0].shape[0]
    out = torch.zeros(B, dtype=torch.float32, device=ts[0].device)
    for t in ts:
        tc = t.contiguous()
        _check(_lib.lib().dttt_seq_sumsq(_p(tc), _p(out), B, tc.numel() // B, 1 if tc.dtype == torch.bfloat16 else 0, _stream()),
               "seq_sumsq")
    return out


def seq_axpy(w, g, coef, want_lo=False):
    """``w - coef[b] * g`` per sequence: ``w [B, ...]`` f32, ``g`` f32 or bf16, ``coef [B]`` f32.  Returns the f32
    result and, with ``want_lo``, its bf16 copy produced in the same pass."""
    B = w.shape[0]
    wc, gc = w.contiguous(), g.contiguous()
    out = torch.empty_like(wc)
    lo = torch.empty(wc.shape, dtype=torch.bfloat16, device=w.device) if want_lo else None
    _check(_lib.lib().dttt_seq_axpy(_p(wc), _p(gc), _p(coef.float().contiguous()), _p(out), _p(lo), B, wc.numel() // B,
                                    1 if gc.dtype == torch.bfloat16 else 0, _stream()), "seq_axpy")
    return (out, lo) if want_lo else out


def seq_dot(a_list, g_list):
    """``[B]`` f32: sum over the pairs of ``sum(a * g)`` per sequence (``a`` f32, ``g`` f32 or bf16, ``[B, ...]`` each)."""
    B = a_list[0].shape[0]
    out = torch.zeros(B, dtype=torch.float32, device=a_list[0].device)
    for a, g in zip(a_list, g_list):
        ac, gc = a.contiguous(), g.contiguous()
        _check(_lib.lib().dttt_seq_dot(_p(ac), _p(gc), _p(out), B, ac.numel() // B, 1 if gc.dtype == torch.bfloat16 else 0, _stream()),
               "seq_dot")
    return out


def seq_lincomb(a, g, alpha, beta):
    """``alpha[b] * a + beta[b] * g`` per sequence in ``g``'s dtype (``a`` f32)."""
    B = a.shape[0]
    ac, gc = a.contiguous(), g.contiguous()
    out = torch.empty_like(gc)
    _check(_lib.lib().dttt_seq_lincomb(_p(ac), _p(gc), _p(alpha.float().contiguous()), _p(beta.float().contiguous()), _p(out), B,
                                       ac.numel() // B, 1 if gc.dtype == torch.bfloat16 else 0, _stream()), "seq_lincomb")
    return out


# =============================================================================== attention family
_lib.register("dttt_attn_fwd", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _f, _i, _i, _vp, _vp])
ATTN_VARIANT = int(os.environ.get("DTTT_ATTN_VARIANT", "0"))
_SYMBOL.update(attention="dttt_attn_fwd")


def _kv_rows(t):
    """A K / V tensor ``[n, rows, heads, d]`` usable without a copy: rows, heads and d contiguous, any stride between
    sequences (a slice of a longer window), 16-byte aligned."""
    n, rows, heads, d = t.shape
    if t.stride(3) != 1 or t.stride(2) != d or t.stride(1) != heads * d or t.data_ptr() % 16 or (n > 1 and t.stride(0) % 8):
        t = t.contiguous()
    return t, (t.stride(0) if n > 1 else rows * heads * d)


MASK_MODES = {"full": 0, "causal": 1, "split": 2, "block": 3, "read": 4}
_lib.register("dttt_attn_fwd_masked", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _ll, _f, _i, _i, _vp, _vp])
_lib.register("dttt_attn_fwd_segment", _i, [_vp] * 7 + [_i] * 10 + [_ll, _ll, _vp, _vp, _f, _vp, _vp])


def parse_pattern(own) -> tuple:
    """``"full" | "causal" | "split:K" | "block:b" | "read:b"`` (or a ``causal`` bool) -> ``(mode, param)`` of the kernels."""
    if isinstance(own, bool):
        return (1, 0) if own else (0, 0)
    if isinstance(own, tuple):
        return own
    name, _, arg = own.partition(":")
    return MASK_MODES[name], int(arg) if arg else 0


def attention_fwd(q, k, v, scale, causal, variant=None, k2=None, v2=None):
    """Flash attention forward on the tcgen05 kernel.  ``q [n, Cq, nh, d]``, ``k / v [n, Kn, nkv, d]`` bf16, every key
    valid.  ``causal``: a bool (causal aligned to the end of the key axis) or an own-chunk pattern ``"full" | "causal" |
    "split:K" | "block:b" | "read:b"`` over the last ``Cq`` keys (``read``: over the last ``2 Cq``, clean own keys first).
    ``k2 / v2 [n, Kn2, nkv, d]``: more keys AFTER ``k / v`` (the chunk's own keys after the window's), read from their own tensors
    instead of a concatenation (``Kn`` a multiple of 128).  Returns ``o`` like ``q`` and ``lse [n, nh, Cq]`` (f32)."""
    n, Cq, nh, d = q.shape
    Kn, nkv = k.shape[1], k.shape[2]
    assert q.dtype == torch.bfloat16 and d in (64, 128), (q.dtype, d)
    mode, param = parse_pattern(causal)
    var = ATTN_VARIANT if variant is None else int(variant)
    if k2 is not None and (Kn % 128 or var != 0 or Kn == 0):
        k, v, k2, v2 = torch.cat([k, k2], 1), torch.cat([v, v2], 1), None, None
        Kn = k.shape[1]
    qc = q.contiguous()
    (kc, kbs), (vc, vbs) = _kv_rows(k), _kv_rows(v)
    (k2c, k2bs), (v2c, v2bs) = (_kv_rows(k2), _kv_rows(v2)) if k2 is not None else ((None, 0), (None, 0))
    o = torch.empty_like(qc)
    lse = torch.empty(n, nh, Cq, dtype=torch.float32, device=q.device)
    st = _lib.status_tensor(q.device)
    if mode >= 2:
        _check(_lib.lib().dttt_attn_fwd_masked(_p(qc), _p(kc), _p(vc), _p(k2c), _p(v2c), _p(o), _p(lse), n, Cq, Kn, 0 if k2 is None else k2.shape[1],
                                               nh, nkv, d, kbs, vbs, k2bs, v2bs, float(scale), mode, param, _p(st), _stream()), "attn_fwd_masked")
        return o, lse
    _check(_lib.lib().dttt_attn_fwd(_p(qc), _p(kc), _p(vc), _p(k2c), _p(v2c), _p(o), _p(lse), n, Cq, Kn, 0 if k2 is None else k2.shape[1],
                                    nh, nkv, d, kbs, vbs, k2bs, v2bs, float(scale), mode, var, _p(st), _stream()), "attn_fwd")
    return o, lse


def _int_array(vals):
    return (ctypes.c_int * len(vals))(*[int(x) for x in vals])


def attention_segment_supported(q, W: int, patterns) -> bool:
    """``q [B, S, T, nh, d]``: the one-launch segment form covers head dimensions 64 and 128, chunks that are multiples of 128 tokens,
    every pattern but the sub-block read, and work lists of at most 512 (stream, chunk, tile) entries per key block."""
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and available("attention_segment")
            and all(parse_pattern(p)[0] < 4 for p in patterns))


def attention_fwd_segment(q, kc, vc, ko, vo, C: int, W: int, first: int, reach, patterns, scale: float):
    """Every chunk of every stream of a segment in one launch.  ``q [B, S, T, nh, d]``; ``kc / vc [B, (W + T / C) C, nkv, d]``: the
    clean stream's keys / values with the previous segment's window in front; ``ko / vo [B, S, T, nkv, d]``: every stream's own
    keys / values.  Returns ``o`` like ``q`` and ``lse [B * S * T / C, nh, C]``."""
    B, S, T, nh, d = q.shape
    nkv = kc.shape[2]
    chunks = T // C
    qc, koc, voc = q.contiguous(), ko.contiguous(), vo.contiguous()
    (kcc, kbs), (vcc, vbs) = _kv_rows(kc), _kv_rows(vc)
    o = torch.empty_like(qc)
    lse = torch.empty(B * S * chunks, nh, C, dtype=torch.float32, device=q.device)
    modes, params = zip(*[parse_pattern(p) for p in patterns])
    st = _lib.status_tensor(q.device)
    _check(_lib.lib().dttt_attn_fwd_segment(_p(qc), _p(kcc), _p(vcc), _p(koc), _p(voc), _p(o), _p(lse), B, S, chunks, C, W, int(first),
                                            -1 if reach is None else int(reach), nh, nkv, d, kbs, vbs, _int_array(modes), _int_array(params),
                                            float(scale), _p(st), _stream()), "attn_fwd_segment")
    return o, lse


def attention_supported(q, k) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and (q.shape[2] % k.shape[2] == 0)


# =============================================================================== linear + cross-entropy family
_lib.register("dttt_linear_ce_scratch_elems", _ll, [_i, _i])
_lib.register("dttt_linear_ce_fwd", _i, [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _vp])
_lib.register("dttt_linear_ce_dlogits", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp])
_SYMBOL.update(linear_ce="dttt_linear_ce_fwd")


def _rows_bf16(t):
    """A 2-D bf16 view whose row stride and base are 16-byte aligned (copying only when they are not)."""
    if t.stride(-1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t


def linear_ce_supported(h, E) -> bool:
    return h.is_cuda and h.dtype == torch.bfloat16 and E.dtype == torch.bfloat16 and h.shape[-1] % 8 == 0


def linear_ce_fwd(h, E, targets):
    """``(lse [N], nll [N])`` (f32) of the logits ``h @ E^T`` without writing them: the GEMM's epilogue reduces every
    128 x 256 logit tile to a (max, sum-exp) pair in a scratch buffer and a second small kernel combines the pairs."""
    N, K = h.shape
    V = E.shape[0]
    hc, Ec = _rows_bf16(h), _rows_bf16(E)
    ti = targets.to(torch.int32).contiguous()
    scratch = torch.empty(int(_lib.lib().dttt_linear_ce_scratch_elems(N, V)), 2, dtype=torch.float32, device=h.device)
    tgt = torch.zeros(N, dtype=torch.float32, device=h.device)
    lse = torch.empty(N, dtype=torch.float32, device=h.device)
    nll = torch.empty(N, dtype=torch.float32, device=h.device)
    st = _lib.status_tensor(h.device)
    _check(_lib.lib().dttt_linear_ce_fwd(_p(hc), _p(Ec), _p(ti), N, V, K, hc.stride(0), Ec.stride(0), _p(scratch), _p(tgt), _p(lse),
                                         _p(nll), _p(st), _stream()), "linear_ce_fwd")
    global LAUNCHES
    LAUNCHES += 1                                   # the combine kernel
    return lse, nll


def linear_ce_dlogits(h, Eb, targets_i32, coef, lse, col0):
    """``coef[:, None] * (softmax(h @ E^T)[:, col0:col0 + len(Eb)] - onehot(targets))`` in bf16, from the GEMM's epilogue."""
    N, K = h.shape
    nb = Eb.shape[0]
    hc, Ec = _rows_bf16(h), _rows_bf16(Eb)
    D = torch.empty(N, nb, dtype=torch.bfloat16, device=h.device)
    st = _lib.status_tensor(h.device)
    _check(_lib.lib().dttt_linear_ce_dlogits(_p(hc), _p(Ec), _p(targets_i32), _p(coef), _p(lse), _p(D), N, nb, K, hc.stride(0),
                                             Ec.stride(0), D.stride(0), int(col0), _p(st), _stream()), "linear_ce_dlogits")
    return D


_lib.register("dttt_attn_bwd", _i, [_vp] * 14 + [_i] * 7 + [_ll] * 4 + [_f, _i, _vp, _vp])
_lib.register("dttt_attn_bwd_masked", _i, [_vp] * 14 + [_i] * 7 + [_ll] * 4 + [_f, _i, _i, _vp, _vp])
_lib.register("dttt_attn_bwd_segment", _i, [_vp] * 14 + [_i] * 10 + [_ll, _ll, _vp, _vp, _f, _vp, _vp])
_SYMBOL.update(attention_bwd="dttt_attn_bwd", attention_segment="dttt_attn_bwd_segment")


def attention_bwd_supported(q, k) -> bool:
    """Head dimensions 64 (``csrc/attn_bwd_tcgen05.cu``) and 128 (``csrc/attn_bwd128_tcgen05.cu``)."""
    return attention_supported(q, k)


def attention_bwd(g, q, k, v, o, lse, scale, causal, k2=None, v2=None):
    """First-order backward of ``attention_fwd`` on the tcgen05 kernel: ``(dq, dk, dv)`` or, with a second key / value pair,
    ``(dq, dk, dv, dk2, dv2)``.  ``causal``: a bool or an own-chunk pattern as in ``attention_fwd``.  ``dq`` is accumulated in
    f32 by the kernel (one bulk reduction per key block and query tile) and cast once at the end."""
    n, Cq, nh, d = q.shape
    Kn, nkv = k.shape[1], k.shape[2]
    mode, param = parse_pattern(causal)
    two = k2 is not None and Kn % 128 == 0 and Kn > 0
    if k2 is not None and not two:
        dq, dk, dv = attention_bwd(g, q, torch.cat([k, k2], 1), torch.cat([v, v2], 1), o, lse, scale, (mode, param))
        return dq, dk[:, :Kn], dv[:, :Kn], dk[:, Kn:], dv[:, Kn:]
    qc, oc, gc = q.contiguous(), o.contiguous(), g.contiguous()
    (kc, kbs), (vc, vbs) = _kv_rows(k), _kv_rows(v)
    (k2c, k2bs), (v2c, v2bs) = (_kv_rows(k2), _kv_rows(v2)) if two else ((None, 0), (None, 0))
    dq32 = torch.zeros(n, Cq, nh, d, dtype=torch.float32, device=q.device)
    delta = torch.empty(n, nh, Cq, dtype=torch.float32, device=q.device)
    mk = lambda t: torch.empty(t.shape, dtype=t.dtype, device=t.device)
    dk, dv = mk(k), mk(v)
    dk2, dv2 = (mk(k2), mk(v2)) if two else (None, None)
    st = _lib.status_tensor(q.device)
    _check(_lib.lib().dttt_attn_bwd_masked(_p(qc), _p(kc), _p(vc), _p(k2c), _p(v2c), _p(oc), _p(gc), _p(lse), _p(delta), _p(dq32), _p(dk), _p(dv),
                                           _p(dk2), _p(dv2), n, Cq, Kn, k2.shape[1] if two else 0, nh, nkv, d, kbs, vbs, k2bs, v2bs, float(scale),
                                           mode, param, _p(st), _stream()), "attn_bwd")
    global LAUNCHES
    LAUNCHES += 1                                   # the delta kernel
    dq = dq32.to(q.dtype)
    return (dq, dk, dv, dk2, dv2) if two else (dq, dk, dv)


def attention_bwd_segment(g, q, kc, vc, ko, vo, o, lse, C: int, W: int, first: int, reach, patterns, scale: float,
                          g_tail_k=None, g_tail_v=None):
    """Backward of ``attention_fwd_segment``: ``(dq [B, S, T, nh, d], dk, dv [B, S, T, nkv, d], dk_prev, dv_prev [B, W C, nkv, d])``.
    The clean stream's ``dk / dv`` (stream 1) hold the gradient of its keys from every window that held them and from its own
    chunks, summed on chip; ``dk_prev / dv_prev`` is the part that falls on the previous segment's window."""
    B, S, T, nh, d = q.shape
    nkv = kc.shape[2]
    chunks = T // C
    qc, oc, gc, koc, voc = q.contiguous(), o.contiguous(), g.contiguous(), ko.contiguous(), vo.contiguous()
    (kcc, kbs), (vcc, vbs) = _kv_rows(kc), _kv_rows(vc)
    dq32 = torch.zeros(B, S, T, nh, d, dtype=torch.float32, device=q.device)
    delta = torch.empty(B * S * chunks, nh, C, dtype=torch.float32, device=q.device)
    dkc = torch.empty(B, (W + chunks) * C, nkv, d, dtype=q.dtype, device=q.device)
    dvc = torch.empty_like(dkc)
    dko = torch.empty(B, S, T, nkv, d, dtype=q.dtype, device=q.device)
    dvo = torch.empty_like(dko)
    modes, params = zip(*[parse_pattern(p) for p in patterns])
    st = _lib.status_tensor(q.device)
    _check(_lib.lib().dttt_attn_bwd_segment(_p(qc), _p(kcc), _p(vcc), _p(koc), _p(voc), _p(oc), _p(gc), _p(lse), _p(delta), _p(dq32), _p(dkc), _p(dvc),
                                            _p(dko), _p(dvo), B, S, chunks, C, W, int(first), -1 if reach is None else int(reach), nh, nkv, d,
                                            kbs, vbs, _int_array(modes), _int_array(params), float(scale), _p(st), _stream()), "attn_bwd_segment")
    global LAUNCHES
    LAUNCHES += 1
    if g_tail_k is not None:                        # what the next segment's windows sent back to this buffer's last W chunks
        dkc[:, T:].add_(g_tail_k)
        dvc[:, T:].add_(g_tail_v)
    # the clean stream (index 1) has its own keys inside the clean buffer: move that part of the gradient to its slot
    dko[:, 1].copy_(dkc[:, W * C:])
    dvo[:, 1].copy_(dvc[:, W * C:])
    return dq32.to(q.dtype), dko, dvo, dkc[:, :W * C], dvc[:, :W * C]


# =============================================================================== second-order attention (row stage)
_lib.register("dttt_attn_bwd2_rows", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _f, _vp])
_SYMBOL.update(attention_bwd2="dttt_attn_bwd2_rows")
ATTN_BWD2_MAX_KEYS = 10240


def attention_bwd2_rows(S, dP, gdS, X, lse, delta, chunk, causal, scale):
    """Row stage of the derivative of the attention backward: f32 ``S, dP, gdS, X [rows, Kn]`` (unscaled scores, ``dO V^T``,
    unscaled ``gQ K^T + Q gK^T``, ``dO gV^T``) and ``lse, delta [rows]`` -> bf16 ``P, scale dS, gdP, scale gS [rows, Kn]``.
    Row ``r`` is query position ``r % chunk`` of its chunk."""
    Kn = S.shape[-1]
    rows = S.numel() // Kn
    outs = [torch.empty(S.shape, dtype=torch.bfloat16, device=S.device) for _ in range(4)]
    for t in (S, dP, gdS, X, lse, delta):
        assert t.is_contiguous() and t.dtype == torch.float32
    _check(_lib.lib().dttt_attn_bwd2_rows(_p(S), _p(dP), _p(gdS), _p(X), _p(lse), _p(delta), *[_p(t) for t in outs], rows, Kn, int(chunk),
                                          1 if causal else 0, float(scale), _stream()), "attn_bwd2_rows")
    return outs


_lib.register("dttt_attn_bwd2_scores", _i, [_vp] * 13 + [_i, _i, _i, _i, _i, _f, _i, _vp, _vp])
_SYMBOL.update(attention_bwd2_scores="dttt_attn_bwd2_scores")


def attention_bwd2_scores_supported(q, K) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 64 and q.shape[1] % 128 == 0 and K.shape[1] % 64 == 0
            and q.shape[2] % K.shape[2] == 0)


def attention_bwd2_scores(q, dO, gQ, K, V, gK, gV, lse, delta, scale, causal):
    """Score stage of the derivative of the attention backward on the tcgen05 kernel (``csrc/attn_bwd2_tcgen05.cu``):
    ``q, dO, gQ [n, C, nh, 64]``, ``K, V, gK, gV [n, Kn, nkv, 64]`` bf16, ``lse, delta [n, nh, C]`` f32 ->
    bf16 ``P, scale dS, gdP, scale gS`` as ``[n * nkv, G * C, Kn]`` (head ``h = kv * G + g``, row ``g * C + c``)."""
    n, C, nh, d = q.shape
    Kn, nkv = K.shape[1], K.shape[2]
    ins = [t.contiguous() for t in (q, dO, gQ, K, V, gK, gV)]
    lse, delta = lse.contiguous(), delta.contiguous()
    assert lse.dtype == torch.float32 and delta.dtype == torch.float32 and all(t.dtype == torch.bfloat16 for t in ins)
    outs = [torch.empty(n * nkv, (nh // nkv) * C, Kn, dtype=torch.bfloat16, device=q.device) for _ in range(4)]
    st = _lib.status_tensor(q.device)
    _check(_lib.lib().dttt_attn_bwd2_scores(*[_p(t) for t in ins], _p(lse), _p(delta), *[_p(t) for t in outs], n, C, Kn, nh, nkv,
                                            float(scale), 1 if causal else 0, _p(st), _stream()), "attn_bwd2_scores")
    return outs


# =============================================================================== second-order linear + cross-entropy (row kernels)
_lib.register("dttt_ce_bwd2_rowdot", _i, [_vp, _vp, _vp, _vp, _ll, _i, _ll, _vp])
_lib.register("dttt_ce_bwd2_make", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _ll, _vp])
_SYMBOL.update(linear_ce_bwd2="dttt_ce_bwd2_rowdot")


def ce_bwd2_rowdot(z, u, lse):
    """``ubar[i] = sum_v exp(z[i, v] - lse[i]) u[i, v]`` for f32 ``z, u [N, W]`` (``W`` a multiple of 4)."""
    N, W = z.shape
    assert z.dtype == torch.float32 and u.dtype == torch.float32 and z.stride() == u.stride() and z.stride(1) == 1
    out = torch.empty(N, dtype=torch.float32, device=z.device)
    _check(_lib.lib().dttt_ce_bwd2_rowdot(_p(z), _p(u), _p(lse.contiguous()), _p(out), N, W, z.stride(0), _stream()), "ce_bwd2_rowdot")
    return out


def ce_bwd2_make(z, u, lse, ubar, gw, targets):
    """``r = gw p (u - ubar)``, ``d = gw (p - onehot(targets))`` with ``p = exp(z - lse)``: bf16 ``[N, W]`` each."""
    N, W = z.shape
    r = torch.empty(N, W, dtype=torch.bfloat16, device=z.device)
    d = torch.empty(N, W, dtype=torch.bfloat16, device=z.device)
    assert z.is_contiguous() and u.is_contiguous()
    _check(_lib.lib().dttt_ce_bwd2_make(_p(z), _p(u), _p(lse.contiguous()), _p(ubar), _p(gw.contiguous()), _p(targets.to(torch.int32).contiguous()),
                                        _p(r), _p(d), N, W, W, _stream()), "ce_bwd2_make")
    return r, d


# =============================================================================== embedding / objective family
_lib.register("dttt_embed_gather", _i, [_vp, _vp, _vp, _ll, _i, _vp])
_lib.register("dttt_embed_scatter_f32", _i, [_vp, _vp, _vp, _ll, _i, _vp])
_lib.register("dttt_cart_band", _i, [_vp, _vp, _vp, _i, _i, _i, _vp])
_lib.register("dttt_threefry_uniform", _i, [_vp, _i, _ll, _vp, _vp, _vp, _vp])
_SYMBOL.update(embed="dttt_embed_gather", cart="dttt_cart_band", mask_rng="dttt_threefry_uniform")


def embed_gather(table, ids):
    """Rows ``ids`` of the bf16 ``table [V, H]`` -> ``[*ids.shape, H]``."""
    idc = ids.reshape(-1).long().contiguous()
    H = table.shape[1]
    out = torch.empty(idc.numel(), H, dtype=torch.bfloat16, device=table.device)
    _check(_lib.lib().dttt_embed_gather(_p(table.contiguous()), _p(idc), _p(out), idc.numel(), H, _stream()), "embed_gather")
    return out.view(*ids.shape, H)


def embed_scatter_f32(dh, ids, grad_table):
    """``grad_table[ids[i]] += dh[i]`` in f32 (``dh`` bf16 ``[n, H]`` rows, ``grad_table`` f32 ``[V, H]`` contiguous)."""
    idc = ids.reshape(-1).long().contiguous()
    d2 = dh.reshape(-1, dh.shape[-1]).contiguous()
    _check(_lib.lib().dttt_embed_scatter_f32(_p(d2), _p(idc), _p(grad_table), idc.numel(), d2.shape[1], _stream()), "embed_scatter")


def cart_band(visible, kernel):
    """``out[b, t] = sum_d kernel[d + W] visible[b, t + d]`` (zero padded); ``visible [B, T]``, ``kernel [2 W + 1]``."""
    x = visible.float().contiguous()
    k = kernel.float().contiguous()
    W = (k.numel() - 1) // 2
    if (4 * W + 257) * 4 > 48 * 1024:
        from . import reference as _r
        return _r.band_correlate(visible, kernel)
    out = torch.empty_like(x)
    _check(_lib.lib().dttt_cart_band(_p(x), _p(k), _p(out), x.shape[0], x.shape[1], W, _stream()), "cart_band")
    return out


def threefry_uniform(keys, n, thresh=None):
    """``keys [R, 2]`` (int64 halves) -> uniforms ``[R, n]`` f32 in [0, 1) identical to ``utils.rng.uniform``; with
    ``thresh [R]`` returns the boolean mask ``u < thresh`` instead (one pass, no float tensor)."""
    kc = keys.reshape(-1, 2).long().contiguous()
    R = kc.shape[0]
    if thresh is None:
        u = torch.empty(R, n, dtype=torch.float32, device=keys.device)
        _check(_lib.lib().dttt_threefry_uniform(_p(kc), R, n, _p(u), _p(None), _p(None), _stream()), "threefry_uniform")
        return u
    m = torch.empty(R, n, dtype=torch.uint8, device=keys.device)
    _check(_lib.lib().dttt_threefry_uniform(_p(kc), R, n, _p(None), _p(thresh.float().contiguous()), _p(m), _stream()), "threefry_mask")
    return m.bool()


# =============================================================================== gated delta rule
# ---- the blocked (WY) form: forward with optional block-state checkpoints, and the backward
_lib.register("dttt_gdn_chunk_state_elems", _ll, [_i, _i, _i, _i])
_lib.register("dttt_gdn_chunk_fwd", _i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp])
_lib.register("dttt_gdn_chunk_bwd", _i, [_vp] * 11 + [_i, _i, _i, _i, _vp])
_SYMBOL.update(gdn_chunk="dttt_gdn_chunk_bwd")
GDN_SLICE_ROWS = 32


def gdn_chunk_supported(k, v, block: int) -> bool:
    return (k.is_cuda and block == 64 and k.shape[1] % 64 == 0 and k.shape[-1] in (64, 128) and v.shape[-1] == k.shape[-1]
            and available("gdn_chunk"))


def _f32c(t):
    return t if (t.dtype == torch.float32 and t.is_contiguous()) else t.float().contiguous()


def gdn_chunk_fwd(k, v, beta, log_alpha, S0, states=None):
    """State after one chunk of the gated delta rule in the blocked form (f32): ``k / v [B, C, nh, D]``, ``beta / log_alpha
    [B, C, nh]``, ``S0 [B, nh, D, D]``.  ``states`` (``[B, nh, C / 64, D, D]`` f32): also record the state at every block start."""
    B, C, nh, D = k.shape
    k, v, beta, log_alpha, S0 = (_f32c(t) for t in (k, v, beta, log_alpha, S0))
    out = torch.empty(B, nh, D, D, dtype=torch.float32, device=k.device)
    _check(_lib.lib().dttt_gdn_chunk_fwd(_p(k), _p(v), _p(beta), _p(log_alpha), _p(S0), _p(out), _p(states), B, C, nh, D, _stream()),
           "gdn_chunk_fwd")
    return out


def gdn_chunk_bwd(k, v, beta, log_alpha, S0, gS):
    """Gradients of ``gdn_chunk_fwd`` w.r.t. ``(k, v, beta, log_alpha, S0)`` given ``gS = dL / dS_out``.  One forward sweep
    re-creates the block states, one reverse sweep produces the gradients; what the value-row slices of a head share is summed
    here over the slices."""
    B, C, nh, D = k.shape
    k, v, beta, log_alpha, S0, gS = (_f32c(t) for t in (k, v, beta, log_alpha, S0, gS))
    dev = k.device
    states = torch.empty(B, nh, C // 64, D, D, dtype=torch.float32, device=dev)
    _check(_lib.lib().dttt_gdn_chunk_fwd(_p(k), _p(v), _p(beta), _p(log_alpha), _p(S0), _p(None), _p(states), B, C, nh, D, _stream()),
           "gdn_chunk_fwd(states)")
    ns = D // GDN_SLICE_ROWS
    dk = torch.empty(ns, B, C, nh, D, dtype=torch.float32, device=dev)
    dv = torch.empty(B, C, nh, D, dtype=torch.float32, device=dev)
    db = torch.empty(ns, B, C, nh, dtype=torch.float32, device=dev)
    dla = torch.empty(ns, B, C, nh, dtype=torch.float32, device=dev)
    dS0 = torch.empty(B, nh, D, D, dtype=torch.float32, device=dev)
    _check(_lib.lib().dttt_gdn_chunk_bwd(_p(k), _p(v), _p(beta), _p(log_alpha), _p(states), _p(gS), _p(dk), _p(dv), _p(db), _p(dla), _p(dS0),
                                         B, C, nh, D, _stream()), "gdn_chunk_bwd")
    return dk.sum(0), dv, db.sum(0), dla.sum(0), dS0
