"""The op surface the model is written against.

Every function here has one meaning (the plain-PyTorch statement in ``ops.reference``) and up to
three executions:

* on CPU, or for f32 tensors: the reference code itself (autograd differentiates it to any order);
* on a CUDA device with bf16 tensors: the hand-written sm_100a kernel for the forward and for the
  first-order backward;
* when a backward pass runs with gradient recording on (``create_graph=True``: the inner step whose
  gradient the meta-gradient differentiates again, reference ``src/ttt/chunk_scan.py:604-625``), the
  backward is computed by differentiating the reference statement, so the result is itself
  differentiable.  This is the staging the reference uses for attention (cuDNN forward and first-order
  backward, XLA for the second order, ``src/ttt/attention.py:357-405``), applied to every op.

``kernel_fn(fast_forward, fast_backward, reference)`` builds such a function.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import reference as ref
from . import gemm as _gemm

mm = _gemm.mm


def use_kernels(*tensors: torch.Tensor) -> bool:
    """Kernels run for CUDA bf16 activations; anything else takes the reference path."""
    t = tensors[0]
    return (t.is_cuda or _gemm.EMULATE) and t.dtype == torch.bfloat16 and not _gemm._FORCE_TORCH


class _Staged(torch.autograd.Function):
    """forward: ``fast_fwd(*tensors)`` -> (out, saved...); backward: ``fast_bwd`` when no graph is being
    recorded; else the optional fourth entry of the spec, a backward that is itself a differentiable
    operation (it may decline by returning ``None``), else the VJP of ``ref_fn`` taken with
    ``create_graph=True``."""

    @staticmethod
    def forward(ctx, spec, n_tensors, *args):
        tensors, consts = args[:n_tensors], args[n_tensors:]
        fast_fwd = spec[0]
        out, saved = fast_fwd(*tensors, *consts)
        ctx.spec, ctx.consts, ctx.n = spec, consts, n_tensors
        ctx.n_saved = len(saved)
        ctx.save_for_backward(*tensors, *saved)
        return out

    @staticmethod
    def backward(ctx, g):
        fast_bwd, ref_fn = ctx.spec[1], ctx.spec[2]
        diff_bwd = ctx.spec[3] if len(ctx.spec) > 3 else None
        tensors = ctx.saved_tensors[:ctx.n]
        saved = ctx.saved_tensors[ctx.n:]
        needs = ctx.needs_input_grad[2:2 + ctx.n]
        full = None
        if torch.is_grad_enabled() and diff_bwd is not None:
            res = diff_bwd(g, tensors, saved, needs, *ctx.consts)
            if res is not None:
                full = [t if nd else None for t, nd in zip(res, needs)]
        if full is not None:
            pass
        elif torch.is_grad_enabled():
            with torch.enable_grad():
                ins = [t if t.requires_grad else t.detach().requires_grad_(nd) for t, nd in zip(tensors, needs)]
                out = ref_fn(*ins, *ctx.consts)
                wrt = [t for t, nd in zip(ins, needs) if nd]
                grads = torch.autograd.grad(out, wrt, g, create_graph=True, allow_unused=True)
            it = iter(grads)
            full = [next(it) if nd else None for nd in needs]
        else:
            full = list(fast_bwd(g.contiguous(), tensors, saved, needs, *ctx.consts))
        return (None, None, *full, *([None] * len(ctx.consts)))


def staged(spec, tensors: Sequence[torch.Tensor], consts: Sequence = ()):
    return _Staged.apply(spec, len(tensors), *tensors, *consts)


# ------------------------------------------------------------------ linear with direct f32 grad accumulation
class _LinearW(torch.autograd.Function):
    """``x @ w`` for a weight leaf that carries ``grad_target = (f32 gradient buffer, layer)``: the first-order
    weight gradient ``x^T g`` is added by the GEMM epilogue into the master's f32 gradient buffer
    (no bf16 round trip, no separate accumulation pass); the weight then receives no autograd gradient.
    When the backward is being recorded (meta-gradient) both gradients are ordinary differentiable
    products instead."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.target = getattr(w, "grad_target", None)
        return _gemm.gemm_raw(x, w, False, False)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        gx = gw = None
        if torch.is_grad_enabled():
            if ctx.needs_input_grad[0]:
                gx = mm(g, w, False, True)
            if ctx.needs_input_grad[1] and not _INNER_BACKWARD[0]:
                gw = mm(x, g, True, False)
            return gx, gw
        if ctx.needs_input_grad[0]:
            gx = _gemm.gemm_raw(g, w, False, True)
        if ctx.needs_input_grad[1] and not _INNER_BACKWARD[0]:
            if ctx.target is not None:
                gbuf, layer = ctx.target
                buf = gbuf if layer is None else gbuf[layer]
                _gemm.gemm_raw(x, g, True, False, torch.float32, out=buf, accumulate=True)
            else:
                gw = _gemm.gemm_raw(x, g, True, False)
        return gx, gw


# True while the inner step's gradient w.r.t. the fast weights is being taken: slow-weight gradients are
# not wanted from that pass (they are not among its inputs) and must not be accumulated by side effect.
_INNER_BACKWARD = [False]


class inner_backward:
    def __enter__(self):
        self.prev = _INNER_BACKWARD[0]
        _INNER_BACKWARD[0] = True

    def __exit__(self, *a):
        _INNER_BACKWARD[0] = self.prev


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w (+ bias)``; ``w [in, out]`` (reference model.py:137-148) or per-sequence ``[B, in, out]``
    with ``x [B, C, in]``."""
    if getattr(w, "tp", None) is not None:
        from ..parallel.tp import tp_linear
        return tp_linear(x, w, bias)
    if getattr(w, "wg", None) is not None:
        from ..parallel.wgather import wg_linear
        return wg_linear(x, w, bias)
    if w.dim() == 3:
        y = mm(x, w.to(x.dtype) if w.dtype != x.dtype else w)
    else:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if use_kernels(x2) and w.dtype == torch.bfloat16 and torch.is_grad_enabled() and w.requires_grad \
                and getattr(w, "grad_target", None) is not None:
            y = _LinearW.apply(x2, w)
        else:
            y = mm(x2, w if w.dtype == x2.dtype else w.to(x2.dtype))
        y = y.view(*lead, w.shape[-1])
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y


# ------------------------------------------------------------------ elementwise / normalisation
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    from . import kernels
    if use_kernels(x) and kernels.available("rmsnorm"):
        return kernels.rms_norm(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


def glu(gate: torch.Tensor, up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    from . import kernels
    if use_kernels(gate) and act == "silu" and kernels.available("swiglu"):
        return kernels.swiglu(gate, up)
    return ref.glu(gate, up, act)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return ref.apply_rope(x, cos, sin)


_INV_FREQ = {}


def inv_freq(head_dim: int, theta: float, scaling, device) -> torch.Tensor:
    key = (head_dim, theta, scaling, str(device))
    t = _INV_FREQ.get(key)
    if t is None:
        t = _INV_FREQ[key] = ref.rope_inv_freq(head_dim, theta, scaling, "cpu").to(device)
    return t


def rope(x: torch.Tensor, pos: torch.Tensor, head_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """Rotary embedding of ``x [..., T, heads, d]`` at positions ``pos [..., T]`` (f32 angles, half-rotation
    layout, optional llama3 frequency scaling; reference model.py:82-117)."""
    from . import kernels
    inv = inv_freq(head_dim, theta, scaling, x.device)
    if use_kernels(x) and kernels.available("rope"):
        return kernels.rope(x, pos.long(), inv)
    ang = pos.float().unsqueeze(-1) * inv
    emb = torch.cat([ang, ang], dim=-1)
    return ref.apply_rope(x, emb.cos(), emb.sin())


rope_cos_sin = ref.rope_cos_sin
l2norm = ref.l2norm
