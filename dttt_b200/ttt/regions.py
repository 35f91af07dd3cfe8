"""Recompute regions: explicit activation checkpointing for code that takes gradients inside itself.

``region(fn, inputs)`` runs ``fn(*inputs)`` (tensors in, tuple of tensors out) without recording a
graph and keeps only the inputs; when a gradient arrives it runs ``fn`` again with recording on and
back-propagates through that run.  Parameters that ``fn`` closes over receive their gradients
directly (leaf ``.grad`` or the f32 buffers the GEMM epilogue accumulates into).  Unlike the stock
checkpoint utilities this works when ``fn`` itself calls ``torch.autograd.grad`` (the inner step):
the first run takes that gradient on detached copies, the re-run takes it with ``create_graph`` so
the outer gradient flows through it.  It replaces the reference's ``jax.checkpoint`` levels
(``src/ttt/remat_scan.py:70-120``; per layer ``model.py:588-592``, per chunk ``chunk_scan.py:730-735``).
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch

from ..utils import prof


class _Region(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, label, *inputs):
        ctx.fn, ctx.label = fn, label
        ctx.save_for_backward(*inputs)
        with torch.no_grad():
            outs = fn(*inputs)
        outs = tuple(outs)
        ctx.mark_non_differentiable(*[o for o in outs if not o.is_floating_point()])
        return outs

    @staticmethod
    def backward(ctx, *gouts):
        inputs = ctx.saved_tensors
        det = [t.detach().requires_grad_(t.is_floating_point() and need)
               for t, need in zip(inputs, ctx.needs_input_grad[2:])]
        with prof.range(ctx.label or "region.bwd"):
            with torch.enable_grad():
                outs = tuple(ctx.fn(*det))
            sel = [(o, g) for o, g in zip(outs, gouts) if g is not None and o.requires_grad]
            if sel:
                torch.autograd.backward([o for o, _ in sel], [g for _, g in sel])
        return (None, None, *[d.grad if d.requires_grad else None for d in det])


def region(fn: Callable, inputs: Sequence[torch.Tensor], enabled: bool = True, label: str = "") -> Tuple[torch.Tensor, ...]:
    """``fn(*inputs)`` as a recompute region (``enabled``) or directly; ``label`` names its backward in ``utils.prof``."""
    if not enabled or not torch.is_grad_enabled():
        return tuple(fn(*inputs))
    return _Region.apply(fn, label, *inputs)
