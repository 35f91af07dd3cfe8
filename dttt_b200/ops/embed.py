"""Token embedding lookup from the f32 master table.

The forward gathers rows of the table's compute copy (the same values as rows of the f32 master cast to
the compute dtype); the backward
scatter-adds every position's gradient row, in f32, straight into the master's gradient buffer.  A
row hit thousands of times per step (the mask token) loses most of its gradient when that sum runs
in bf16 (reference ``src/ttt/model.py:534-542``: 53 % on the mask row), hence f32 end to end.
"""
from __future__ import annotations

import torch


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids, dtype, gradbuf):
        ctx.save_for_backward(ids)
        ctx.gradbuf, ctx.shape, ctx.tdtype = gradbuf, table.shape, table.dtype
        return _gather(table.detach(), ids, dtype)

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        if torch.is_grad_enabled() or ctx.gradbuf is None:
            gt = torch.zeros(ctx.shape, dtype=torch.float32, device=g.device).index_add(0, ids.flatten(), g.float().flatten(0, -2))
            return gt.to(ctx.tdtype), None, None, None
        if _kernel_ok(g, ctx.gradbuf) and g.dtype == torch.bfloat16 and ctx.gradbuf.is_contiguous():
            from . import kernels
            kernels.embed_scatter_f32(g, ids, ctx.gradbuf)
        else:
            ctx.gradbuf.index_add_(0, ids.flatten(), g.float().flatten(0, -2))
        return None, None, None, None


def _kernel_ok(*ts) -> bool:
    from . import kernels
    return all(t.is_cuda for t in ts) and kernels.available("embed")


def _gather(table: torch.Tensor, ids: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if _kernel_ok(table) and table.dtype == torch.bfloat16 and dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
        from . import kernels
        return kernels.embed_gather(table, ids)
    return table[ids].to(dtype)


def embedding(table: torch.Tensor, ids: torch.Tensor, dtype: torch.dtype, gradbuf=None) -> torch.Tensor:
    """``table [V, H]`` (compute copy of the embedding, a leaf), ``ids [...]`` -> ``[..., H]`` in ``dtype``;
    ``gradbuf``: the f32 ``[V, H]`` gradient buffer the backward scatter-adds into."""
    ids = ids.long()
    if table.requires_grad and torch.is_grad_enabled():
        return _Embedding.apply(table, ids, dtype, gradbuf)
    return _gather(table.detach(), ids, dtype)
