"""Token embedding lookup from the f32 master table.

The forward gathers rows of the f32 table and casts them to the compute dtype; the backward
scatter-adds every position's gradient row, in f32, straight into the master's gradient buffer.  A
row hit thousands of times per step (the mask token) loses most of its gradient when that sum runs
in bf16 (reference ``src/ttt/model.py:534-542``: 53 % on the mask row), hence f32 end to end.
"""
from __future__ import annotations

import torch


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, table, ids, dtype):
        ctx.save_for_backward(ids)
        ctx.table = table
        return table.detach()[ids.long()].to(dtype)

    @staticmethod
    def backward(ctx, g):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        if torch.is_grad_enabled():
            # recorded backward: an ordinary differentiable scatter (never on the training path)
            gt = torch.zeros_like(table).index_add(0, ids.long().flatten(), g.float().flatten(0, -2))
            return gt, None, None
        if table.grad is None:
            table.grad = torch.zeros_like(table)
        table.grad.index_add_(0, ids.long().flatten(), g.float().flatten(0, -2))
        return None, None, None


def embedding(table: torch.Tensor, ids: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``table [V, H]`` f32 leaf, ``ids [...]`` -> ``[..., H]`` in ``dtype``."""
    if table.requires_grad and torch.is_grad_enabled() and table.is_cuda:
        return _Embedding.apply(table, ids, dtype)
    return torch.nn.functional.embedding(ids.long(), table).to(dtype)
