"""Chunked gated delta rule.

The token recurrence ``S_t = a_t S_{t-1} + b_t (v_t - a_t S_{t-1} k_t) k_t^T`` over a block of ``L``
tokens has the closed form (WY representation with the UT transform)

    g_i   = sum_{j<=i} log a_j                          cumulative log-decay inside the block
    A     = strict_lower( diag(b) (K K^T) * exp(g_i - g_j) )
    U     = (I + A)^{-1} diag(b) (V - diag(exp(g)) K S_0^T)       "pseudo values" of the block
    S_L   = exp(g_L) S_0 + sum_j exp(g_L - g_j) u_j k_j^T

so a 1024-token chunk is 16 blocks of 64 tokens with three small GEMMs and one triangular solve each,
instead of 1024 rank-one updates (the reference scans token by token, ``src/ttt/gdn.py:106-123``; its
plain loop ``update_reference`` ``:125-136`` is the oracle of ``tests``).  All math in f32.
"""
from __future__ import annotations

import torch


class _ChunkKernel(torch.autograd.Function):
    """The chunk update on the CUDA kernels: the forward keeps only its inputs, the backward re-creates the block states
    (``csrc/gdn_chunked.cu``) and runs the reverse sweep."""

    @staticmethod
    def forward(ctx, k, v, beta, log_alpha, S0):
        from . import kernels
        ctx.save_for_backward(k, v, beta, log_alpha, S0)
        return kernels.gdn_chunk_fwd(k, v, beta, log_alpha, S0)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gS):
        from . import kernels
        k, v, beta, log_alpha, S0 = ctx.saved_tensors
        dk, dv, db, dla, dS0 = kernels.gdn_chunk_bwd(k, v, beta, log_alpha, S0, gS)
        return dk.to(k.dtype), dv.to(v.dtype), db.to(beta.dtype), dla.to(log_alpha.dtype), dS0.to(S0.dtype)


def delta_rule_chunked(k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, log_alpha: torch.Tensor, S0: torch.Tensor,
                       block: int = 64) -> torch.Tensor:
    """``k [B, C, nh, dk]``, ``v [B, C, nh, dv]``, ``beta / log_alpha [B, C, nh]``, ``S0 [B, nh, dv, dk]`` -> ``S_C``.
    On a GPU (head dimension 64 / 128, blocks of 64) both directions run on the blocked kernel; elsewhere the same block
    algebra is stated in PyTorch below and differentiated by autograd."""
    from . import kernels
    if kernels.gdn_chunk_supported(k, v, min(block, k.shape[1])):
        if torch.is_grad_enabled() and any(t.requires_grad for t in (k, v, beta, log_alpha, S0)):
            return _ChunkKernel.apply(k, v, beta, log_alpha, S0)
        return kernels.gdn_chunk_fwd(k, v, beta, log_alpha, S0)
    B, C, nh, dk = k.shape
    L = min(block, C)
    assert C % L == 0, (C, L)
    S = S0.float()
    kb = k.float().permute(0, 2, 1, 3).unflatten(2, (C // L, L))            # [B, nh, nb, L, dk]
    vb = v.float().permute(0, 2, 1, 3).unflatten(2, (C // L, L))
    bb = beta.float().permute(0, 2, 1).unflatten(2, (C // L, L))            # [B, nh, nb, L]
    gb = log_alpha.float().permute(0, 2, 1).unflatten(2, (C // L, L)).cumsum(-1)
    eye = torch.eye(L, dtype=torch.float32, device=k.device)
    tril = torch.tril(torch.ones(L, L, dtype=torch.bool, device=k.device), -1)
    for n in range(C // L):
        K, V, b, g = kb[:, :, n], vb[:, :, n], bb[:, :, n], gb[:, :, n]
        decay = torch.exp((g[..., :, None] - g[..., None, :]).masked_fill(~tril, 0.0))
        Amat = (b[..., :, None] * (K @ K.transpose(-1, -2)) * decay).masked_fill(~tril, 0.0)
        rhs = b[..., None] * (V - torch.exp(g)[..., None] * (K @ S.transpose(-1, -2)))     # [B, nh, L, dv]
        U = torch.linalg.solve_triangular(eye + Amat, rhs, upper=False, unitriangular=True)
        gL = g[..., -1]
        S = torch.exp(gL)[..., None, None] * S + (U * torch.exp(gL[..., None] - g)[..., None]).transpose(-1, -2) @ K
    return S
