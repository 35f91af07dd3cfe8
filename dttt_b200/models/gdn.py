"""Gated DeltaNet memory: a per-head linear state in place of the fast weight.

One state ``S [nh, dv, dk]`` per suffix layer and sequence, carried across chunks, written from the
clean stream by the gated delta rule over the chunk's tokens

    S_t = a_t S_{t-1} + b_t (v_t - a_t S_{t-1} k_t) k_t^T

and read by every stream of the next chunk as ``o = S q`` (RMS-normalised per head, gated, projected)
at the place of the fast-weight residual (reference ``src/ttt/gdn.py:1-24``; ``read`` ``:97-104``,
``update`` ``:106-123``).  ``q, k`` are SiLU'd and L2-normalised, ``v`` SiLU'd,
``a = exp(-softplus(dt + dt_bias) exp(A_log))``, ``b = sigmoid``.

The write is evaluated in the chunked (WY / UT-transform) form on blocks of ``gdn_chunk`` tokens
(``ops.gdn_scan``), which equals the token-sequential recurrence of the reference
(``update_reference``, gdn.py:125-136) up to rounding.  ``gdn_conv > 0`` adds a causal depthwise short
convolution on the q/k/v projections (an option of this package, identity-initialised, default off).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import functional as Fn
from ..ops import gdn_scan


class GDN:
    @staticmethod
    def _proj(net, f: int, name: str, x: torch.Tensor) -> torch.Tensor:
        bias = net.p("gdn.beta.bias", f) if name == "beta" else None
        return Fn.linear(x, net.p(f"gdn.{name}.weight", f), bias)

    @staticmethod
    def _conv(net, f: int, which: int, y: torch.Tensor) -> torch.Tensor:
        cfg = net.cfg
        if not cfg.gdn_conv:
            return y
        width = cfg.gdn_heads * cfg.gdn_head_dim
        w = net.p("gdn.conv.weight", f)[which * width:(which + 1) * width]          # [width, kw]
        B, C, D = y.shape
        yp = F.pad(y.float().transpose(1, 2), (cfg.gdn_conv - 1, 0))
        return F.conv1d(yp, w.float().unsqueeze(1), groups=D).transpose(1, 2).to(y.dtype)

    @staticmethod
    def read(net, f: int, x: torch.Tensor, S: torch.Tensor) -> torch.Tensor:
        """``x [B, C, H]`` (normed residual), ``S [B, nh, dv, dk]`` -> ``[B, C, H]``."""
        cfg = net.cfg
        nh, dk = cfg.gdn_heads, cfg.gdn_head_dim
        B, C, _ = x.shape
        q = Fn.l2norm(F.silu(GDN._conv(net, f, 0, GDN._proj(net, f, "q", x))).unflatten(-1, (nh, dk)))
        o = torch.einsum("bchk,bhvk->bchv", q.float(), S.float())
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * net.p("gdn.o_norm_w", f).float()
        o = o * F.silu(GDN._proj(net, f, "gate", x).unflatten(-1, (nh, dk)).float())
        return Fn.linear(o.flatten(-2).to(x.dtype), net.p("gdn.o.weight", f))

    @staticmethod
    def write_inputs(net, f: int, x: torch.Tensor):
        cfg = net.cfg
        nh, dk = cfg.gdn_heads, cfg.gdn_head_dim
        k = Fn.l2norm(F.silu(GDN._conv(net, f, 1, GDN._proj(net, f, "k", x))).unflatten(-1, (nh, dk))).float()
        v = F.silu(GDN._conv(net, f, 2, GDN._proj(net, f, "v", x))).unflatten(-1, (nh, dk)).float()
        beta = torch.sigmoid(GDN._proj(net, f, "beta", x).float())
        log_alpha = -F.softplus(GDN._proj(net, f, "dt", x).float() + net.p("gdn.dt_bias", f).float()) \
            * torch.exp(net.p("gdn.A_log", f).float())
        return k, v, beta, log_alpha

    @staticmethod
    def update(net, f: int, x: torch.Tensor, S: torch.Tensor) -> torch.Tensor:
        """The state after the clean chunk ``x [B, C, H]``: ``S [B, nh, dv, dk]`` f32."""
        k, v, beta, log_alpha = GDN.write_inputs(net, f, x)
        return gdn_scan.delta_rule_chunked(k, v, beta, log_alpha, S.float(), net.cfg.gdn_chunk)
