"""Outer optimiser: global-norm clip + AdamW with a warmup-stable-decay schedule, on the FSDP shards.

Semantics are those of the reference's ``optax.chain(clip_by_global_norm, adamw(schedule, mask))``
(``src/ttt/train.py:137-167``):

    g      <- g * min(1, clip / ||g||)                          one norm over every parameter
    m      <- b1 m + (1 - b1) g ;  v <- b2 v + (1 - b2) g^2
    update  = (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps) + wd * p      wd only where the name does not
                                                                            match ``no_decay_pattern``
    p      <- p - lr(t - 1) * scale * update                    scale = fast_weight_lr_scale on the W_0 template

with ``t`` counting from 1 and ``lr(s)`` = linear warm-up ``0 -> lr`` over ``warmup_steps``, flat, then
linear ``lr -> end_lr`` between ``decay_start`` and ``decay_end`` (all in global steps).  State lives on
the flat master shards of ``parallel.store.ParamStore``; the gradient arrives in ``store.grad_shard``
(already summed over data ranks) and is divided by ``grad_scale`` (the global loss normaliser) on the fly.
"""
from __future__ import annotations

import math
import re
from typing import Dict, List, Optional, Tuple

import torch

from .parallel.store import ParamStore

GROUPS = ("embed", "prefix", "suffix", "fast_weight", "other")


def lr_at(step: int, lr: float, end_lr: float, warmup_steps: int, decay_start: int = -1, decay_end: int = -1) -> float:
    """Warm-up-stable-decay over global steps (reference train.py:137-145)."""
    w = max(1, warmup_steps)
    if decay_start >= 0 and step >= decay_start:
        frac = min(1.0, (step - decay_start) / max(1, decay_end - decay_start))
        return lr + (end_lr - lr) * frac
    return lr * min(1.0, step / w)


def group_of(name: str) -> str:
    if name == "embed" or name == "lm_head":
        return "embed"
    if name.startswith("prefix."):
        return "prefix"
    if name.startswith("suffix."):
        return "suffix"
    if name.startswith("fast_weight.") or name.startswith("gdn."):
        return "fast_weight"
    return "other"


class ShardedAdamW:
    def __init__(self, store: ParamStore, lr: float, end_lr: float, warmup_steps: int, decay_start: int = -1,
                 decay_end: int = -1, weight_decay: float = 0.1, grad_clip: float = 1.0, b1: float = 0.9, b2: float = 0.95,
                 eps: float = 1e-8, no_decay_pattern: str = r"embed|norm|bias|inner_|A_log", fast_weight_lr_scale: float = 1.0):
        self.store = store
        self.hp = dict(lr=lr, end_lr=end_lr, warmup_steps=warmup_steps, decay_start=decay_start, decay_end=decay_end)
        self.wd, self.clip, self.b1, self.b2, self.eps = weight_decay, grad_clip, b1, b2, eps
        self.fw_scale = fast_weight_lr_scale
        self.m = torch.zeros_like(store.master)
        self.v = torch.zeros_like(store.master)
        self.count = 0                                   # optimiser steps taken (optax's ``count``)
        self.wrote_compute = False                       # the fused step also refreshed every rank's compute copies
        nd = re.compile(no_decay_pattern) if no_decay_pattern else None
        fast = re.compile(r"(^|\.)fast_weight(\.|$)")
        self.segs: List[Tuple[str, int, int, float, float]] = []
        for name, a, b in store.segments():
            decay = 0.0 if (nd is not None and nd.search(name)) else weight_decay
            scale = fast_weight_lr_scale if fast.search(name) else 1.0
            self.segs.append((name, a, b, decay, scale))

    def lr(self, step: Optional[int] = None) -> float:
        return lr_at(self.count if step is None else step, **self.hp)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> Dict[str, float]:
        """One update from ``store.grad_shard``; ``grad_scale`` divides the gradient first.  Returns the global
        gradient norm (before clipping), its per-group parts and the finiteness flag."""
        st = self.store
        g = st.grad_shard
        if grad_scale != 1.0:
            g.mul_(1.0 / grad_scale)
        # squared norms per group; the slices of tensor-parallel weights add up over the TP group, whole parameters count once
        sq2 = torch.zeros(2, len(GROUPS), dtype=torch.float32, device=g.device)
        for name, a, b, _, _ in self.segs:
            sq2[1 if st.tp_layout.get(name) is not None else 0, GROUPS.index(group_of(name))] += g[a:b].pow(2).sum()
        sq2 = st.all_reduce_scalar(sq2, groups=("fsdp",))
        if st.mesh.tp > 1:
            st.all_reduce_scalar(sq2[1], groups=("tp",))
        sq = sq2[0] + sq2[1]
        sq_host = sq.tolist()
        gnorm = math.sqrt(sum(sq_host))
        finite = math.isfinite(gnorm)
        factor = 1.0
        if self.clip > 0 and finite and gnorm > self.clip:
            factor = self.clip / gnorm
        lr = self.lr()
        self.count += 1
        t = self.count
        bc1, bc2 = 1.0 - self.b1 ** t, 1.0 - self.b2 ** t
        from .ops import kernels
        fused = g.is_cuda and kernels.available("adamw")
        if st.fused:
            # AdamW on the shard and the all-gather of the updated compute copies in one kernel per segment: the new
            # value of every element is stored into every FSDP rank's compute buffer over NVLink as it is produced.
            from .parallel import symm
            me = st.mesh.fsdp_index
            for name, a, b, decay, scale in self.segs:
                space, off = st.space_of_master_index(a)
                # (a matrix gathered per use keeps only this rank's slice current: the same kernel with this rank as the only peer)
                table, world, who = (st._lo_self_tables[space], 1, 0) if name in st.sharded_names else (st._lo_tables[space], st.fs, me)
                symm.adamw_allgather(st.master[a:b], self.m[a:b], self.v[a:b], g[a:b], lr * scale, self.b1, self.b2, self.eps,
                                     decay, bc1, bc2, factor, table, world, who, off, space == "big" and st.dtype == torch.bfloat16)
            st.barrier()                                     # every rank's stores have landed before anyone reads
            self.wrote_compute = True
        for name, a, b, decay, scale in ([] if st.fused else self.segs):
            p, m, v, gg = st.master[a:b], self.m[a:b], self.v[a:b], g[a:b]
            if fused:
                kernels.adamw(p, m, v, gg, lr * scale, self.b1, self.b2, self.eps, decay, bc1, bc2, factor)
                continue
            if factor != 1.0:
                gg = gg * factor
            m.mul_(self.b1).add_(gg, alpha=1.0 - self.b1)
            v.mul_(self.b2).addcmul_(gg, gg, value=1.0 - self.b2)
            upd = (m / bc1) / ((v / bc2).sqrt_().add_(self.eps))
            if decay:
                upd.add_(p, alpha=decay)
            p.add_(upd, alpha=-lr * scale)
        out = {"grad_norm": gnorm, "finite": float(finite), "lr": lr}
        for k, s in zip(GROUPS, sq_host):
            out[f"gnorm_{k}"] = math.sqrt(max(s, 0.0))
        return out

    # ---- state for checkpoints: the optax leaf order is (adam count, mu tree, nu tree, schedule count)
    def state_dict(self) -> dict:
        return {"count": self.count}
