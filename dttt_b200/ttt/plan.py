"""What a batch asks of the model, decided once before the first layer runs.

``StreamPlan.build`` turns ``(token ids, step key, loss configuration)`` into everything the chunk scan consumes and
nothing it computes: the token streams that go through the prefix (outer-masked, clean, inner views, teacher, extra
outer views), their key / query positions and own-chunk patterns, and per chunk the targets, masks and weights of the
outer read, the inner write and the optional heads.  ``loss_fn`` only walks the plan.

Randomness is stateless and its key tree is a contract with the reference (``src/ttt/chunk_scan.py:229-237``, ``:314-325``,
``:346-373``, ``:437-452``): ``split(key, 3) -> (unused, outer mask, inner)``; extra outer views fold the view number into the
outer key; the inner key is split per chunk (row-wise keys) or per (chunk, sequence); the re-read copies use
``fold_in(inner, 1)``, the teacher ``fold_in(inner, 2)``, the window drop ``fold_in(key, 7)`` and the self-prior rows
``fold_in(key, 8)``.  Keeping that tree is what makes a resumed run, a differently sharded run and an evaluation with
row-wise keys draw the masks the reference would.

The plan is built on the device the ids live on: on a GPU the uniform draws run on the counter-RNG kernel and the CART
weights on the band-correlation kernel, so a step neither waits for the host nor copies ``[B, T]`` arrays across.  The few
scalar decisions (window drop) are taken from a host copy of the key.
"""
from __future__ import annotations

import dataclasses as dc
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import attention as A
from ..ops import reference as ref
from ..utils import rng
from . import objective as OBJ
from . import validate as VAL


def ahead(x: torch.Tensor, k: int) -> torch.Tensor:
    """``y[:, i] = x[:, i + k]`` with zeros past the end: slot ``i`` looks at what is ``k`` tokens ahead."""
    return torch.cat([x[:, k:], torch.zeros_like(x[:, :k])], dim=1)


def _next_slots(x: torch.Tensor, k: int) -> torch.Tensor:
    """Along the last axis: ``y[..., i] = x[..., i + k]``; the last ``k`` slots (never scored) keep the final entries."""
    return torch.cat([x[..., k:], x[..., -k:]], dim=-1)


@dc.dataclass
class OuterView:
    """One noisy read of the batch: the masked tokens, which slots are scored and with what weight."""
    tokens: torch.Tensor          # [B, T] ids with [MASK] at the noised slots
    noise: torch.Tensor           # [B] noise level
    masked: torch.Tensor          # [B, T] bool, the noised slots
    raw_weight: torch.Tensor      # [B, T] time weight before masking
    scored: torch.Tensor          # [B, T] bool, the slots whose prediction is scored
    weight: torch.Tensor          # [B, T] f32, zero outside ``scored``


@dc.dataclass
class StreamPlan:
    B: int
    T: int                         # tokens per sequence as laid out (re-read chunks included)
    T_data: int                    # tokens per sequence of the data
    nc: int
    chunk: int
    reread: int                    # chunks that are read twice (evaluation)
    segment_chunks: int
    reach: Optional[int]
    # prefix streams
    streams: torch.Tensor          # [B, NS, T] token ids
    pos_k: torch.Tensor            # [B, NS, T] key positions
    pos_q: Optional[torch.Tensor]  # [B, NS, T] query positions where they differ
    owns: List[str]                # own-chunk pattern of every stream
    n_inner: int
    n_teacher: int
    n_views: int
    # per chunk, [nc, B, C] unless said otherwise
    pos: torch.Tensor
    outer_target: torch.Tensor
    outer_weight: torch.Tensor
    outer_scored: torch.Tensor
    view_weight: List[torch.Tensor]
    view_scored: List[torch.Tensor]
    inner_own: str
    inner_target: Optional[torch.Tensor] = None
    inner_mask: Optional[torch.Tensor] = None        # bool or f32 weights; [nc, B, V, C] with several views
    inner_pos: Optional[torch.Tensor] = None
    inner_pos_q: Optional[torch.Tensor] = None
    feat_index: Optional[torch.Tensor] = None
    teacher_mask: Optional[torch.Tensor] = None
    mtp_outer: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None     # (target, weight, scored)
    mtp_inner: Optional[Tuple[torch.Tensor, torch.Tensor]] = None                   # (target, mask)
    self_prior_rows: Optional[torch.Tensor] = None   # [B] bool
    write_steps: Optional[Tuple[int, ...]] = None    # per chunk, with a write plan
    read_mask: Optional[torch.Tensor] = None         # [C, 2C] sub-block read pattern
    window: int = 0                                  # window chunks of the model
    write_inputs: bool = True                        # the write (or the outer-driven write) reads the inner mask

    @property
    def NS(self) -> int:
        return self.streams.shape[1]

    def data_chunk(self, c: int) -> int:
        """Index within the data of laid-out chunk ``c`` (the second pass of a re-read restarts at 0)."""
        return c - self.reread if (self.reread and c >= self.reread) else c

    def at(self, c: int) -> Dict[str, object]:
        """Everything chunk ``c`` needs, as the keyword bundle of ``scan._suffix_step``."""
        pick = lambda t: None if t is None else t[c]
        has_write_inputs = self.write_inputs and self.inner_mask is not None
        mtp_o = self.mtp_outer or (None, None, None)
        mtp_i = self.mtp_inner or (None, None)
        return dict(c=c, nv=A.valid_window_chunks(self.data_chunk(c), self.window, self.reach), p=self.pos[c],
                    tok=self.outer_target[c], wgt=self.outer_weight[c], tm=self.outer_scored[c],
                    im=self.inner_mask[c] if has_write_inputs else None, tgt=pick(self.inner_target), p_in=pick(self.inner_pos),
                    p_q=pick(self.inner_pos_q), ti=pick(self.feat_index), mt=pick(self.teacher_mask),
                    tok2=pick(mtp_o[0]), wgt2=pick(mtp_o[1]), tm2=pick(mtp_o[2]), mtp_t=pick(mtp_i[0]), mtp_m=pick(mtp_i[1]),
                    wv=[w[c] for w in self.view_weight], tmv=[m[c] for m in self.view_scored],
                    k_c=None if self.write_steps is None else self.write_steps[c])

    # ------------------------------------------------------------------------------------------------ construction
    @staticmethod
    def build(batch, key: torch.Tensor, step: int, cfg, mc, device: torch.device) -> "StreamPlan":
        """``batch``: a ``scan.Batch`` whose tensors may live anywhere; ``key [2]`` or row-wise ``[B, 2]``."""
        on = lambda x: None if x is None else x.to(device, non_blocking=True)
        ids = on(batch.input_ids).long()
        B, T = ids.shape
        C, Wn = mc.chunk_size, mc.window_chunks
        if T % C:
            raise ValueError(f"seq_len {T} not a multiple of chunk_size {C}")
        nc = T // C
        # the key tree is derived where the key lives (a handful of 64-bit integers, normally the host); only the bulk
        # draws happen on `device` (objective.q_sample / inner_masks move the derived keys over)
        key_host = key.detach().to("cpu")
        key = key_host
        rowwise = key.dim() == 2
        pos = torch.arange(T, device=device)[None].expand(B, T) if batch.position_ids is None else on(batch.position_ids).long()
        _, key_outer, key_inner = rng.split(key, 3).unbind(-2)
        per_chunk_keys = lambda k, n: (rng.split(k, n).transpose(0, 1) if rowwise else rng.split(k, n * B).reshape(n, B, 2))

        # ---- the outer read(s)
        scorable = on(batch.loss_mask)
        if cfg.score_from_chunk:
            late = (torch.arange(T, device=device) >= cfg.score_from_chunk * C)[None]
            scorable = late.expand(B, T) if scorable is None else (scorable.bool() & late)
        level = on(batch.outer_t)
        if cfg.outer_t >= 0:
            level = torch.full((B,), cfg.outer_t, dtype=torch.float32, device=device)
        cart = ref.cart_kernel(cfg.cart_p, cfg.cart_window, device) if (cfg.time_reweighting == "cart" or cfg.inner_cart) else None
        look = 1 if cfg.outer_shift else 0                       # a slot predicts the token `look` places ahead

        def read(k) -> OuterView:
            tokens, noise, masked = OBJ.q_sample(k, ids, scorable, mc.mask_token_id, t=level)
            raw = OBJ.time_weights(cfg.time_reweighting, noise, masked, cart)
            scored = ahead(masked, look) if look else masked
            return OuterView(tokens, noise, masked, raw, scored, (ahead(raw, look) if look else raw) * scored.float())

        main = read(key_outer)
        more = [read(rng.fold_in(key_outer, v)) for v in range(1, cfg.outer_views)]
        outer_target = ahead(ids, look) if look else ids

        # ---- draws that are one number per batch or per sequence
        reach = mc.reach
        if cfg.window_drop > 0:
            first_key = key_host if key_host.dim() == 1 else key_host[0]
            dropped = bool(rng.uniform(rng.fold_in(first_key, 7), ()) < cfg.window_drop) and step < cfg.window_drop_until
            reach = 0 if dropped else (Wn if mc.reach is None else mc.reach)
        prior_rows = None
        if cfg.self_prior > 0:
            k8 = rng.fold_in(key, 8)
            prior_rows = on((rng.uniform(k8, ()) if rowwise else rng.uniform(k8, (B,))) < cfg.self_prior)

        mtp_outer = None
        if cfg.mtp:
            seen2 = ahead(main.masked, 2)
            mtp_outer = (ahead(ids, 2), ahead(main.raw_weight, 2) * seen2.float(), seen2)

        # ---- re-read layout (evaluation): the first `n_rr` chunks are laid out twice, the first pass clean and unscored
        n_rr = cfg.reread_chunks
        inner_keys = per_chunk_keys(key_inner, nc)
        host_mask, host_order = on(batch.inner_mask), on(batch.inner_perm)
        x_outer = main.tokens
        scored, weight = main.scored, main.weight
        if n_rr:
            lead = n_rr * C
            twice = lambda a: torch.cat([a[:, :lead], a], dim=1)
            muted = lambda a: torch.cat([torch.zeros_like(a[:, :lead]), a], dim=1)
            x_outer = torch.cat([ids[:, :lead], x_outer], dim=1)
            ids, pos, outer_target = twice(ids), twice(pos), twice(outer_target)
            scored, weight = muted(scored), muted(weight)
            if mtp_outer is not None:
                mtp_outer = (twice(mtp_outer[0]), muted(mtp_outer[1]), muted(mtp_outer[2]))
            host_mask = None if host_mask is None else twice(host_mask)
            if host_order is not None:
                host_order = torch.cat([host_order[:, :lead], host_order + lead], dim=1)
            inner_keys = torch.cat([per_chunk_keys(rng.fold_in(key_inner, 1), n_rr), inner_keys], dim=0)
        T_all, nc_all = T + n_rr * C, nc + n_rr
        write_steps = (tuple(cfg.write_plan) + (1,) * nc_all)[:nc_all] if cfg.write_plan else None

        plan = StreamPlan(B=B, T=T_all, T_data=T, nc=nc_all, chunk=C, reread=n_rr, window=Wn,
                          segment_chunks=VAL.check_geometry(T_all, mc, cfg.segment_chunks, nc_all), reach=reach,
                          streams=None, pos_k=None, pos_q=None, owns=[], n_inner=0, n_teacher=int(bool(cfg.distill)),
                          n_views=cfg.outer_views, pos=OBJ.to_chunks(pos, C), outer_target=OBJ.to_chunks(outer_target, C),
                          outer_weight=OBJ.to_chunks(weight, C), outer_scored=OBJ.to_chunks(scored, C),
                          view_weight=[OBJ.to_chunks(v.weight, C) for v in more], view_scored=[OBJ.to_chunks(v.scored, C) for v in more],
                          inner_own="full", self_prior_rows=prior_rows, write_steps=write_steps,
                          write_inputs=not (cfg.no_write and not cfg.inner_from_outer),
                          mtp_outer=None if mtp_outer is None else tuple(OBJ.to_chunks(t, C) for t in mtp_outer),
                          read_mask=A.read_mask_matrix(C, mc.read_block, device) if mc.read_block else None)
        inner_tokens = plan._inner_task(cfg, mc, ids, pos, inner_keys, host_mask, host_order, cart)
        teacher_tokens = None
        if cfg.distill:
            teacher_keys = per_chunk_keys(rng.fold_in(key_inner, 2), nc_all)
            teacher_c, plan.teacher_mask = OBJ.inner_masks(teacher_keys, OBJ.to_chunks(ids, C), -1.0, cfg.distill_t_range,
                                                           mc.mask_token_id, mc.pad_token_id)
            teacher_tokens = OBJ.from_chunks(teacher_c)
        plan._streams(cfg, ids, pos, x_outer, inner_tokens, teacher_tokens, [v.tokens for v in more], look)
        return plan

    def _inner_task(self, cfg, mc, ids, pos, inner_keys, host_mask, host_order, cart) -> List[torch.Tensor]:
        """What stream C sees and predicts (reference chunk_scan.py:375-427); returns the inner token streams ``[B, T]``."""
        C, B, T, nc, dev = self.chunk, self.B, self.T, self.nc, ids.device
        ids_c, pos_c = OBJ.to_chunks(ids, C), OBJ.to_chunks(pos, C)
        views = cfg.inner_views
        slot = torch.arange(C, device=dev)
        local_order = None
        if cfg.inner_task == "mask":
            if host_mask is not None:
                if views != 1:
                    raise ValueError("host-side inner masks support one view")
                hidden = OBJ.to_chunks(host_mask.bool(), C)
                seen = torch.where(hidden, torch.full_like(ids_c, mc.mask_token_id), ids_c)
            else:
                seen, hidden = OBJ.inner_masks(inner_keys, ids_c, cfg.inner_mask_ratio, cfg.inner_mask_range, mc.mask_token_id,
                                               mc.pad_token_id, views, cfg.inner_mask_span, cfg.inner_view_mode)
            if cfg.inner_cart:
                flat = hidden.reshape(-1, C).float()
                hidden = (OBJ.cart_weights(1.0 - flat, cart) * flat).reshape(hidden.shape)
            self.inner_target, self.inner_mask, self.inner_pos = ids_c, hidden, pos_c
        else:
            if views != 1:
                raise ValueError("causal / split inner tasks are single-view")
            if cfg.inner_task == "split":
                if host_order is None:
                    raise ValueError("inner_task split needs Batch.inner_perm (host-side, data.masks.split_perm)")
                order = OBJ.to_chunks(host_order.long(), C)
                n_ctx = int(round(cfg.inner_context_frac * C))
                self.inner_own = f"split:{n_ctx}"
            else:
                order = torch.arange(T, device=dev).reshape(nc, 1, C).expand(nc, B, C)
                n_ctx = 0
                self.inner_own = "causal"
            take = lambda a: torch.gather(a[None].expand(nc, B, T), 2, order)
            seen = take(ids)
            self.inner_pos = take(pos)
            # slot i predicts the token at slot i + 1 of the physical order; it is asked from the first target's predecessor on
            self.inner_target, self.inner_pos_q = _next_slots(seen, 1), _next_slots(self.inner_pos, 1)
            self.inner_mask = ((slot >= max(n_ctx - 1, 0)) & (slot <= C - 2))[None, None].expand(nc, B, C)
            local_order = order - (torch.arange(nc, device=dev) * C)[:, None, None]
        if cfg.inner_feat != "off":
            if cfg.inner_task == "mask":
                self.feat_index = slot[None, None].expand(nc, B, C)
            elif cfg.inner_task == "causal":
                self.feat_index = torch.clamp(slot + 1, max=C - 1)[None, None].expand(nc, B, C)
            else:
                self.feat_index = _next_slots(local_order, 1)
        if cfg.mtp:
            self.mtp_inner = (_next_slots(seen, 2), (slot <= C - 3)[None, None].expand(nc, B, C).float())
        if cfg.no_write or cfg.inner_from_outer:
            return []
        self.n_inner = views
        return [OBJ.from_chunks(seen)] if views == 1 else [OBJ.from_chunks(seen[:, :, v]) for v in range(views)]

    def _streams(self, cfg, ids, pos, x_outer, inner_tokens, teacher_tokens, view_tokens, look: int) -> None:
        """Stack the prefix streams ``[outer, clean, inner views..., teacher, extra outer views...]`` with their positions."""
        tail = ([teacher_tokens] if teacher_tokens is not None else []) + view_tokens
        self.streams = torch.stack([x_outer, ids] + inner_tokens + tail, dim=1)
        self.owns = ["full", "full"] + [self.inner_own] * len(inner_tokens) + ["full"] * len(tail)
        natural_inner = cfg.inner_task == "mask" or not inner_tokens
        if not look and natural_inner:
            self.pos_k, self.pos_q = pos[:, None].expand(self.B, self.NS, self.T), None
            return
        # outer-like streams ask for the token `look` ahead; the inner stream has its own physical order and asks for the next slot
        inner_k = pos if natural_inner else OBJ.from_chunks(self.inner_pos)
        inner_q = pos if (natural_inner or self.inner_pos_q is None) else OBJ.from_chunks(self.inner_pos_q)
        ask = pos + look
        self.pos_k = torch.stack([pos, pos] + [inner_k] * len(inner_tokens) + [pos] * len(tail), dim=1)
        self.pos_q = torch.stack([ask, pos] + [inner_q] * len(inner_tokens) + [ask] * len(tail), dim=1)
