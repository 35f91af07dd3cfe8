"""The training objective over a batch: chunk-parallel prefix, then a sequential pass over chunks for the
suffix with the KV window and the per-sequence memory (fast weight or GDN state) carried along.

Per chunk the suffix runs three forwards on the same chunk, key set and memory (reference
``src/ttt/chunk_scan.py:6-23``):

    A  outer-masked -> CART-weighted CE against the clean tokens          (the loss)
    B  clean        -> this chunk's K/V, shifted into the window
    C  inner        -> gradient w.r.t. W, one clipped step                 (the write)

and the outer gradient flows through every write.  Memory scheduling is explicit: each prefix layer
and each chunk step is a *recompute region* (``regions.region``): its inputs are kept, its forward runs
without a graph, and its backward re-runs it with the graph (the inner step then with
``create_graph``) — the reference's remat scan (``src/ttt/remat_scan.py``, ``model.py:588-592``,
``chunk_scan.py:730-735``) as per-layer / per-chunk activation checkpointing.  Segments
(``segment_chunks``) bound the prefix transients for long sequences and are where
``truncate_fast_weight`` cuts the meta-gradient (``chunk_scan.py:39-49``).
"""
from __future__ import annotations

import dataclasses as dc
from typing import NamedTuple, Optional, Tuple

import torch

from ..models.blocks import CLEAN, INNER, OUTER, Net
from ..ops import ce as CE
from ..ops import functional as Fn
from ..utils import prof, rng
from . import inner as IN
from . import validate as VAL
from .plan import StreamPlan
from .regions import region


# From this many segments on a segment is a recompute region of its own.  Below it the per-chunk carries of the whole
# sequence (0.9 GB per chunk and sequence at 1B) still fit beside the working set and the extra forward pass (about 15 % of a
# step) is not worth paying; from 64 chunks (128k tokens of 1024-token chunks in segments of 8) they no longer do.
NEST_SEGMENTS_FROM = 8
STREAMS_TOGETHER = True      # the read and the clean pass of a chunk step in one pass through the suffix where they share the memory


class Batch(NamedTuple):
    input_ids: torch.Tensor                          # [B, T]
    loss_mask: Optional[torch.Tensor] = None         # [B, T] bool
    position_ids: Optional[torch.Tensor] = None      # [B, T]
    inner_mask: Optional[torch.Tensor] = None        # [B, T] bool: host-chosen inner targets
    inner_perm: Optional[torch.Tensor] = None        # [B, T] physical order of the inner stream (split task)
    outer_t: Optional[torch.Tensor] = None           # [B] explicit noise level per sequence


@dc.dataclass(frozen=True)
class LossConfig:
    """Everything ``loss_fn`` needs that is not in ``ModelConfig`` (reference chunk_scan.py:81-143)."""
    time_reweighting: str = "cart"
    cart_p: float = 0.1
    cart_window: int = 512
    outer_t: float = -1.0
    outer_shift: bool = False
    inner_lr: float = 1.0
    inner_clip: float = 1.0
    inner_lr_warmup_steps: int = 0
    inner_mask_range: Tuple[float, float] = (0.5, 1.0)
    inner_mask_ratio: float = -1.0
    second_order: bool = True
    remat_levels: int = 1
    remat_prefix: bool = False
    prefix_remat_levels: int = 1
    keep_prefix_layers: int = 0           # the first k prefix layers are not recompute regions: their activations stay resident
    keep_suffix_chunks: int = 0           # likewise the first k chunk steps of every segment (their recorded graph stays resident)
    segment_chunks: int = 0
    truncate_fast_weight: bool = False
    inner_views: int = 1
    inner_view_mode: str = "complement"
    inner_views_sequential: bool = False
    inner_cart: bool = False
    inner_mask_span: float = 0.0
    inner_update: str = "sgd"
    inner_task: str = "mask"
    inner_from_outer: bool = False
    inner_feat: str = "off"
    inner_feat_weight: float = 1.0
    inner_update_frac: float = 1.0
    write: IN.WriteConfig = IN.WriteConfig()
    write_plan: Tuple[int, ...] = ()
    distill: bool = False
    distill_t_range: Tuple[float, float] = (0.1, 0.3)
    distill_weight: float = 1.0
    distill_topk: int = 64
    distill_meta: bool = True
    distill_warmup_steps: int = 0
    mtp: bool = False
    mtp_weight: float = 0.3
    inner_mtp_weight: float = 0.5
    inner_context_frac: float = 0.5
    no_write: bool = False
    write_off: bool = False
    aux_causal_weight: float = 0.0
    per_sequence: bool = False
    per_token: bool = False
    score_from_chunk: int = 0
    reread_chunks: int = 0
    window_drop: float = 0.0
    window_drop_until: int = 0
    self_prior: float = 0.0
    outer_views: int = 1
    fused_ce_block: int = 8192
    attn_chunk_batch: int = 2
    compute_dtype: str = "bfloat16"
    remat: bool = True                    # False: keep every activation (small models, tests)


def shift_slots(x: torch.Tensor, k: int):
    """``(y, valid)``: ``y[:, i] = x[:, i + k]`` along dim 1, the edge slot repeated where out of range."""
    C = x.shape[1]
    i = torch.arange(C, device=x.device)
    if k == 0:
        return x, torch.ones(C, dtype=torch.bool, device=x.device)
    if k > 0:
        return torch.cat([x[:, k:], x[:, -1:].expand(-1, k, *x.shape[2:])], 1), i <= C - 1 - k
    return torch.cat([x[:, :1].expand(-1, -k, *x.shape[2:]), x[:, :k]], 1), i >= -k


def make_feat_target(hc: torch.Tensor, tgt_idx: torch.Tensor) -> torch.Tensor:
    t = torch.gather(hc.float(), 1, tgt_idx.long()[..., None].expand(-1, -1, hc.shape[-1]))
    return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6)).detach()


def loss_fn(net: Net, batch: Batch, key: torch.Tensor, step: int, cfg: LossConfig):
    """Batch loss and diagnostics.  ``key``: ``[2]`` (training) or row-wise ``[B, 2]`` (evaluation)."""
    mc = net.cfg
    use_gdn = mc.memory == "gdn"
    asked_of_gdn = dict(inner_from_outer=cfg.inner_from_outer, write_off=cfg.write_off, distill=cfg.distill, mtp=cfg.mtp,
                        inner_feat=cfg.inner_feat != "off")
    if use_gdn:
        cfg = dc.replace(cfg, no_write=True)                 # the GDN state is written by its own recurrence, not by a gradient step
    VAL.check_options(cfg, mc, net.cw.has, use_gdn, asked_of_gdn)
    run_dev = net.p("final_norm.weight").device
    tp = net.tp_size
    if tp > 1:
        # the micro-batch belongs to the tensor-parallel group: this rank scores its own B / tp sequences
        if batch.position_ids is not None or cfg.inner_task == "split":
            raise NotImplementedError("tensor parallel: the sequences of a group must share their positions "
                                      "(no position_ids, no split inner task)")
        Bg = batch.input_ids.shape[0]
        if Bg % tp:
            raise ValueError(f"tensor parallel {tp}: the micro-batch of {Bg} sequences does not divide over the group")
        lo_, hi_ = net.tp.index * (Bg // tp), (net.tp.index + 1) * (Bg // tp)
        batch = Batch(*[None if x is None else x[lo_:hi_] for x in batch])
        key = key[lo_:hi_] if key.dim() == 2 else rng.fold_in(key, 7_000_001 + net.tp.index)
    train_graph = torch.is_grad_enabled()
    use_regions = cfg.remat and train_graph

    # ---- what the batch asks of the model: streams, positions, targets, masks, weights (ttt.plan), built on the run device
    plan = StreamPlan.build(batch, key, step, cfg, mc, run_dev)
    dev = run_dev
    B, T, nc, T0, n_rr = plan.B, plan.T, plan.nc, plan.T_data, plan.reread
    C, Wn, S, F_ = mc.chunk_size, mc.window_chunks, mc.suffix_len, mc.fast_len
    V, VO = cfg.inner_views, cfg.outer_views
    reach, sp_flags, read_own, own_inner = plan.reach, plan.self_prior_rows, plan.read_mask, plan.inner_own
    ids_streams, pos_k_streams, pos_q_streams, owns = plan.streams, plan.pos_k, plan.pos_q, plan.owns
    NS, n_inner, n_teacher = plan.NS, plan.n_inner, plan.n_teacher
    has_inner = n_inner > 0
    eff = plan.data_chunk
    s_S = 1 if cfg.inner_task == "causal" else 0
    s_T = 1 if cfg.outer_shift else 0

    # ---- segments
    n_seg_chunks = plan.segment_chunks
    n_seg = nc // n_seg_chunks
    T_seg = n_seg_chunks * C
    nkv, d = mc.num_key_value_heads // tp, mc.head_dim                       # this rank's KV heads
    Lp = mc.prefix_len
    cdt = net.dtype
    lr_now = IN.inner_lr(step, cfg.inner_lr, cfg.inner_lr_warmup_steps)
    distill_w = cfg.distill_weight
    if cfg.distill and cfg.distill_warmup_steps > 0:
        distill_w = cfg.distill_weight * min(1.0, step / cfg.distill_warmup_steps)
    clean_prime = (not cfg.write.plain) and cfg.write.kvb_weight > 0 and cfg.write.kvb_value == "clean"
    rb = mc.read_block
    clean_own = "full" if not rb else f"block:{rb}"
    create_graph = train_graph and cfg.second_order

    # ---- carries at the sequence start
    kvp = None                                                                      # per prefix layer (k, v) tails
    Bkv = B * tp                                                                    # windows hold every sequence of the TP group
    kvs = [(torch.zeros(Bkv, Wn * C, nkv, d, dtype=cdt, device=dev), torch.zeros(Bkv, Wn * C, nkv, d, dtype=cdt, device=dev))
           for _ in range(S)]
    if use_gdn:
        mem = torch.zeros(B, S, mc.gdn_heads, mc.gdn_head_dim, mc.gdn_head_dim, dtype=torch.float32, device=dev)
        W0 = None
    else:
        W0 = net.template_fast(B)
        if train_graph:
            W0 = [tuple(t.clone() for t in w) for w in W0]          # differentiable views of the template, materialised
        mem = None
    W = W0

    acc = dict(ce_sum=0.0, mask_count=0.0, ce2_sum=0.0, mask2_count=0.0, distill_mass=0.0, aux=0.0)
    inner_stats = IN.zero_stats(dev)
    plan_ce = torch.zeros(2, device=dev)
    ce_chunk = [None] * nc
    mask_chunk = [None] * nc
    ce_seq = torch.zeros(B, device=dev)
    mask_seq = torch.zeros(B, device=dev)
    ce_tok, mask_tok = [None] * nc, [None] * nc

    def run_segment(g, kvp, kvs, W, mem):
        """Prefix layers and the chunk scan of segment ``g`` from the carries ``(kvp, kvs, W | mem)``.  Returns the new carries and
        the segment's sums: ``sums [6]`` (ce, count, ce2, count2, distill mass, aux), inner stats, plan CE, per-sequence CE / count,
        per-chunk CE / count ``[ncs]`` and, with ``per_token``, the per-token arrays ``[ncs, B, C]``."""
        zero = torch.zeros((), dtype=torch.float32, device=dev)
        acc = dict(ce_sum=zero, mask_count=zero, ce2_sum=zero, mask2_count=zero, distill_mass=zero, aux=zero)
        inner_stats = IN.zero_stats(dev)
        plan_ce = torch.zeros(2, device=dev)
        ce_chunk, mask_chunk = [None] * n_seg_chunks, [None] * n_seg_chunks
        ce_seq = torch.zeros(B, device=dev)
        mask_seq = torch.zeros(B, device=dev)
        ce_tok, mask_tok = [None] * n_seg_chunks, [None] * n_seg_chunks
        sl = slice(g * T_seg, (g + 1) * T_seg)
        first = eff(g * n_seg_chunks)
        if n_rr and g * n_seg_chunks == n_rr:
            kvp = None                                                              # the second pass restarts the window
        # ---- prefix: all chunks of the segment, all streams, layer by layer
        h = net.embed_tokens(ids_streams[:, :, sl])                                 # [B, NS, T_seg, H]
        pk_seg = pos_k_streams[:, :, sl]
        pq_seg = None if pos_q_streams is None else pos_q_streams[:, :, sl]
        kvp_next = []
        for l in range(Lp):
            win = None if kvp is None else kvp[l]

            def layer_fn(h_in, *w, _l=l, _has=win is not None, _pk=pk_seg, _pq=pq_seg, _first=first):
                hh, tail = net.prefix_layer(_l, h_in, _pk, _pq, _first, (w[0], w[1]) if _has else None, owns, reach, rb)
                return hh, tail[0], tail[1]
            ins = (h,) + (tuple(win) if win is not None else ())
            with prof.range("prefix_layer.fwd"):
                h, tk, tv = region(layer_fn, ins, use_regions and l >= cfg.keep_prefix_layers, "prefix_layer.bwd")
            kvp_next.append((tk, tv))
        kvp = kvp_next if n_seg > 1 else None
        hch = h.unflatten(2, (n_seg_chunks, C))                                     # [B, NS, ncs, C, H]
        # every (stream, chunk) slice is taken from one unbind per axis: its backward stacks the slices' gradients in one pass,
        # where indexing ``hch[:, s, j]`` inside the loop would build a zero tensor of the whole segment per slice and add it up
        hsj = [hs.unbind(1) for hs in hch.unbind(1)]                                # hsj[s][j]: [B, C, H]

        # ---- suffix: chunk by chunk
        for j in range(n_seg_chunks):
            c = g * n_seg_chunks + j
            ho, hc = hsj[OUTER][j], hsj[CLEAN][j]
            hi = None
            if has_inner:
                hi = hsj[INNER][j] if V == 1 else torch.stack([hsj[INNER + v][j] for v in range(V)], 1)
            ht = hsj[INNER + n_inner][j] if cfg.distill else None
            hv = [hsj[NS - VO + 1 + k][j] for k in range(VO - 1)]
            consts = plan.at(c)
            nv = consts["nv"]

            n_kv = 2 * S
            mem_flat = [mem] if use_gdn else ([] if cfg.no_write else IN.flat(W))
            n_mem = len(mem_flat)
            dyn = [t for pair in kvs for t in pair] + mem_flat + [ho, hc] + ([hi] if hi is not None else []) \
                + ([ht] if ht is not None else []) + hv

            def step_fn(*ts, _k=consts, _n_kv=n_kv, _n_mem=n_mem, _has_hi=hi is not None, _has_ht=ht is not None):
                kv_l = [(ts[2 * i], ts[2 * i + 1]) for i in range(S)]
                o = _n_kv
                memv = ts[o:o + _n_mem]; o += _n_mem
                ho_, hc_ = ts[o], ts[o + 1]; o += 2
                hi_ = ts[o] if _has_hi else None; o += int(_has_hi)
                ht_ = ts[o] if _has_ht else None; o += int(_has_ht)
                hv_ = ts[o:]
                return _suffix_step(net, cfg, kv_l, memv, ho_, hc_, hi_, ht_, hv_, _k, W0, sp_flags, lr_now, distill_w,
                                    create_graph, own_inner, clean_own, read_own, clean_prime, s_S, s_T, B, C, S, use_gdn)
            with prof.range("suffix_step.fwd"):
                outs = region(step_fn, tuple(dyn), use_regions and j >= cfg.keep_suffix_chunks, "suffix_step.bwd")
            kvs = [(outs[2 * i], outs[2 * i + 1]) for i in range(S)]
            o = n_kv
            if use_gdn:
                mem = outs[o]; o += 1
            elif not cfg.no_write:
                W = IN.unflat(outs[o:o + n_mem]); o += n_mem
            ce_sum_c, mask_count_c, ce2_c, m2_c, dmass_c, st_c, plan_c, ce_seq_c, mask_seq_c, ce_tok_c, mask_tok_c, aux_c = outs[o:o + 12]
            acc["aux"] = acc["aux"] + aux_c
            acc["ce_sum"] = acc["ce_sum"] + ce_sum_c
            acc["mask_count"] = acc["mask_count"] + mask_count_c
            acc["ce2_sum"] = acc["ce2_sum"] + ce2_c
            acc["mask2_count"] = acc["mask2_count"] + m2_c
            acc["distill_mass"] = acc["distill_mass"] + dmass_c
            inner_stats = inner_stats + st_c.detach()
            plan_ce = plan_ce + plan_c.detach()
            ce_chunk[j], mask_chunk[j] = ce_sum_c.detach(), mask_count_c.detach()
            ce_seq, mask_seq = ce_seq + ce_seq_c.detach(), mask_seq + mask_seq_c.detach()
            ce_tok[j], mask_tok[j] = ce_tok_c, mask_tok_c
        as_f = lambda x: x.float() if torch.is_tensor(x) else torch.tensor(float(x), device=dev)
        sums = torch.stack([as_f(acc[k]).reshape(()) for k in ("ce_sum", "mask_count", "ce2_sum", "mask2_count", "distill_mass", "aux")])
        tok = (torch.stack(ce_tok), torch.stack(mask_tok)) if cfg.per_token else None
        return kvp, kvs, W, mem, (sums, inner_stats, plan_ce, ce_seq, mask_seq, torch.stack(ce_chunk), torch.stack(mask_chunk)), tok


    # Segments: with more than one segment under recompute regions, a segment is itself a region (nested around the per-layer
    # and per-chunk ones): the backward keeps one set of carries per segment and re-runs one segment at a time, so memory
    # does not grow with the number of chunks (reference chunk_scan.py:679-779, the outer scan over checkpointed segments).
    nest = use_regions and n_seg >= NEST_SEGMENTS_FROM
    zero = torch.zeros((), dtype=torch.float32, device=dev)
    acc = dict(ce_sum=zero, mask_count=zero, ce2_sum=zero, mask2_count=zero, distill_mass=zero, aux=zero)
    for g in range(n_seg):
        if not nest:
            kvp, kvs, W, mem, outs_g, tok_g = run_segment(g, kvp, kvs, W, mem)
        else:
            has_kvp = kvp is not None
            flat_in = ([t for pair in kvp for t in pair] if has_kvp else []) + [t for pair in kvs for t in pair] \
                + ([mem] if use_gdn else ([] if cfg.no_write else IN.flat(W)))

            def seg_fn(*ts, _g=g, _has_kvp=has_kvp):
                o = 0
                kvp_i = None
                if _has_kvp:
                    kvp_i = [(ts[2 * i], ts[2 * i + 1]) for i in range(Lp)]; o += 2 * Lp
                kvs_i = [(ts[o + 2 * i], ts[o + 2 * i + 1]) for i in range(S)]; o += 2 * S
                mem_i, W_i = mem, W
                if use_gdn:
                    mem_i = ts[o]
                elif not cfg.no_write:
                    W_i = IN.unflat(ts[o:])
                kvp_o, kvs_o, W_o, mem_o, outs_o, tok_o = run_segment(_g, kvp_i, kvs_i, W_i, mem_i)
                flat_out = [t for pair in kvp_o for t in pair] + [t for pair in kvs_o for t in pair] \
                    + ([mem_o] if use_gdn else ([] if cfg.no_write else IN.flat(W_o))) + list(outs_o) + (list(tok_o) if tok_o is not None else [])
                return tuple(flat_out)
            res = region(seg_fn, tuple(flat_in), True, "segment.bwd")
            o = 0
            kvp = [(res[2 * i], res[2 * i + 1]) for i in range(Lp)]; o += 2 * Lp
            kvs = [(res[o + 2 * i], res[o + 2 * i + 1]) for i in range(S)]; o += 2 * S
            if use_gdn:
                mem = res[o]; o += 1
            elif not cfg.no_write:
                W = IN.unflat(res[o:o + 3 * F_]); o += 3 * F_
            outs_g = res[o:o + 7]; o += 7
            tok_g = (res[o], res[o + 1]) if cfg.per_token else None
        sums_g, st_g, plan_g, ce_seq_g, mask_seq_g, ce_chunk_g, mask_chunk_g = outs_g
        for i, k in enumerate(("ce_sum", "mask_count", "ce2_sum", "mask2_count", "distill_mass", "aux")):
            acc[k] = acc[k] + sums_g[i]
        inner_stats = inner_stats + st_g.detach()
        plan_ce = plan_ce + plan_g.detach()
        ce_seq, mask_seq = ce_seq + ce_seq_g.detach(), mask_seq + mask_seq_g.detach()
        for j in range(n_seg_chunks):
            c = g * n_seg_chunks + j
            ce_chunk[c], mask_chunk[c] = ce_chunk_g[j].detach(), mask_chunk_g[j].detach()
            if tok_g is not None:
                ce_tok[c], mask_tok[c] = tok_g[0][j], tok_g[1][j]
        if cfg.truncate_fast_weight and not use_gdn and not cfg.no_write:
            W = [tuple(t.detach() for t in w) for w in W]

    main_loss = acc["ce_sum"] / (acc["mask_count"] + 1e-6)
    mtp_loss = acc["ce2_sum"] / (acc["mask2_count"] + 1e-6)
    loss = main_loss + cfg.mtp_weight * mtp_loss if cfg.mtp and cfg.mtp_weight > 0 else main_loss
    n_in = nc * B
    n_plan = sum(1 for k in cfg.write_plan[:nc] if k > 1)
    st = dict(zip(IN.STAT_NAMES, inner_stats.unbind(0)))
    if cfg.aux_causal_weight > 0:
        # the inner stream's mean CE (before any write) as an auxiliary objective of the shared weights
        loss = loss + cfg.aux_causal_weight * acc["aux"] / n_in
    if use_gdn:
        rms = torch.sqrt(mem.detach().pow(2).mean())
        drift = {"ttt_drift_rel": rms, "ttt_delta_norm": torch.sqrt(mem.detach().pow(2).sum()),
                 "ttt_init_norm": torch.zeros((), device=dev)}
    else:
        with torch.no_grad():
            drift = IN.drift_stats(W if not cfg.no_write else W0, W0)
    ce_chunk_t, mask_chunk_t = torch.stack(ce_chunk), torch.stack(mask_chunk)
    as_t = lambda x: x.detach() if torch.is_tensor(x) else torch.tensor(float(x), device=dev)
    stats = {
        **drift,
        "inner_loss": st["loss"] / n_in,
        **({"inner_plan_pre": plan_ce[0] / (B * n_plan), "inner_plan_post": plan_ce[1] / (B * n_plan)} if n_plan else {}),
        "inner_grad_norm": st["grad_norm"] / n_in, "inner_clipped_frac": st["clipped"] / n_in,
        "inner_feat": st["feat"] / n_in, "inner_distill": st["distill"] / n_in, "inner_mtp": st["mtp"] / n_in,
        "inner_kvb": st["kvb"] / n_in,
        "main_loss": as_t(main_loss), "mtp_loss": as_t(mtp_loss), "mtp_mask_count": as_t(acc["mask2_count"]),
        "distill_mass": as_t(acc["distill_mass"]) / n_in,
        "inner_lr": torch.tensor(lr_now, device=dev),
        "masked_frac": as_t(acc["mask_count"]) / (B * T0 * VO), "mask_count": as_t(acc["mask_count"]),
        "loss_by_chunk": (ce_chunk_t / (mask_chunk_t + 1e-6))[n_rr:], "mask_by_chunk": mask_chunk_t[n_rr:],
    }
    if cfg.per_sequence:
        stats["loss_by_seq"] = ce_seq / (mask_seq + 1e-6)
        stats["mask_by_seq"] = mask_seq
    if cfg.per_token:
        ce_flat = torch.stack(ce_tok, 1).reshape(B, T)[:, n_rr * C:]
        mask_flat = torch.stack(mask_tok, 1).reshape(B, T)[:, n_rr * C:]
        if cfg.outer_shift:
            ce_flat = torch.cat([torch.zeros_like(ce_flat[:, :1]), ce_flat[:, :-1]], 1)
            mask_flat = torch.cat([torch.zeros_like(mask_flat[:, :1]), mask_flat[:, :-1]], 1)
        stats["ce_by_token"], stats["mask_by_token"] = ce_flat, mask_flat
    return loss, stats


def _suffix_step(net: Net, cfg: LossConfig, kv, memv, ho, hc, hi, ht, hv, k, W0, sp_flags, lr_now, distill_w, create_graph,
                 own_inner, clean_own, read_own, clean_prime, s_S, s_T, B, C, S, use_gdn):
    """One chunk: streams B, C, A (reference chunk_scan.py:516-677).  Returns the flat tuple
    ``(kv_next..., memory..., ce_sum, mask_count, ce2_sum, mask2_count, distill_mass, inner stats [7], plan_ce [2],
    ce_seq [B], mask_seq [B], ce_tok, mask_tok, aux)``."""
    dev = ho.device
    # the outer gradient flows through the write only in a recorded pass; a region's first (unrecorded) run
    # takes the inner gradient at first order
    create_graph = create_graph and torch.is_grad_enabled()
    nv, p = k["nv"], k["p"]
    fb = cfg.fused_ce_block
    lm_w = net.lm_weight()
    zero = torch.zeros((), dtype=torch.float32, device=dev)
    W = None if (use_gdn or not memv) else IN.unflat(list(memv))
    if W is None and not use_gdn:
        W = W0                                                                       # no_write: the constant template
    mem = memv[0] if use_gdn else None
    Wc = None if use_gdn else IN.cast_fast(W, net.dtype)
    p_q_outer = (p + 1) if cfg.outer_shift else None
    rb = net.cfg.read_block

    def sf(h, Wm, pq=None, update=False, prime=False, own="full", own_mask=None, own_kv=None):
        if use_gdn:
            return net.suffix_forward(h, p, kv, None, nv, pos_q=pq, memory_state=Wm, update_memory=update, own=own,
                                      own_mask=own_mask, own_kv=own_kv)
        return net.suffix_forward(h, p, kv, Wm, nv, pos_q=pq, return_prime=prime, own=own, own_mask=own_mask, own_kv=own_kv)

    # T. distillation teacher (forward only) -> the write's soft targets
    extras = None
    distill_mass = zero
    if cfg.distill or cfg.mtp:
        soft_ids = soft_q = soft_mask = None
        if cfg.distill:
            with torch.no_grad():
                hT = sf(ht, Wc, p_q_outer)[0]
                ids_k, logp = CE.topk_logprobs(hT.reshape(B * C, -1), lm_w, cfg.distill_topk, fb or 8192)
                q_k = torch.exp(logp)
                mass = q_k.sum(-1).view(B, C).mean(1)
                distill_mass = mass.sum()
                ids_k, q_k = ids_k.view(B, C, -1), q_k.view(B, C, -1)
                soft_ids, ok_a = shift_slots(ids_k, s_S - s_T)
                soft_q, _ = shift_slots(q_k, s_S - s_T)
                masked_t, ok_b = shift_slots(k["mt"], s_S)
                first = k["im"].reshape(B, -1, C)[:, 0]
                soft_mask = (masked_t & (first > 0) & (ok_a & ok_b)[None]).float()
        extras = IN.InnerExtras(soft_ids, soft_q, soft_mask, k["mtp_t"], k["mtp_m"])

    # B. clean -> next KV window; with memory gdn also the state written from this chunk.  When the read (A) uses the very
    # memory the clean pass uses (no self-prior rows, no sub-block read, no GDN state), A, its extra views and B go through
    # the suffix together (Net.suffix_forward_streams): the same arithmetic on two or more times the rows per launch.
    together = (STREAMS_TOGETHER and not use_gdn and sp_flags is None and not rb and read_own is None and Wc is not None
                and net.tp_size == 1)
    hA = None
    hV_together = []
    if together:
        with prof.range("step.AB_together"):
            hs = torch.stack([ho, hc] + list(hv), dim=1)                                  # OUTER = 0, CLEAN = 1, extra outer views
            n_s = hs.shape[1]
            pos_s = p[:, None].expand(B, n_s, C)
            pq = p if p_q_outer is None else p_q_outer
            pos_q_s = torch.stack([pq, p] + [pq] * len(hv), dim=1)
            owns_s = ["full", clean_own] + ["full"] * len(hv)
            hn_s, own_kv_s, extra_s = net.suffix_forward_streams(hs, pos_s, pos_q_s, kv, Wc, nv, owns_s, return_prime=clean_prime)
        hA = hn_s[:, 0]
        hV_together = [hn_s[:, 2 + i] for i in range(len(hv))]
        resB = (hn_s[:, 1], own_kv_s, extra_s)
    else:
        with prof.range("step.B_clean"):
            resB = sf(hc, mem if use_gdn else Wc, update=use_gdn, prime=clean_prime, own=clean_own)
    own_kv = resB[1]
    kv_next = [(torch.cat([ck[:, C:], ok], dim=1), torch.cat([cv[:, C:], ov], dim=1)) if ck.shape[1] else (ck, cv)
               for (ck, cv), (ok, ov) in zip(kv, own_kv)]
    mem_next = None
    if use_gdn:
        mem_next = resB[2] if lr_now > 0 else mem

    # C. the write
    plan_ce = torch.zeros(2, device=dev)
    st = IN.zero_stats(dev)
    aux_term = None
    if cfg.no_write:
        W_next = W
    elif cfg.write_off:
        pq = None if cfg.inner_task == "mask" else k["p_q"]
        obj, terms = IN.inner_objective(W, net, hi, k["tgt"], k["im"], kv, k["p_in"], nv, fb, pos_q=pq, own=own_inner)
        W_next = W
        st = st.clone(); st[0] = terms[0]
        aux_term = obj
    else:
        feat_tgt = make_feat_target(hc, k["ti"]) if cfg.inner_feat != "off" else None
        V = cfg.inner_views
        if cfg.inner_from_outer:
            W_next, st = IN.inner_update(W, net, ho, k["tok"], k["wgt"].float(), kv, p, nv, lr_now, cfg.inner_clip, fb,
                                         cfg.inner_update, create_graph=create_graph, h_clean=hc, pos_q=p_q_outer,
                                         frac=cfg.inner_update_frac)
        elif V > 1 and cfg.inner_views_sequential:
            W_next, sts = W, []
            for v in range(V):
                W_next, st_v = IN.inner_update(W_next, net, hi[:, v], k["tgt"], k["im"][:, v], kv, k["p_in"], nv, lr_now / V,
                                               cfg.inner_clip / V, fb, cfg.inner_update, create_graph=create_graph,
                                               h_clean=hc, feat_tgt=feat_tgt, feat_mode=cfg.inner_feat,
                                               feat_weight=cfg.inner_feat_weight, frac=cfg.inner_update_frac)
                sts.append(st_v)
            st = torch.stack(sts).mean(0)
        elif not cfg.write.plain:
            W_next, st = IN.write_chunk(W, net, hi, k["tgt"], k["im"], kv, k["p_in"], nv, lr_now, cfg.inner_clip, fb,
                                        cfg.inner_update, hc, k["p_q"], own_inner, cfg.write, create_graph=create_graph,
                                        W0=W0, kvb_src=resB[2][0] if clean_prime else None)
        else:
            def plain_step(w, cg=create_graph):
                return IN.inner_update(w, net, hi, k["tgt"], k["im"], kv, k["p_in"], nv, lr_now, cfg.inner_clip, fb,
                                       cfg.inner_update, create_graph=cg, h_clean=hc,
                                       pos_q=None if cfg.inner_task == "mask" else k["p_q"], own=own_inner,
                                       feat_tgt=feat_tgt, feat_mode=cfg.inner_feat, feat_weight=cfg.inner_feat_weight,
                                       frac=cfg.inner_update_frac, extras=extras, distill_weight=distill_w,
                                       mtp_weight=cfg.inner_mtp_weight, distill_meta=cfg.distill_meta,
                                       W_cast=Wc if w is W else None)
            if cfg.write_plan:
                k_c = k["k_c"]
                W1, st = plain_step(W)
                Wk = W1
                for _ in range(1, max(k_c, 1)):
                    Wk = plain_step(Wk)[0]
                W_next = Wk if k_c > 0 else W
                if k_c > 1:
                    post = plain_step(Wk, False)[1][0]
                    plan_ce = torch.stack([st[0], post])
            else:
                with prof.range("step.C_write"):
                    W_next, st = plain_step(W)
        if not cfg.second_order:
            W_next = [tuple(t.detach() for t in w) for w in W_next]
    if cfg.aux_causal_weight > 0 and not cfg.no_write and aux_term is None:
        pq = None if cfg.inner_task == "mask" else k["p_q"]
        aux_term, _ = IN.inner_objective(W, net, hi, k["tgt"], k["im"], kv, k["p_in"], nv, fb, pos_q=pq, own=own_inner)

    # A. the read: the memory as it was before this chunk's write, or (self-prior rows) after it
    if use_gdn:
        W_read = mem
    elif sp_flags is None:
        W_read = Wc
    else:
        sel = [tuple(torch.where(sp_flags.view(B, 1, 1), b_, a_) for a_, b_ in zip(wa, wb)) for wa, wb in zip(W, W_next)]
        W_read = IN.cast_fast(sel, net.dtype)
    read_kv = own_kv if rb else None
    if hA is None:
        with prof.range("step.A_read"):
            hA = sf(ho, W_read, p_q_outer, own="full", own_mask=read_own, own_kv=read_kv)[0]
    tok, wgt, tm = k["tok"], k["wgt"], k["tm"]
    ce_seq = mask_seq = torch.zeros(B, device=dev)
    if cfg.per_sequence:
        ce_seq = torch.stack([CE.weighted_ce(hA[b], lm_w, tok[b], wgt[b].float(), fb) for b in range(B)])
        ce_sum = ce_seq.sum()
        mask_seq = tm.float().sum(1)
    else:
        with prof.range("step.A_ce"):
            ce_sum = CE.weighted_ce(hA.reshape(B * C, -1), lm_w, tok.reshape(-1), wgt.reshape(-1).float(), fb)
    ce2_sum = mask2 = zero
    if cfg.mtp and cfg.mtp_weight > 0:
        h2 = Fn.linear(hA, net.p("mtp_head.weight"))
        ce2_sum = CE.weighted_ce(h2.reshape(B * C, -1), lm_w, k["tok2"].reshape(-1), k["wgt2"].reshape(-1).float(), fb)
        mask2 = k["tm2"].float().sum()
    mask_count = tm.float().sum()
    for i, hvi in enumerate(hv):
        hV = hV_together[i] if hV_together else sf(hvi, W_read, p_q_outer)[0]
        ce_sum = ce_sum + CE.weighted_ce(hV.reshape(B * C, -1), lm_w, tok.reshape(-1), k["wv"][i].reshape(-1).float(), fb)
        mask_count = mask_count + k["tmv"][i].float().sum()
    if cfg.per_token:
        ce_tok = CE.per_token_ce(hA.reshape(B * C, -1).detach(), lm_w.detach(), tok.reshape(-1), fb or 8192).view(B, C)
        mask_tok = tm.float()
    else:
        ce_tok = mask_tok = torch.zeros(1, device=dev)
    aux_out = aux_term if (aux_term is not None and cfg.aux_causal_weight > 0) else zero
    outs = [t for pair in kv_next for t in pair]
    if use_gdn:
        outs.append(mem_next)
    elif not cfg.no_write:
        outs += IN.flat(W_next)
    outs += [ce_sum.float(), mask_count, ce2_sum.float() if torch.is_tensor(ce2_sum) else zero, mask2, distill_mass,
             st, plan_ce, ce_seq, mask_seq, ce_tok, mask_tok, aux_out.float()]
    return tuple(outs)
