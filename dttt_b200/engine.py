"""The training / evaluation engine: parameters, optimiser and one public ``train_step``.

``Engine`` is what ``dttt_b200.train``, ``bench.py`` and the tools drive:

    eng = Engine(model_cfg, train_cfg, mesh)          # builds (or later loads) the sharded parameters
    metrics = eng.train_step(batch, step)             # batch: host or device token ids, [B_local, T] or [N, B_local, T]

One optimiser step (reference ``src/ttt/train.py:713-794``): for each micro-batch the loss
``sum(ce) / sum(mask)`` is back-propagated weighted by its mask count, gradients accumulate in the f32
buffers, the sum is divided by the global mask count of the step (over micro-batches and data ranks:
exactly the gradient of one large batch), reduced over the data ranks, clipped and applied by AdamW on
the parameter shards; then the compute copies are refreshed.  Step keys are stateless,
``fold_in(key(seed), step)`` then split per micro-batch and folded with the data rank, so a resumed run
draws the masks the uninterrupted run drew (``train.py:1123-1126``).
"""
from __future__ import annotations

import dataclasses as dc
import math
from typing import Dict, Optional

import torch

from .models.blocks import Net
from .models.params import count_params, init_params, param_spec
from .optim import ShardedAdamW
from .parallel.mesh import Mesh
from .parallel.store import ComputeWeights, ParamStore
from .schema import ModelConfig, TrainConfig
from .ttt.inner import WriteConfig
from .ttt.scan import Batch, LossConfig, loss_fn
from .utils import prof, rng

NORM_STATS = ("ttt_delta_norm", "ttt_init_norm", "ttt_drift_rel")


def write_config(cfg: TrainConfig) -> WriteConfig:
    return WriteConfig(subchunks=cfg.inner_subchunks, subchunk_scale=cfg.inner_subchunk_scale,
                       surprise_gamma=cfg.inner_surprise_gamma, kvb_weight=cfg.inner_kvb_weight,
                       kvb_value=cfg.inner_kvb_value, fast_frac=cfg.inner_fast_frac,
                       fast_lr_scale=cfg.inner_fast_lr_scale, fast_decay=cfg.inner_fast_decay,
                       steps=cfg.inner_write_steps, norm_alpha=cfg.inner_norm_alpha, norm_cap=cfg.inner_norm_cap)


def loss_config(cfg: TrainConfig) -> LossConfig:
    """The flat run configuration as a ``LossConfig`` (reference train.py:244-264)."""
    return LossConfig(
        time_reweighting=cfg.time_reweighting, cart_p=cfg.cart_p, cart_window=cfg.cart_window,
        outer_t=cfg.outer_t, outer_shift=cfg.outer_shift, inner_lr=cfg.inner_lr, inner_clip=cfg.inner_clip,
        inner_lr_warmup_steps=cfg.inner_lr_warmup_steps, inner_mask_range=tuple(cfg.inner_mask_range),
        inner_mask_ratio=cfg.inner_mask_ratio, second_order=cfg.second_order, remat_levels=cfg.remat_levels,
        remat_prefix=cfg.remat_prefix, prefix_remat_levels=cfg.prefix_remat_levels, keep_prefix_layers=cfg.keep_prefix_layers, keep_suffix_chunks=cfg.keep_suffix_chunks,
        segment_chunks=cfg.segment_chunks,
        truncate_fast_weight=cfg.truncate_fast_weight, inner_views=cfg.inner_views, inner_view_mode=cfg.inner_view_mode,
        inner_views_sequential=cfg.inner_views_sequential, inner_cart=cfg.inner_cart, inner_mask_span=cfg.inner_mask_span,
        inner_update=cfg.inner_update, no_write=cfg.no_write, inner_task=cfg.inner_task,
        inner_context_frac=1.0 - cfg.inner_target_frac, inner_from_outer=cfg.inner_from_outer, inner_feat=cfg.inner_feat,
        inner_feat_weight=cfg.inner_feat_weight, inner_update_frac=cfg.inner_update_frac, distill=cfg.distill,
        distill_t_range=tuple(cfg.distill_t_range), distill_weight=cfg.distill_weight, distill_topk=cfg.distill_topk,
        distill_meta=cfg.distill_meta, distill_warmup_steps=cfg.distill_warmup_steps, mtp=cfg.mtp, mtp_weight=cfg.mtp_weight,
        inner_mtp_weight=cfg.inner_mtp_weight, write_off=cfg.write_off, aux_causal_weight=cfg.aux_causal_weight,
        write=write_config(cfg), window_drop=cfg.window_drop, window_drop_until=int(cfg.window_drop_frac * cfg.steps),
        self_prior=cfg.self_prior, outer_views=cfg.outer_views, fused_ce_block=cfg.fused_ce_block,
        attn_chunk_batch=cfg.attn_chunk_batch, compute_dtype=cfg.compute_dtype)


def resolve_keep(tc: TrainConfig, mc: ModelConfig, free_bytes: float, seqs_per_pass: int) -> TrainConfig:
    """``keep_prefix_layers`` / ``keep_suffix_chunks`` below zero mean "as many as fit": fill them in from the memory model
    (``tools.memory_model``) and the bytes free on the device after the parameters are in place.  What must stay free besides
    the kept graphs: the region inputs, the transients of the pass in flight (about 19 GB per 16k tokens for the 1B model,
    scaled by width) and a safety margin.  Chunk steps are kept before prefix layers (they save more time per byte: a kept
    chunk step also drops its unrecorded first pass)."""
    if tc.keep_prefix_layers >= 0 and tc.keep_suffix_chunks >= 0:
        return tc
    import dataclasses as dc
    from .tools import memory_model as MM
    c = dc.asdict(mc)
    c.setdefault("ttt_intermediate_size", None)
    seq_len, n_prefix = tc.seq_len, mc.num_hidden_layers - mc.suffix_len
    per_segment = tc.segment_chunks or max(1, seq_len // mc.chunk_size)
    tokens = seqs_per_pass * seq_len
    carried = MM.carry_bytes(c)
    regions = seqs_per_pass * (n_prefix * 3 * seq_len * mc.hidden_size * 2 + (seq_len // mc.chunk_size) * (carried["fast_weight"] + carried["kv"]))
    transients = 19e9 * tokens / 16384 * (mc.hidden_size / 2048)
    budget = free_bytes - regions - transients - 15e9
    # a chunk step of the method arm (normalised write, self-prior: `write_chunk`) records about twice the graph of the plain
    # step the memory model describes (measured at 32k: 13.1 GiB per kept step and segment against 6.8)
    step_factor = 1.0 if loss_config(tc).write.plain else 1.95
    kept = lambda layers, chunks: seqs_per_pass * (MM.kept_bytes(c, seq_len, layers, 0, tc.segment_chunks)
                                                   + step_factor * MM.kept_bytes(c, seq_len, 0, chunks, tc.segment_chunks))
    chunks = tc.keep_suffix_chunks
    if chunks < 0:
        chunks = max((k for k in range(per_segment + 1) if kept(0, k) <= budget), default=0)
    layers = tc.keep_prefix_layers
    if layers < 0:
        layers = max((k for k in range(n_prefix + 1) if kept(k, chunks) <= budget), default=0)
    return tc.replace(keep_prefix_layers=layers, keep_suffix_chunks=chunks)


def torch_dtype(name: str) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[name]


class Engine:
    def __init__(self, model_cfg: ModelConfig, train_cfg: TrainConfig, mesh: Optional[Mesh] = None,
                 device: Optional[torch.device] = None, init: bool = True, trainable: bool = True):
        self.mc, self.tc = model_cfg, train_cfg
        self.mesh = mesh or Mesh(device=device or torch.device("cuda" if torch.cuda.is_available() else "cpu"))
        self.device = device or self.mesh.device
        self.dtype = torch_dtype(train_cfg.compute_dtype)
        tp = self.mesh.tp
        self.spec = param_spec(model_cfg, tp)
        self.tp_ctx = None
        if tp > 1:
            from .parallel.tp import TPContext
            self.tp_ctx = TPContext(self.mesh.tp_group, tp, self.mesh.tp_index, self.device)
        self.store = ParamStore(self.spec, self.mesh, self.dtype, self.device, trainable=trainable,
                                fused_comm=train_cfg.fused_comm, tp_ctx=self.tp_ctx)
        self.n_params = count_params(model_cfg)
        if train_cfg.shard_compute and trainable:
            self.store.enable_shard_compute([n for n in self.spec if n.startswith("prefix.") and n.endswith(".weight")])
        if init:
            self.init_weights(train_cfg.seed)
        self.opt = None
        if trainable:
            c = train_cfg
            self.opt = ShardedAdamW(self.store, c.lr, c.end_lr, c.warmup_steps, c.decay_start, c.decay_end, c.weight_decay,
                                    c.grad_clip, c.adam_b1, c.adam_b2, no_decay_pattern=c.no_decay_pattern,
                                    fast_weight_lr_scale=c.fast_weight_lr_scale)
        if train_cfg.keep_prefix_layers < 0 or train_cfg.keep_suffix_chunks < 0:
            free = float(torch.cuda.mem_get_info(self.device)[0]) if self.device.type == "cuda" else 0.0
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                # every rank must resolve the same numbers: under tensor parallelism a rank that recomputes a region issues
                # collectives its peers would not
                t = torch.tensor([free], dtype=torch.float64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                free = float(t.item())
            train_cfg = self.tc = resolve_keep(train_cfg, model_cfg, free, max(1, train_cfg.batch_size // self.mesh.batch_ranks))
        self.lcfg = loss_config(train_cfg)
        self.key = rng.key(train_cfg.seed)
        self.overflow = 0

    # ---- parameters
    def init_weights(self, seed: int) -> None:
        gen_dev = self.device
        base = rng.key(seed, gen_dev)
        from .models import params as P
        for name, value in P.iter_init(self.mc, seed, gen_dev, self.mesh.tp, self.mesh.tp_index):
            self.store.load_full(name, value)
            del value

    def net(self, train: bool = True) -> Net:
        return Net(self.mc, ComputeWeights(self.store, train=train), self.tp_ctx)

    # ---- batches
    def to_device(self, ids) -> torch.Tensor:
        t = torch.as_tensor(ids)
        if t.device != self.device:
            t = t.to(self.device, non_blocking=True)
        return t.long()

    def step_key(self, step: int, micro: int = 0, n_micro: int = 1) -> torch.Tensor:
        k = rng.fold_in(self.key, step)
        if n_micro > 1:
            k = rng.split(k, n_micro)[micro]
        if self.mesh.batch_ranks > 1:
            k = rng.fold_in(k, 1_000_003 + self.mesh.batch_index)
        return k

    # ---- one optimiser step
    def train_step(self, batch, step: int, lcfg: Optional[LossConfig] = None) -> Dict[str, float]:
        """``batch``: token ids ``[B, T]`` or ``[N, B, T]`` (N micro-batches), or a ``Batch`` / list of them."""
        lcfg = lcfg or self.lcfg
        micro = self._as_micro_batches(batch)
        N = len(micro)
        st = self.store
        st.zero_grad()
        wsum = torch.zeros((), dtype=torch.float32, device=self.device)
        loss_w = torch.zeros((), dtype=torch.float32, device=self.device)
        sum_stats: Dict[str, torch.Tensor] = {}
        # Gradient noise scale from the micro-batches (reference train.py:767-779): every micro-batch's own gradient norm is
        # needed, so each one lands in the (zeroed) gradient buffers and is then moved into an accumulator.
        noise = N > 1 and self.mesh.tp == 1
        micro_sq = torch.zeros((), dtype=torch.float32, device=self.device)
        if noise:
            if getattr(self, "_grad_acc", None) is None:
                self._grad_acc = {k: torch.zeros_like(v) for k, v in st.grad.items()}
            for v in self._grad_acc.values():
                v.zero_()
        for i, b in enumerate(micro):
            cw = ComputeWeights(st, train=True)
            net = Net(self.mc, cw, self.tp_ctx)
            loss, stats = loss_fn(net, b, self.step_key(step, i, N), step, lcfg)
            w = stats["mask_count"].detach() + 1e-6
            (loss * w).backward()
            cw.fold_grads()
            if noise:
                sq = sum(g.float().pow(2).sum() for g in st.grad.values())
                micro_sq += sq / (w * w)                       # the buffers hold w_m * grad(ce_m / n_m)
                for k, g in st.grad.items():
                    self._grad_acc[k] += g
                    g.zero_()
            wsum += w
            loss_w += loss.detach().float() * w
            for k, v in stats.items():
                if v.dim() == 0:
                    if k == "main_loss":
                        v = v * w
                    elif k == "mtp_loss":
                        v = v * (stats["mtp_mask_count"] + 1e-6)
                    elif k in NORM_STATS:
                        v = v.pow(2)
                    sum_stats[k] = sum_stats.get(k, 0) + v.detach().float()
            del cw, net, loss
            if self.tp_ctx is not None:
                self.tp_ctx.last_gather = None                 # the shared gather of the last layer input goes with the pass
        # one global normaliser: micro-batches and data ranks together are one batch
        if noise:
            for k, g in st.grad.items():
                g.copy_(self._grad_acc[k])
        red = torch.stack([wsum, loss_w, micro_sq])
        red = st.all_reduce_scalar(red)
        wsum_g, loss_g, micro_sq_g = red[0].item(), red[1].item(), red[2].item()
        with prof.range("reduce_grads"):
            st.reduce_grads()
        with prof.range("optimizer"):
            om = self.opt.step(grad_scale=wsum_g)
        with prof.range("sync_compute"):
            if not self.opt.wrote_compute:
                st.sync_compute()
        from .ops import _lib
        if self.device.type == "cuda":
            _lib.check_status(self.device)
        out = {"loss": loss_g / wsum_g, **om}
        if noise:
            # E|g_b|^2 = |G|^2 + tr(S) / b: the per-rank micro-batches (b_s sequences) and the whole step (b_l) give both
            R = self.mesh.batch_ranks
            b_s = float(micro[0].input_ids.shape[0])
            b_l = b_s * N * R
            m_sq, f_sq = micro_sq_g / (N * R), om["grad_norm"] ** 2
            tr_sigma = (m_sq - f_sq) / (1.0 / b_s - 1.0 / b_l)
            signal = (b_l * f_sq - b_s * m_sq) / (b_l - b_s)
            out["grad_norm_micro"] = math.sqrt(max(m_sq, 0.0))
            out["grad_noise_scale"] = tr_sigma / signal if signal > 0 else float("nan")
        host = {k: float(v) for k, v in sum_stats.items()}
        for k, v in host.items():
            out[k] = v / N
        out["mask_count"] = host.get("mask_count", 0.0)
        out["mtp_mask_count"] = host.get("mtp_mask_count", 0.0)
        out["main_loss"] = host.get("main_loss", 0.0) / float(wsum)
        out["mtp_loss"] = host.get("mtp_loss", 0.0) / (host.get("mtp_mask_count", 0.0) + N * 1e-6)
        d, i0 = math.sqrt(host.get("ttt_delta_norm", 0.0)), math.sqrt(host.get("ttt_init_norm", 0.0))
        out["ttt_delta_norm"], out["ttt_init_norm"] = d, i0
        out["ttt_drift_rel"] = d / (i0 + 1e-12) if i0 > 0 else math.sqrt(host.get("ttt_drift_rel", 0.0) / N)
        self.overflow += int(not om["finite"])
        out["overflow"] = self.overflow
        return out

    def grad_of(self, batch: Batch, key: torch.Tensor, step: int, lcfg: Optional[LossConfig] = None, weight: str = "sum"):
        """Gradient of one batch's loss into ``store.grad`` (no reduction, no optimiser step): ``weight = "sum"`` scales the
        mean loss by its scored-token count (a sequence's share of a batch gradient), ``"mean"`` leaves it.  Returns
        ``(loss, scored tokens)``.  Analysis tools use this (gradient noise, Jacobian probes)."""
        lcfg = lcfg or self.lcfg
        st = self.store
        st.zero_grad()
        cw = ComputeWeights(st, train=True)
        net = Net(self.mc, cw, self.tp_ctx)
        loss, stats = loss_fn(net, batch, key, step, lcfg)
        w = stats["mask_count"].detach() + 1e-6
        (loss * w if weight == "sum" else loss).backward()
        cw.fold_grads()
        return float(loss.detach()), float(w)

    def _as_micro_batches(self, batch):
        if isinstance(batch, Batch):
            return [batch]
        if isinstance(batch, (list, tuple)) and batch and isinstance(batch[0], Batch):
            return list(batch)
        ids = self.to_device(batch)
        if ids.dim() == 2:
            return [Batch(ids)]
        return [Batch(ids[i]) for i in range(ids.shape[0])]

    @torch.no_grad()
    def eval_step(self, batch: Batch, key: torch.Tensor, step: int, lcfg: LossConfig):
        net = self.net(train=False)
        loss, stats = loss_fn(net, batch, key, step, lcfg)
        if self.mesh.tp > 1:
            loss, stats = self._merge_over_tp(loss, stats)
        return loss, stats

    def _merge_over_tp(self, loss: torch.Tensor, stats: Dict[str, torch.Tensor]):
        """Under tensor parallelism every rank scored its own sequences of the group's batch: put the per-sequence arrays back
        in batch order, add the counts, and average the rest by scored tokens, so callers see the group's batch."""
        import torch.distributed as dist
        g, tp = self.mesh.tp_group, self.mesh.tp
        w = stats["mask_count"].detach().float() + 1e-6
        wsum = w.clone()
        dist.all_reduce(wsum, group=g)

        def cat(x):
            parts = [torch.empty_like(x) for _ in range(tp)]
            dist.all_gather(parts, x.contiguous(), group=g)
            return torch.cat(parts, 0)

        def wmean(x, wl, wt):
            y = x.detach().float() * wl
            dist.all_reduce(y, group=g)
            return y / wt
        out = {}
        mbc = stats.get("mask_by_chunk")
        mbc_sum = None
        if mbc is not None:
            mbc_sum = mbc.detach().float().clone()
            dist.all_reduce(mbc_sum, group=g)
        for k, v in stats.items():
            if k in ("loss_by_seq", "mask_by_seq", "ce_by_token", "mask_by_token"):
                out[k] = cat(v)
            elif k in ("mask_count", "mtp_mask_count", "mask_by_chunk"):
                y = v.detach().float().clone()
                dist.all_reduce(y, group=g)
                out[k] = y
            elif k == "loss_by_chunk" and mbc is not None:
                out[k] = wmean(v, mbc.detach().float() + 1e-6, mbc_sum + tp * 1e-6)
            elif torch.is_tensor(v) and v.is_floating_point():
                out[k] = wmean(v, w, wsum)
            else:
                out[k] = v
        return wmean(loss, w, wsum), out
