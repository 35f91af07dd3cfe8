"""Held-out evaluation: loss per source, the write ablation, loss by chunk position, token-class probes, planted recall.

``evaluate`` scores the held-out tail of every source under *fixed, stratified* noise: held-out sequence ``j`` gets the masking rate
``(perm[j] + u_j) / n`` and its own row key, both functions of ``eval_seed`` and ``j`` alone, so the figures do not depend on batch
shape or rank count and are paired across checkpoints and runs.  Every batch runs once per programme: inner-rate scale 1 is the
trained setting, scale 0 its no-write twin, and ``gain = loss(0) - loss(1)`` is the write ablation, reported overall, per source,
per chunk position and per "tokens of the document beyond the window" bucket, with the paired standard error over sequences.
Per-sequence results are written to ``<log_dir>/eval_<step>.npz`` for the offline tools.

The record keys (``eval/...``), the log lines and the ``.npz`` fields are those of the reference's evaluation
(src/ttt/train.py:277-672), so its readers and comparison tools work on these outputs.  The work is split into small pieces here:
``_Tally`` (means over optimiser-step batches), ``_SourceRun`` (all batches of one source), ``_ProbeTable`` (class tables of the
probes) and the report functions.
"""
from __future__ import annotations

import dataclasses as dc
import os
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..schema import ModelConfig, TrainConfig
from ..utils import rng
from . import probes as PR

# (low, high, name): tokens of the sequence's first document that lie beyond the attention window
BUCKETS = ((0, 1, "0"), (1, 1024, "1-1K"), (1024, 3072, "1-3K"), (3072, 1 << 62, ">=3K"))
_TINY = 1e-6


def _label(scale) -> str:
    return scale if isinstance(scale, str) else f"x{scale:g}"


def _stderr(values: np.ndarray) -> float:
    return float(values.std(ddof=1) / np.sqrt(len(values))) if len(values) > 1 else float("nan")


def _output_dir(cfg: TrainConfig) -> str:
    return cfg.log_dir or os.environ.get("DTTT_LOG_DIR", os.environ.get("TTT_LOG_DIR", ""))


def _bucket_of(beyond: int) -> str:
    for low, high, name in BUCKETS:
        if low <= beyond < high:
            return name
    raise ValueError(beyond)


def row_keys(eval_seed: int, j_indices: Sequence[int]):
    """Per held-out sequence ``(u [n] in [0, 1), row keys [n, 2])``: ``fold_in(key(eval_seed), j)`` split in two."""
    folded = rng.fold_in(rng.key(eval_seed).unsqueeze(0).expand(len(j_indices), 2), torch.as_tensor(list(j_indices), dtype=torch.int64))
    halves = rng.split(folded, 2)
    return rng.uniform(halves[:, 0], ()).numpy(), halves[:, 1]


# ------------------------------------------------------------------------------------------------------------ accumulation
class _Tally:
    """Loss of one programme on one source: micro-batches are pooled (token-weighted) into optimiser-step batches, whose means are
    then averaged; the same per chunk position."""

    def __init__(self, n_chunks: int, accum: int):
        self.accum, self.n_chunks = accum, n_chunks
        self.mean, self.by_chunk = 0.0, np.zeros(n_chunks)
        self._seen = 0
        self._reset()

    def _reset(self) -> None:
        self._loss, self._count = 0.0, 0.0
        self._chunk_loss, self._chunk_count = np.zeros(self.n_chunks), np.zeros(self.n_chunks)

    def add(self, loss_times_count: float, count: float, chunk_loss_times_count: np.ndarray, chunk_count: np.ndarray) -> None:
        self._loss += loss_times_count
        self._count += count
        self._chunk_loss += chunk_loss_times_count
        self._chunk_count += chunk_count
        self._seen += 1
        if self._seen % self.accum == 0:
            self.mean += self._loss / max(self._count, _TINY)
            self.by_chunk += self._chunk_loss / np.maximum(self._chunk_count, _TINY)
            self._reset()

    def finish(self, n_step_batches: int) -> None:
        self.mean /= n_step_batches
        self.by_chunk = self.by_chunk / n_step_batches


@dc.dataclass
class _Records:
    """What goes into ``eval_<step>.npz``: one entry per held-out sequence of this rank."""
    sources: List[str] = dc.field(default_factory=list)
    doc_ids: List[np.ndarray] = dc.field(default_factory=list)
    doc_lens: List[np.ndarray] = dc.field(default_factory=list)
    beyond: List[np.ndarray] = dc.field(default_factory=list)
    gain: List[np.ndarray] = dc.field(default_factory=list)
    mask: List[np.ndarray] = dc.field(default_factory=list)
    loss: Dict = dc.field(default_factory=dict)

    def save(self, path: str) -> None:
        joined = lambda parts: np.concatenate(parts) if parts else np.array([], dtype=np.int64)
        fields = {"sources": np.array(self.sources), "doc_ids": joined(self.doc_ids), "doc_lens": joined(self.doc_lens),
                  "beyond": joined(self.beyond)}
        for scale, parts in self.loss.items():
            if parts:
                fields[f"loss_{scale}"] = np.concatenate(parts)
        for name in ("gain", "mask"):
            if getattr(self, name):
                fields[name] = np.concatenate(getattr(self, name))
        np.savez_compressed(path, **fields)


class _SourceRun:
    """All held-out batches of one source under every programme."""

    def __init__(self, ctx: "_EvalContext", sampler, index: int, source, weighted: bool):
        self.ctx, self.sampler, self.index, self.source, self.weighted = ctx, sampler, index, source, weighted
        self.tally = {sc: _Tally(ctx.n_chunks, sampler.accum) for sc in ctx.scales}
        self.gain: List[np.ndarray] = []                 # per sequence: loss(ablation) - loss(1)
        self.reread_gain: List[np.ndarray] = []          # per sequence: loss(1) - loss(reread)
        n_step_batches = sampler.eval_step_batches(index)
        if weighted:
            n_step_batches = min(ctx.cfg.eval_batches, n_step_batches)
        self.n_batches = sampler.accum * n_step_batches
        n_held = max(1, int(sampler.n_eval_seq[index]))
        self._n_held = n_held
        self._strata = np.random.default_rng(ctx.cfg.eval_seed).permutation(n_held)

    def _batch(self, k: int):
        s = self.sampler
        first = k * s.G + s.rank * s.local
        rows = [(first + j) % self._n_held for j in range(s.local)]
        u, keys = row_keys(self.ctx.cfg.eval_seed, rows)
        rate = ((self._strata[rows].astype(np.float32) + u) / float(self._n_held)).astype(np.float32)
        return self.ctx.make_batch(s.eval_batch(self.index, k), outer_t=rate), keys

    def run(self) -> None:
        ctx, s = self.ctx, self.sampler
        base, ablation = 1.0, ctx.ablation
        for k in range(self.n_batches):
            batch, keys = self._batch(k)
            per_seq, per_tok = {}, {}
            for sc in ctx.scales:
                loss, st = ctx.programmes[sc](batch, keys, ctx.step)
                totals = torch.stack([loss.float() * st["mask_count"], st["mask_count"]]).double()
                chunk_count = st["mask_by_chunk"].double()
                chunk_total = st["loss_by_chunk"].double() * chunk_count
                if ctx.all_reduce is not None:
                    totals, chunk_total, chunk_count = (ctx.all_reduce(t) for t in (totals, chunk_total, chunk_count))
                self.tally[sc].add(float(totals[0]), float(totals[1]), chunk_total.cpu().numpy(), chunk_count.cpu().numpy())
                if "loss_by_seq" in st:
                    per_seq[sc] = st["loss_by_seq"].float().cpu().numpy()
                    if sc == base:
                        ctx.records.mask.append(st["mask_by_seq"].float().cpu().numpy())
                if "ce_by_token" in st and sc in (ablation, base, "reread"):
                    per_tok[sc] = (st["ce_by_token"].float().cpu().numpy(), st["mask_by_token"].cpu().numpy() > 0.5)
            has_pair = ablation != base and ablation in per_seq and base in per_seq
            if ctx.cfg.eval_probes and ablation != base and ablation in per_tok and base in per_tok:
                ctx.probe_batches.append((self.source.name, k, per_tok[base][0], per_tok[ablation][0], per_tok[base][1]))
                if "reread" in per_tok:
                    ctx.probe_reread.append((self.source.name, k, per_tok["reread"][0], per_tok[ablation][0], per_tok["reread"][1]))
            if "reread" in per_seq and base in per_seq:
                self.reread_gain.append(per_seq[base] - per_seq["reread"])
            doc_len, beyond, doc_id = (a[s.rank * s.local:(s.rank + 1) * s.local]
                                       for a in s.eval_doc_info(self.index, k, ctx.mcfg.eos_token_id, ctx.window_tokens))
            if has_pair:
                delta = per_seq[ablation] - per_seq[base]
                self.gain.append(delta)
                ctx.records.gain.append(delta)
                for j, far in enumerate(beyond):
                    row = (float(per_seq[base][j]), float(delta[j]), int(far))
                    ctx.bucket_rows[_bucket_of(far)].append(row)
                    ctx.source_bucket_rows.setdefault((self.source.name, _bucket_of(far)), []).append(row)
            ctx.records.sources.extend([self.source.name] * len(doc_id))
            ctx.records.doc_ids.append(doc_id)
            ctx.records.doc_lens.append(doc_len)
            ctx.records.beyond.append(beyond)
            for sc in ctx.scales:
                if sc in per_seq:
                    ctx.records.loss[sc].append(per_seq[sc])
        for t in self.tally.values():
            t.finish(max(1, self.n_batches // s.accum))

    def report(self, out: dict) -> None:
        ctx, name = self.ctx, self.source.name
        mean = {sc: t.mean for sc, t in self.tally.items()}
        chunk = {sc: t.by_chunk for sc, t in self.tally.items()}
        out[f"eval/{name}/loss"], out[f"eval/{name}/loss_nottt"] = mean[1.0], mean[ctx.ablation]
        out[f"eval/{name}/gain"] = mean[ctx.ablation] - mean[1.0]
        for sc in ctx.other_scales(include_reread=True):
            out[f"eval/{name}/loss@{_label(sc)}"] = mean[sc]
        for i in range(ctx.n_chunks):
            out[f"eval/{name}/gain_chunk{i}"] = float(chunk[ctx.ablation][i] - chunk[1.0][i])
        if self.reread_gain:
            out[f"eval/{name}/reread_gain"] = mean[1.0] - mean["reread"]
            out[f"eval/{name}/reread_gain_se"] = _stderr(np.concatenate(self.reread_gain))
        if self.gain:
            out[f"eval/{name}/gain_se"] = _stderr(np.concatenate(self.gain))


@dc.dataclass
class _EvalContext:
    cfg: TrainConfig
    mcfg: ModelConfig
    programmes: Dict
    make_batch: Callable
    step: int
    all_reduce: Optional[Callable]
    scales: List = dc.field(default_factory=list)
    ablation: float = 1.0
    n_chunks: int = 0
    window_tokens: int = 0
    records: _Records = dc.field(default_factory=_Records)
    probe_batches: List = dc.field(default_factory=list)
    probe_reread: List = dc.field(default_factory=list)
    bucket_rows: Dict = dc.field(default_factory=dict)
    source_bucket_rows: Dict = dc.field(default_factory=dict)

    def __post_init__(self):
        numeric_first = lambda k: (isinstance(k, str), 0.0 if isinstance(k, str) else k)
        self.scales = sorted(self.programmes, key=numeric_first)
        self.ablation = 0.0 if 0.0 in self.programmes else 1.0
        self.n_chunks = self.cfg.seq_len // self.mcfg.chunk_size
        self.window_tokens = self.mcfg.window_chunks * self.mcfg.chunk_size
        self.records.loss = {sc: [] for sc in self.scales}
        self.bucket_rows = {name: [] for _, _, name in BUCKETS}

    def other_scales(self, include_reread: bool) -> List:
        skip = (self.ablation, 1.0) if include_reread else (self.ablation, 1.0, "reread")
        return [sc for sc in self.scales if sc not in skip]


def _pooled_stderr(weighted_gains: Iterable[Tuple[float, np.ndarray]], weight_sum: float) -> float:
    """Standard error of a weighted mean of per-source means (sources independent)."""
    return float(np.sqrt(sum((w / weight_sum) ** 2 * g.var(ddof=1) / len(g) for w, g in weighted_gains if len(g) > 1)))


def evaluate(eval_fns: Dict, groups, cfg: TrainConfig, mcfg: ModelConfig, make_batch: Callable, step: int, log, is_main: bool = True,
             tag: str = "", all_reduce: Optional[Callable] = None) -> dict:
    """``eval_fns``: ``scale -> fn(batch, row_keys, step) -> (loss, stats)`` (plus the key ``"reread"``); ``groups``:
    ``[(sampler, sources, weighted)]`` (``weighted`` groups form the pooled figures and are limited to ``eval_batches``);
    ``make_batch(ids, outer_t=, loss_mask=) -> Batch``.  Returns the flat record ``{"eval/...": value}``."""
    ctx = _EvalContext(cfg, mcfg, eval_fns, make_batch, step, all_reduce)
    head = f"[eval {step:>6}{tag}]"
    z, nc = ctx.ablation, ctx.n_chunks
    runs: List[_SourceRun] = []
    probe_lookup = {}
    for sampler, sources, weighted in groups:
        for index, source in enumerate(sources):
            probe_lookup[source.name] = (sampler, index)
            run = _SourceRun(ctx, sampler, index, source, weighted)
            run.run()
            runs.append(run)
    out: Dict[str, float] = {}
    for run in runs:
        run.report(out)
    # pooled over the weighted (training-mix) sources
    pooled_runs = [r for r in runs if r.weighted]
    weight_sum = sum(r.source.weight for r in pooled_runs) or 1.0
    total = {sc: sum(r.source.weight * r.tally[sc].mean for r in pooled_runs) / weight_sum for sc in ctx.scales}
    chunk = {sc: sum((r.source.weight * r.tally[sc].by_chunk for r in pooled_runs), np.zeros(nc)) / weight_sum for sc in ctx.scales}
    gains = [(r.source.weight, np.concatenate(r.gain)) for r in pooled_runs if r.gain]
    reread_gains = [(r.source.weight, np.concatenate(r.reread_gain)) for r in pooled_runs if r.reread_gain]
    out.update({"eval/loss": total[1.0], "eval/loss_nottt": total[z], "eval/ttt_gain": total[z] - total[1.0]})
    out.update({f"eval/chunk{i}": float(v) for i, v in enumerate(chunk[1.0])})
    out.update({f"eval/gain_chunk{i}": float(chunk[z][i] - chunk[1.0][i]) for i in range(nc)})
    for sc in ctx.other_scales(include_reread=True):
        out[f"eval/loss@{_label(sc)}"] = total[sc]
    if reread_gains:
        out["eval/reread_gain"], out["eval/reread_gain_se"] = total[1.0] - total["reread"], _pooled_stderr(reread_gains, weight_sum)
        out.update({f"eval/reread_chunk{i}": float(chunk[1.0][i] - chunk["reread"][i]) for i in range(nc)})
    if gains:
        out["eval/ttt_gain_se"] = _pooled_stderr(gains, weight_sum)

    sources = [r.source for r in runs]
    fmt = lambda values, spec: " ".join(format(v, spec) for v in values)
    per_source = lambda text: " ".join(text(s.name) for s in sources)
    log(f"{head} loss {total[1.0]:.4f}  no-ttt {total[z]:.4f}  gain {total[z] - total[1.0]:+.4f}"
        + (f" (se {out['eval/ttt_gain_se']:.4f})" if gains else "") + " | by chunk " + fmt(chunk[1.0], ".2f")
        + " | " + per_source(lambda n: f"{n} {out[f'eval/{n}/loss']:.2f}"))
    others = ctx.other_scales(include_reread=False)

    def gain_with_se(n: str) -> str:
        se = out.get(f"eval/{n}/gain_se")
        return f"{n} {out[f'eval/{n}/gain']:+.3f}" + (f"±{se:.3f}" if se is not None else "")

    log(f"{head} gain by chunk " + fmt(chunk[z] - chunk[1.0], "+.3f") + " | " + per_source(gain_with_se)
        + (" | lr scale " + " ".join(f"{_label(sc)} {total[sc]:.4f}" for sc in others) if others else ""))
    log(f"{head} gain by chunk per source: " + " | ".join(
        f"{s.name} " + fmt((out[f"eval/{s.name}/gain_chunk{i}"] for i in range(nc)), "+.3f") for s in sources))
    pool = {r.source.name for r in pooled_runs}
    if ctx.probe_batches:
        out.update(probe_report(ctx.probe_batches, probe_lookup, sources, mcfg, cfg, head, log, pool=pool))
    if "reread" in eval_fns:
        log(f"{head} reread(n={cfg.eval_reread_chunks}): loss {total['reread']:.4f}  single {total[1.0]:.4f}  benefit "
            f"{total[1.0] - total['reread']:+.4f}" + (f" (se {out['eval/reread_gain_se']:.4f})" if reread_gains else "")
            + f" | ablation single {total[z] - total[1.0]:+.4f} reread {total[z] - total['reread']:+.4f} | by chunk "
            + fmt(chunk[1.0] - chunk["reread"], "+.3f"))
        if ctx.probe_reread:
            out.update(probe_report(ctx.probe_reread, probe_lookup, sources, mcfg, cfg, head, log, label="reread probe",
                                    key_prefix="eval/probe_reread", pool=pool))
    _report_buckets(ctx, out, head, log)
    folder = _output_dir(cfg)
    if folder and is_main:
        os.makedirs(folder, exist_ok=True)
        ctx.records.save(os.path.join(folder, f"eval_{step}{tag.replace(' ', '_').replace('=', '')}.npz"))
    for sc in others:
        log(f"{head} {_label(sc)} vs x1: by chunk " + fmt(chunk[1.0] - chunk[sc], "+.3f") + " | "
            + per_source(lambda n: f"{n} {out[f'eval/{n}/loss'] - out[f'eval/{n}/loss@{_label(sc)}']:+.3f}"))
    if tag:
        out = {k.replace("eval/", f"eval{tag}/", 1): v for k, v in out.items()}
    return out


def _report_buckets(ctx: _EvalContext, out: dict, head: str, log) -> None:
    """The ablation by how much of the sequence's first document lies beyond the attention window."""
    filled = {name: np.array(rows) for name, rows in ctx.bucket_rows.items() if rows}
    if not filled:
        return
    texts = []
    for name, a in filled.items():
        out[f"eval/bucket/{name}/loss"], out[f"eval/bucket/{name}/gain"] = float(a[:, 0].mean()), float(a[:, 1].mean())
        out[f"eval/bucket/{name}/n"] = len(a)
        texts.append(f"{name}: n={len(a)} loss {a[:, 0].mean():.3f} gain {a[:, 1].mean():+.4f} beyond {a[:, 2].mean() / 1024:.1f}K")
    log(f"{head} by beyond window: " + " | ".join(texts))
    log(f"{head} by source x beyond: " + " | ".join(
        f"{src}/{bucket} {np.array(rows)[:, 1].mean():+.4f} (n={len(rows)})" for (src, bucket), rows in sorted(ctx.source_bucket_rows.items())))


# ------------------------------------------------------------------------------------------------------------ token-class probes
class _ProbeTable:
    """Class tables (``probes.aggregate``) of one probe, pooled by token count."""

    def __init__(self):
        self.parts: List[dict] = []

    def add(self, table: dict) -> None:
        self.parts.append(table)

    def __bool__(self) -> bool:
        return bool(self.parts)

    def merged(self):
        n = sum(p["n"] for p in self.parts)
        weight = np.maximum(n, 1)
        loss = sum(p["loss"] * p["n"] for p in self.parts) / weight
        gain = sum(p["gain"] * p["n"] for p in self.parts) / weight
        per_sequence = np.concatenate([p["seq_gain"] for p in self.parts], axis=1)
        chunk_n = sum(p["n_by_chunk"] for p in self.parts)
        chunk_gain = sum(p["gain_by_chunk"] * p["n_by_chunk"] for p in self.parts) / np.maximum(chunk_n, 1)
        return n, loss, gain, per_sequence, chunk_gain


def _rarity_bins(cfg: TrainConfig, mcfg: ModelConfig) -> Optional[np.ndarray]:
    path = cfg.data_path(cfg.unigram_path)
    if not (path and os.path.exists(path)):
        return None
    counts = np.fromfile(path, dtype=np.int64)
    return PR.rarity_bins(counts[:mcfg.vocab_size]) if len(counts) >= mcfg.vocab_size else None


def probe_report(batches, probe_ctx, sources, mcfg: ModelConfig, cfg: TrainConfig, pre: str, log, label: str = "probe",
                 key_prefix: str = "eval/probe", pool=None) -> dict:
    """P1 / P2 / P3 classes of every scored held-out token: tables per source and pooled over the sources in ``pool`` (all when
    ``None``).  ``batches``: ``[(source name, batch index, ce_on, ce_off, scored)]``; ``probe_ctx``: name -> ``(sampler, index)``."""
    chunk, window = mcfg.chunk_size, mcfg.window_chunks
    bins = _rarity_bins(cfg, mcfg)
    kinds = (("P1", PR.P1_CLASSES), ("P2", PR.P2_CLASSES), ("P3", PR.P3_CLASSES))
    pooled = {kind: _ProbeTable() for kind, _ in kinds}
    by_source: Dict[Tuple[str, str], _ProbeTable] = {}
    for name, k, ce_on, ce_off, scored in batches:
        sampler, index = probe_ctx[name]
        rows, T = ce_on.shape
        mine = slice(sampler.rank * sampler.local, sampler.rank * sampler.local + rows)
        recurrence = np.zeros((rows, T), np.int8)
        tokens = np.zeros((rows, T), np.int64)
        for j, (context, at, doc_starts) in enumerate(sampler.eval_context(index, k, mcfg.eos_token_id, lookback=131072)[mine]):
            recurrence[j] = PR.recurrence_classes(context, at, T, doc_starts, chunk, window)
            tokens[j] = context[at:at + T]
        labelled = [("P1", recurrence, len(PR.P1_CLASSES)), ("P3", PR.neighbour_classes(scored), len(PR.P3_CLASSES))]
        if bins is not None:
            labelled.append(("P2", bins[np.clip(tokens, 0, len(bins) - 1)], len(PR.P2_CLASSES)))
        for kind, labels, n_classes in labelled:
            table = PR.aggregate(ce_on, ce_off, scored, labels, n_classes, chunk)
            by_source.setdefault((kind, name), _ProbeTable()).add(table)
            if pool is None or name in pool:
                pooled[kind].add(table)
    out = {}
    for kind, classes in kinds:
        if not pooled[kind]:
            continue
        n, loss, gain, per_sequence, chunk_gain = pooled[kind].merged()
        cells = []
        for c, cname in enumerate(classes):
            se = PR.se_over_sequences(per_sequence[c])
            stem = f"{key_prefix}/{kind}/{cname}"
            out.update({f"{stem}/n": int(n[c]), f"{stem}/loss": float(loss[c]), f"{stem}/gain": float(gain[c]), f"{stem}/se": se})
            cells.append(f"{cname} n={int(n[c])} loss {loss[c]:.3f} gain {gain[c]:+.4f}±{se:.4f}")
        if kind == "P3":                                         # does a visible LEFT neighbour help more than a visible right one?
            paired = per_sequence[1] - per_sequence[2]
            paired_se = _stderr(paired[~np.isnan(paired)])
            out[f"{key_prefix}/P3/left_minus_right"], out[f"{key_prefix}/P3/left_minus_right_se"] = float(gain[1] - gain[2]), paired_se
            cells.append(f"Lv_Rm - Lm_Rv {gain[1] - gain[2]:+.4f}±{paired_se:.4f}")
        log(f"{pre} {label} {kind} pooled: " + " | ".join(cells))
        log(f"{pre} {label} {kind} gain by chunk: " + " | ".join(
            f"{cname} " + " ".join(f"{v:+.3f}" for v in chunk_gain[c]) for c, cname in enumerate(classes)))
        for src in sources:
            table = by_source.get((kind, src.name))
            if not table:
                continue
            n, loss, gain, _, _ = table.merged()
            for c, cname in enumerate(classes):
                out[f"{key_prefix}/{kind}/{src.name}/{cname}/gain"] = float(gain[c])
                out[f"{key_prefix}/{kind}/{src.name}/{cname}/n"] = int(n[c])
            log(f"{pre} {label} {kind} {src.name}: " + " | ".join(
                f"{cname} n={int(n[c])} loss {loss[c]:.3f} gain {gain[c]:+.4f}" for c, cname in enumerate(classes)))
    return out


# ------------------------------------------------------------------------------------------------------------ planted recall
def _planted_losses(planted_fns: Dict, groups, cfg: TrainConfig, mcfg: ModelConfig, make_batch: Callable, step: int):
    """Mean CE of the scored tail per held-out sequence for every (placement, mode, scale); also the source name per sequence
    and, when a write plan is evaluated, its (before, after) own-chunk CE."""
    chunk, window = mcfg.chunk_size, mcfg.window_chunks
    scales = sorted(planted_fns)
    losses: Dict[Tuple[str, str, float], List[np.ndarray]] = {}
    names: List[str] = []
    plan_pairs: List[Tuple[float, float]] = []
    for sampler, sources, _ in groups:
        for index, source in enumerate(sources):
            n_batches = sampler.accum * min(cfg.eval_planted_batches, sampler.eval_step_batches(index))
            for k in range(n_batches):
                local = sampler.eval_batch(index, k)
                first = k * sampler.G + sampler.rank * sampler.local
                rows = list(range(first, first + sampler.local))
                keys = rng.fold_in(rng.key(cfg.eval_seed).unsqueeze(0).expand(len(rows), 2), torch.as_tensor(rows))
                names.extend([source.name] * sampler.local)
                for placement in PR.PLANT_PLACEMENTS:
                    for mode in PR.PLANT_MODES:
                        ids, scored = PR.planted_probe_batch(local, rows, cfg.eval_seed, chunk, window, cfg.eval_planted_len,
                                                             cfg.eval_planted_cue, placement, mode, eos=mcfg.eos_token_id)
                        batch = make_batch(ids, outer_t=np.ones(len(ids), np.float32), loss_mask=scored)
                        for sc in scales:
                            _, st = planted_fns[sc](batch, keys, step)
                            ce = st["ce_by_token"].double().cpu().numpy()
                            m = st["mask_by_token"].cpu().numpy() > 0.5
                            losses.setdefault((placement, mode, sc), []).append((ce * m).sum(1) / np.maximum(m.sum(1), 1))
                            if "inner_plan_pre" in st and (placement, mode, sc) == ("beyond", "alt", 1.0):
                                plan_pairs.append((float(st["inner_plan_pre"]), float(st["inner_plan_post"])))
    return {key: np.concatenate(parts) for key, parts in losses.items()}, names, plan_pairs, scales


def evaluate_planted(planted_fns: Dict, groups, cfg: TrainConfig, mcfg: ModelConfig, make_batch: Callable, step: int, log,
                     is_main: bool = True) -> dict:
    """Planted-recall probe: a span of chunk 1 copied beyond the attention window (and, as the ceiling, inside it), its tail after
    the cue masked; mean CE of that tail with the memory on and off, the gain of the write, and how much of the copy ceiling
    (what a visible copy is worth) the memory recovers."""
    arr, names, plan_pairs, scales = _planted_losses(planted_fns, groups, cfg, mcfg, make_batch, step)
    out: Dict[str, float] = {}
    if not arr:
        return out
    head = f"[eval {step:>6}]"
    if plan_pairs:
        before, after = np.mean(plan_pairs, axis=0)
        out.update({"eval/plan_own_ce_before": float(before), "eval/plan_own_ce_after": float(after)})
        log(f"{head} write plan {cfg.eval_write_plan}: own causal CE of the chunks written > once {before:.3f} -> {after:.3f} after their steps")
    name_of = np.array(names)
    with_ablation = 0.0 in scales
    for mode in PR.PLANT_MODES:
        beyond_on, within_on = arr[("beyond", mode, 1.0)], arr[("within", mode, 1.0)]
        out[f"eval/planted_{mode}_beyond"], out[f"eval/planted_{mode}_within"] = float(beyond_on.mean()), float(within_on.mean())
        opening = (f"{head} planted recall {mode} (n={len(beyond_on)}, span {cfg.eval_planted_len}, cue {cfg.eval_planted_cue}): "
                   f"beyond on {beyond_on.mean():.3f}")
        if not with_ablation:
            log(opening + f" | within on {within_on.mean():.3f}")
            continue
        beyond_off, within_off = arr[("beyond", mode, 0.0)], arr[("within", mode, 0.0)]
        unplanted_gain = arr[("none", mode, 0.0)] - arr[("none", mode, 1.0)]
        gain = beyond_off - beyond_on
        recall = gain - unplanted_gain                            # the part of the gain that the plant itself explains
        ceiling = float(beyond_off.mean() - within_off.mean())
        recovered = float(gain.mean() / ceiling) if ceiling > 0.01 else float("nan")
        out.update({f"eval/planted_{mode}_recall": float(recall.mean()), f"eval/planted_{mode}_recall_se": _stderr(recall),
                    f"eval/planted_{mode}_gain": float(gain.mean()), f"eval/planted_{mode}_gain_se": _stderr(gain),
                    f"eval/planted_{mode}_ceiling": ceiling})
        if np.isfinite(recovered):
            out[f"eval/planted_{mode}_recovered"] = recovered
        share = f"{100 * recovered:.1f}%" if np.isfinite(recovered) else "n/a (no copy ceiling)"
        log(opening + f" off {beyond_off.mean():.3f} gain {gain.mean():+.4f} (se {_stderr(gain):.4f}) | within on {within_on.mean():.3f} "
            f"off {within_off.mean():.3f} | copy ceiling {ceiling:+.3f} recovered {share}"
            f" | unplanted gain {float(unplanted_gain.mean()):+.4f} -> recall {float(recall.mean()):+.4f} (se {_stderr(recall):.4f})")
        log(f"{head} planted recall {mode} gain by source: " + " | ".join(
            f"{n} {gain[name_of == n].mean():+.3f}" for n in dict.fromkeys(names)))
    folder = _output_dir(cfg)
    if folder and is_main:
        os.makedirs(folder, exist_ok=True)
        np.savez_compressed(os.path.join(folder, f"eval_{step}_planted.npz"), sources=name_of,
                            **{f"{placement}_{mode}_x{sc:g}": v for (placement, mode, sc), v in arr.items()})
    return out
