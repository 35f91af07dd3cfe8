"""Held-out evaluation: loss per source, the write ablation, loss by chunk position, probes, planted recall.

``evaluate`` scores the held-out tail of every source with *fixed, stratified* noise: sequence ``j`` gets the
noise level ``(perm[j] + u_j) / n`` and its own row key, both derived from ``eval_seed`` and ``j`` alone, so the
numbers do not depend on the batch shape or the rank count and are paired across checkpoints and runs
(reference ``src/ttt/train.py:277-496``).  Every batch is run once per inner-lr scale: 1 is the trained setting,
0 the no-write twin; ``gain = loss(0) - loss(1)`` is the write ablation, reported overall, per source, per chunk
position, per "tokens beyond the window" bucket, with the paired standard error over sequences.  Per-sequence
results go to ``eval_<step>.npz`` for the offline tools.  ``evaluate_planted`` is the planted-recall probe
(``train.py:499-585``), ``probe_report`` the P1/P2/P3 token-class probes (``train.py:588-672``).
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..schema import ModelConfig, TrainConfig
from ..ttt.scan import Batch
from ..utils import rng
from . import probes as PR

BUCKETS = ((0, 1, "0"), (1, 1024, "1-1K"), (1024, 3072, "1-3K"), (3072, 1 << 62, ">=3K"))


def _label(k) -> str:
    return k if isinstance(k, str) else f"x{k:g}"


def row_keys(eval_seed: int, j_indices: Sequence[int]):
    """Per-sequence ``(u [n], row keys [n, 2])`` from ``fold_in(key(eval_seed), j)`` split in two."""
    base = rng.key(eval_seed)
    ks = rng.fold_in(base.unsqueeze(0).expand(len(j_indices), 2), torch.as_tensor(list(j_indices), dtype=torch.int64))
    sp = rng.split(ks, 2)
    return rng.uniform(sp[:, 0], ()).numpy(), sp[:, 1]


def evaluate(eval_fns: Dict, groups, cfg: TrainConfig, mcfg: ModelConfig, make_batch: Callable, step: int, log, is_main: bool = True,
             tag: str = "", all_reduce: Optional[Callable] = None) -> dict:
    """``eval_fns``: ``scale -> fn(batch, row_keys, step) -> (loss, stats)`` (plus the key ``"reread"``);
    ``groups``: ``[(sampler, sources, weighted)]``; ``make_batch(ids, outer_t=, loss_mask=) -> Batch``."""
    pre = f"[eval {step:>6}{tag}]"
    scales = sorted(eval_fns, key=lambda k: (isinstance(k, str), 0.0 if isinstance(k, str) else k))
    z = 0.0 if 0.0 in eval_fns else 1.0
    C = mcfg.chunk_size
    nc = cfg.seq_len // C
    window_tokens = mcfg.window_chunks * C
    out: Dict[str, float] = {}
    tot = {k: 0.0 for k in scales}
    chunk = {k: np.zeros(nc) for k in scales}
    wsum = 0.0
    gains, rr_gains, probe_batches, probe_rr = [], [], [], []
    by_bucket = {b[2]: [] for b in BUCKETS}
    src_bucket: Dict = {}
    sources = [s for _, srcs, _ in groups for s in srcs]
    pool = {s.name for _, srcs, weighted in groups if weighted for s in srcs}
    probe_ctx = {}
    rec = {"sources": [], "doc_ids": [], "doc_lens": [], "beyond": [], "gain": [], "mask": []}
    rec_loss = {sc: [] for sc in scales}
    for sampler, srcs, weighted in groups:
        for si, src in enumerate(srcs):
            probe_ctx[src.name] = (sampler, si)
            n_hold = max(1, int(sampler.n_eval_seq[si]))
            perm = np.random.default_rng(cfg.eval_seed).permutation(n_hold)
            n_steps = sampler.eval_step_batches(si)
            n_b = sampler.accum * (n_steps if not weighted else min(cfg.eval_batches, n_steps))
            acc = {k: 0.0 for k in scales}
            ch = {k: np.zeros(nc) for k in scales}
            g_src, rr_src = [], []
            part = {k: [0.0, 0.0, np.zeros(nc), np.zeros(nc)] for k in scales}
            for k in range(n_b):
                j0 = k * sampler.G + sampler.rank * sampler.local
                j_idx = [(j0 + j) % n_hold for j in range(sampler.local)]
                u, keys_row = row_keys(cfg.eval_seed, j_idx)
                t_local = ((perm[j_idx].astype(np.float32) + u) / float(n_hold)).astype(np.float32)
                b = make_batch(sampler.eval_batch(si, k), outer_t=t_local)
                seq, tok = {}, {}
                for sc in scales:
                    loss, st = eval_fns[sc](b, keys_row, step)
                    red = torch.stack([loss.float() * st["mask_count"], st["mask_count"]]).double()
                    lbc, mbc = st["loss_by_chunk"].double() * st["mask_by_chunk"].double(), st["mask_by_chunk"].double()
                    if all_reduce is not None:
                        red, lbc, mbc = all_reduce(red), all_reduce(lbc), all_reduce(mbc)
                    pt = part[sc]
                    pt[0] += float(red[0]); pt[1] += float(red[1])
                    pt[2] += lbc.cpu().numpy(); pt[3] += mbc.cpu().numpy()
                    if (k + 1) % sampler.accum == 0:
                        acc[sc] += pt[0] / max(pt[1], 1e-6)
                        ch[sc] += pt[2] / np.maximum(pt[3], 1e-6)
                        part[sc] = [0.0, 0.0, np.zeros(nc), np.zeros(nc)]
                    if "loss_by_seq" in st:
                        seq[sc] = st["loss_by_seq"].float().cpu().numpy()
                        if sc == 1.0:
                            rec["mask"].append(st["mask_by_seq"].float().cpu().numpy())
                    if "ce_by_token" in st and sc in (z, 1.0, "reread"):
                        tok[sc] = (st["ce_by_token"].float().cpu().numpy(), st["mask_by_token"].cpu().numpy() > 0.5)
                if cfg.eval_probes and z in tok and 1.0 in tok and z != 1.0:
                    probe_batches.append((src.name, k, tok[1.0][0], tok[z][0], tok[1.0][1]))
                    if "reread" in tok:
                        probe_rr.append((src.name, k, tok["reread"][0], tok[z][0], tok["reread"][1]))
                if "reread" in seq and 1.0 in seq:
                    rr_src.append(seq[1.0] - seq["reread"])
                doc_len, beyond, doc_id = sampler.eval_doc_info(si, k, mcfg.eos_token_id, window_tokens)
                lo = sampler.rank * sampler.local
                dl, by, di = (a[lo:lo + sampler.local] for a in (doc_len, beyond, doc_id))
                if z in seq and 1.0 in seq and z != 1.0:
                    g_src.append(seq[z] - seq[1.0])
                    for j in range(len(by)):
                        name = next(bk[2] for bk in BUCKETS if bk[0] <= by[j] < bk[1])
                        r = (float(seq[1.0][j]), float(seq[z][j] - seq[1.0][j]), int(by[j]))
                        by_bucket[name].append(r)
                        src_bucket.setdefault((src.name, name), []).append(r)
                    rec["gain"].append(seq[z] - seq[1.0])
                rec["sources"].extend([src.name] * len(di))
                rec["doc_ids"].append(di); rec["doc_lens"].append(dl); rec["beyond"].append(by)
                for sc in scales:
                    if sc in seq:
                        rec_loss[sc].append(seq[sc])
            denom = max(1, n_b // sampler.accum)
            for sc in scales:
                acc[sc] /= denom
                ch[sc] /= denom
                if weighted:
                    tot[sc] += src.weight * acc[sc]
                    chunk[sc] += src.weight * ch[sc]
            if weighted:
                wsum += src.weight
            out[f"eval/{src.name}/loss"], out[f"eval/{src.name}/loss_nottt"] = acc[1.0], acc[z]
            out[f"eval/{src.name}/gain"] = acc[z] - acc[1.0]
            for sc in scales:
                if sc not in (z, 1.0):
                    out[f"eval/{src.name}/loss@{_label(sc)}"] = acc[sc]
            for i in range(nc):
                out[f"eval/{src.name}/gain_chunk{i}"] = float(ch[z][i] - ch[1.0][i])
            if rr_src:
                g = np.concatenate(rr_src)
                out[f"eval/{src.name}/reread_gain"] = acc[1.0] - acc["reread"]
                out[f"eval/{src.name}/reread_gain_se"] = float(g.std(ddof=1) / np.sqrt(len(g))) if len(g) > 1 else float("nan")
                if weighted:
                    rr_gains.append((src.weight, g))
            if g_src:
                g = np.concatenate(g_src)
                out[f"eval/{src.name}/gain_se"] = float(g.std(ddof=1) / np.sqrt(len(g))) if len(g) > 1 else float("nan")
                if weighted:
                    gains.append((src.weight, g))
    wsum = wsum or 1.0
    for sc in scales:
        tot[sc] /= wsum
        chunk[sc] /= wsum
    out.update({"eval/loss": tot[1.0], "eval/loss_nottt": tot[z], "eval/ttt_gain": tot[z] - tot[1.0]})
    out.update({f"eval/chunk{i}": float(v) for i, v in enumerate(chunk[1.0])})
    out.update({f"eval/gain_chunk{i}": float(chunk[z][i] - chunk[1.0][i]) for i in range(nc)})
    for sc in scales:
        if sc not in (z, 1.0):
            out[f"eval/loss@{_label(sc)}"] = tot[sc]
    se_of = lambda pairs: float(np.sqrt(sum((w / wsum) ** 2 * g.var(ddof=1) / len(g) for w, g in pairs if len(g) > 1)))
    if rr_gains:
        out["eval/reread_gain"], out["eval/reread_gain_se"] = tot[1.0] - tot["reread"], se_of(rr_gains)
        out.update({f"eval/reread_chunk{i}": float(chunk[1.0][i] - chunk["reread"][i]) for i in range(nc)})
    if gains:
        out["eval/ttt_gain_se"] = se_of(gains)
    log(f"{pre} loss {tot[1.0]:.4f}  no-ttt {tot[z]:.4f}  gain {tot[z] - tot[1.0]:+.4f}"
        + (f" (se {out['eval/ttt_gain_se']:.4f})" if gains else "") + " | by chunk " + " ".join(f"{v:.2f}" for v in chunk[1.0])
        + " | " + " ".join(f"{s.name} {out[f'eval/{s.name}/loss']:.2f}" for s in sources))
    others = [sc for sc in scales if sc not in (z, 1.0, "reread")]
    log(f"{pre} gain by chunk " + " ".join(f"{v:+.3f}" for v in chunk[z] - chunk[1.0]) + " | "
        + " ".join(f"{s.name} {out[f'eval/{s.name}/gain']:+.3f}"
                   + (f"±{out[f'eval/{s.name}/gain_se']:.3f}" if f"eval/{s.name}/gain_se" in out else "") for s in sources)
        + (" | lr scale " + " ".join(f"{_label(sc)} {tot[sc]:.4f}" for sc in others) if others else ""))
    log(f"{pre} gain by chunk per source: " + " | ".join(
        f"{s.name} " + " ".join(f"{out[f'eval/{s.name}/gain_chunk{i}']:+.3f}" for i in range(nc)) for s in sources))
    if probe_batches:
        out.update(probe_report(probe_batches, probe_ctx, sources, mcfg, cfg, pre, log, pool=pool))
    if "reread" in eval_fns:
        log(f"{pre} reread(n={cfg.eval_reread_chunks}): loss {tot['reread']:.4f}  single {tot[1.0]:.4f}  benefit "
            f"{tot[1.0] - tot['reread']:+.4f}" + (f" (se {out['eval/reread_gain_se']:.4f})" if rr_gains else "")
            + f" | ablation single {tot[z] - tot[1.0]:+.4f} reread {tot[z] - tot['reread']:+.4f} | by chunk "
            + " ".join(f"{v:+.3f}" for v in chunk[1.0] - chunk["reread"]))
        if probe_rr:
            out.update(probe_report(probe_rr, probe_ctx, sources, mcfg, cfg, pre, log, label="reread probe",
                                    key_prefix="eval/probe_reread", pool=pool))
    if any(by_bucket.values()):
        def fmt(recs):
            a = np.array(recs)
            return f"n={len(a)} loss {a[:, 0].mean():.3f} gain {a[:, 1].mean():+.4f} beyond {a[:, 2].mean() / 1024:.1f}K"
        for name, recs in by_bucket.items():
            if recs:
                a = np.array(recs)
                out[f"eval/bucket/{name}/loss"], out[f"eval/bucket/{name}/gain"] = float(a[:, 0].mean()), float(a[:, 1].mean())
                out[f"eval/bucket/{name}/n"] = len(a)
        log(f"{pre} by beyond window: " + " | ".join(f"{n}: {fmt(r)}" for n, r in by_bucket.items() if r))
        log(f"{pre} by source x beyond: " + " | ".join(
            f"{s_}/{b_} {np.array(r)[:, 1].mean():+.4f} (n={len(r)})" for (s_, b_), r in sorted(src_bucket.items())))
    eval_dir = cfg.log_dir or os.environ.get("DTTT_LOG_DIR", os.environ.get("TTT_LOG_DIR", ""))
    if eval_dir and is_main:
        os.makedirs(eval_dir, exist_ok=True)
        cat = lambda xs, dt=np.int64: np.concatenate(xs) if xs else np.array([], dtype=dt)
        save = {"sources": np.array(rec["sources"]), "doc_ids": cat(rec["doc_ids"]), "doc_lens": cat(rec["doc_lens"]),
                "beyond": cat(rec["beyond"])}
        for sc, ls in rec_loss.items():
            if ls:
                save[f"loss_{sc}"] = np.concatenate(ls)
        if rec["gain"]:
            save["gain"] = np.concatenate(rec["gain"])
        if rec["mask"]:
            save["mask"] = np.concatenate(rec["mask"])
        np.savez_compressed(os.path.join(eval_dir, f"eval_{step}{tag.replace(' ', '_').replace('=', '')}.npz"), **save)
    for sc in others:
        log(f"{pre} {_label(sc)} vs x1: by chunk " + " ".join(f"{v:+.3f}" for v in chunk[1.0] - chunk[sc]) + " | "
            + " ".join(f"{s.name} {out[f'eval/{s.name}/loss'] - out[f'eval/{s.name}/loss@{_label(sc)}']:+.3f}" for s in sources))
    if tag:
        out = {k.replace("eval/", f"eval{tag}/", 1): v for k, v in out.items()}
    return out


def probe_report(batches, probe_ctx, sources, mcfg: ModelConfig, cfg: TrainConfig, pre: str, log, label: str = "probe",
                 key_prefix: str = "eval/probe", pool=None) -> dict:
    """P1 / P2 / P3 classes of every scored held-out token, aggregated per source and pooled over the training mix."""
    C, W = mcfg.chunk_size, mcfg.window_chunks
    bins = None
    uni = cfg.data_path(cfg.unigram_path)
    if uni and os.path.exists(uni):
        counts = np.fromfile(uni, dtype=np.int64)
        if len(counts) >= mcfg.vocab_size:
            bins = PR.rarity_bins(counts[:mcfg.vocab_size])
    pooled = {"P1": [], "P2": [], "P3": []}
    per_src: Dict = {}
    for sname, k, ce_on, ce_off, scored in batches:
        sampler, si = probe_ctx[sname]
        lo = sampler.rank * sampler.local
        ctx = sampler.eval_context(si, k, mcfg.eos_token_id, lookback=131072)[lo:lo + ce_on.shape[0]]
        B, T = ce_on.shape
        lab1 = np.zeros((B, T), np.int8)
        toks = np.zeros((B, T), np.int64)
        for j, (c_tokens, off, dstarts) in enumerate(ctx):
            lab1[j] = PR.recurrence_classes(c_tokens, off, T, dstarts, C, W)
            toks[j] = c_tokens[off:off + T]
        sets = [("P1", lab1, len(PR.P1_CLASSES)), ("P3", PR.neighbour_classes(scored), len(PR.P3_CLASSES))]
        if bins is not None:
            sets.append(("P2", bins[np.clip(toks, 0, len(bins) - 1)], len(PR.P2_CLASSES)))
        for probe, labels, n_cls in sets:
            a = PR.aggregate(ce_on, ce_off, scored, labels, n_cls, C)
            per_src.setdefault((probe, sname), []).append(a)
            if pool is None or sname in pool:
                pooled[probe].append(a)

    def merge(aggs):
        n = sum(a["n"] for a in aggs)
        loss = sum(a["loss"] * a["n"] for a in aggs) / np.maximum(n, 1)
        gain = sum(a["gain"] * a["n"] for a in aggs) / np.maximum(n, 1)
        seq = np.concatenate([a["seq_gain"] for a in aggs], axis=1)
        nbc = sum(a["n_by_chunk"] for a in aggs)
        gbc = sum(a["gain_by_chunk"] * a["n_by_chunk"] for a in aggs) / np.maximum(nbc, 1)
        return n, loss, gain, seq, gbc

    out = {}
    for probe, classes in (("P1", PR.P1_CLASSES), ("P2", PR.P2_CLASSES), ("P3", PR.P3_CLASSES)):
        if not pooled[probe]:
            continue
        n, loss, gain, seq, gbc = merge(pooled[probe])
        parts = []
        for ci, name in enumerate(classes):
            se = PR.se_over_sequences(seq[ci])
            out.update({f"{key_prefix}/{probe}/{name}/n": int(n[ci]), f"{key_prefix}/{probe}/{name}/loss": float(loss[ci]),
                        f"{key_prefix}/{probe}/{name}/gain": float(gain[ci]), f"{key_prefix}/{probe}/{name}/se": se})
            parts.append(f"{name} n={int(n[ci])} loss {loss[ci]:.3f} gain {gain[ci]:+.4f}±{se:.4f}")
        if probe == "P3":
            dd = seq[1] - seq[2]
            dd = dd[~np.isnan(dd)]
            dse = float(dd.std(ddof=1) / np.sqrt(len(dd))) if len(dd) > 1 else float("nan")
            out[f"{key_prefix}/P3/left_minus_right"], out[f"{key_prefix}/P3/left_minus_right_se"] = float(gain[1] - gain[2]), dse
            parts.append(f"Lv_Rm - Lm_Rv {gain[1] - gain[2]:+.4f}±{dse:.4f}")
        log(f"{pre} {label} {probe} pooled: " + " | ".join(parts))
        log(f"{pre} {label} {probe} gain by chunk: " + " | ".join(
            f"{name} " + " ".join(f"{v:+.3f}" for v in gbc[ci]) for ci, name in enumerate(classes)))
        for src in sources:
            aggs = per_src.get((probe, src.name))
            if not aggs:
                continue
            n, loss, gain, seq, _ = merge(aggs)
            for ci, name in enumerate(classes):
                out[f"{key_prefix}/{probe}/{src.name}/{name}/gain"] = float(gain[ci])
                out[f"{key_prefix}/{probe}/{src.name}/{name}/n"] = int(n[ci])
            log(f"{pre} {label} {probe} {src.name}: " + " | ".join(
                f"{name} n={int(n[ci])} loss {loss[ci]:.3f} gain {gain[ci]:+.4f}" for ci, name in enumerate(classes)))
    return out


def evaluate_planted(planted_fns: Dict, groups, cfg: TrainConfig, mcfg: ModelConfig, make_batch: Callable, step: int, log,
                     is_main: bool = True) -> dict:
    """Planted-recall probe: a span of chunk 1 copied beyond the attention window (and, as the ceiling, inside
    it), its tail after the cue masked; mean CE of that tail with the memory on and off."""
    C, Wn = mcfg.chunk_size, mcfg.window_chunks
    scales = sorted(planted_fns)
    per: Dict = {}
    names: List[str] = []
    plan_ce = []
    for sampler, srcs, _ in groups:
        for si, src in enumerate(srcs):
            for k in range(sampler.accum * min(cfg.eval_planted_batches, sampler.eval_step_batches(si))):
                local = sampler.eval_batch(si, k)
                j0 = k * sampler.G + sampler.rank * sampler.local
                j_global = [j0 + j for j in range(sampler.local)]
                keys = rng.fold_in(rng.key(cfg.eval_seed).unsqueeze(0).expand(len(j_global), 2), torch.as_tensor(j_global))
                names.extend([src.name] * sampler.local)
                for pl in PR.PLANT_PLACEMENTS:
                    for mode in PR.PLANT_MODES:
                        ids, lm = PR.planted_probe_batch(local, j_global, cfg.eval_seed, C, Wn, cfg.eval_planted_len,
                                                         cfg.eval_planted_cue, pl, mode, eos=mcfg.eos_token_id)
                        b = make_batch(ids, outer_t=np.ones(len(ids), np.float32), loss_mask=lm)
                        for sc in scales:
                            _, st = planted_fns[sc](b, keys, step)
                            ce = st["ce_by_token"].double().cpu().numpy()
                            m = st["mask_by_token"].cpu().numpy() > 0.5
                            per.setdefault((pl, mode, sc), []).append((ce * m).sum(1) / np.maximum(m.sum(1), 1))
                            if "inner_plan_pre" in st and pl == "beyond" and mode == "alt" and sc == 1.0:
                                plan_ce.append((float(st["inner_plan_pre"]), float(st["inner_plan_post"])))
    out: Dict[str, float] = {}
    if not per:
        return out
    pre = f"[eval {step:>6}]"
    if plan_ce:
        a, b = np.mean(plan_ce, axis=0)
        out.update({"eval/plan_own_ce_before": float(a), "eval/plan_own_ce_after": float(b)})
        log(f"{pre} write plan {cfg.eval_write_plan}: own causal CE of the chunks written > once {a:.3f} -> {b:.3f} after their steps")
    arr = {kk: np.concatenate(v) for kk, v in per.items()}
    nm = np.array(names)
    for mode in PR.PLANT_MODES:
        b_on, w_on = arr[("beyond", mode, 1.0)], arr[("within", mode, 1.0)]
        out[f"eval/planted_{mode}_beyond"], out[f"eval/planted_{mode}_within"] = float(b_on.mean()), float(w_on.mean())
        line = f"{pre} planted recall {mode} (n={len(b_on)}, span {cfg.eval_planted_len}, cue {cfg.eval_planted_cue}): beyond on {b_on.mean():.3f}"
        if 0.0 not in scales:
            log(line + f" | within on {w_on.mean():.3f}")
            continue
        b_off, w_off = arr[("beyond", mode, 0.0)], arr[("within", mode, 0.0)]
        n_on, n_off = arr[("none", mode, 1.0)], arr[("none", mode, 0.0)]
        g = b_off - b_on
        se = float(g.std(ddof=1) / np.sqrt(len(g))) if len(g) > 1 else float("nan")
        rec_g = g - (n_off - n_on)
        rse = float(rec_g.std(ddof=1) / np.sqrt(len(rec_g))) if len(rec_g) > 1 else float("nan")
        ceil = float(b_off.mean() - w_off.mean())
        rec = float(g.mean() / ceil) if ceil > 0.01 else float("nan")
        out.update({f"eval/planted_{mode}_recall": float(rec_g.mean()), f"eval/planted_{mode}_recall_se": rse,
                    f"eval/planted_{mode}_gain": float(g.mean()), f"eval/planted_{mode}_gain_se": se, f"eval/planted_{mode}_ceiling": ceil})
        if np.isfinite(rec):
            out[f"eval/planted_{mode}_recovered"] = rec
        log(line + f" off {b_off.mean():.3f} gain {g.mean():+.4f} (se {se:.4f}) | within on {w_on.mean():.3f} off {w_off.mean():.3f} | "
            f"copy ceiling {ceil:+.3f} recovered " + (f"{100 * rec:.1f}%" if np.isfinite(rec) else "n/a (no copy ceiling)")
            + f" | unplanted gain {float((n_off - n_on).mean()):+.4f} -> recall {float(rec_g.mean()):+.4f} (se {rse:.4f})")
        log(f"{pre} planted recall {mode} gain by source: " + " | ".join(f"{s_} {g[nm == s_].mean():+.3f}" for s_ in dict.fromkeys(names)))
    eval_dir = cfg.log_dir or os.environ.get("DTTT_LOG_DIR", os.environ.get("TTT_LOG_DIR", ""))
    if eval_dir and is_main:
        os.makedirs(eval_dir, exist_ok=True)
        np.savez_compressed(os.path.join(eval_dir, f"eval_{step}_planted.npz"), sources=nm,
                            **{f"{pl}_{mode}_x{sc:g}": v for (pl, mode, sc), v in arr.items()})
    return out
