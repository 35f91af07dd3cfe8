"""Paired comparison of runs on the post-training evaluation suite, section by section: for every pair ``A-B`` the
differences A - B with paired standard errors.

    python -m dttt_b200.tools.round_compare --step 179000 M=log/method P=log/plain --pairs M-P

    8K        eval_<step>.npz (written during training): mix-weighted headline (write on), no-write twin and write gain,
              document-cluster bootstrap SE (``tools.paired_diff``)
    32K       eval32k/eval_0.npz: the same at 32K
    distance  distance_32k.npz, distance_128k.npz (``tools.j_lens.memory_distance``): recall of a planted span by distance
              as a share of the copy ceiling, for the own read and the isolated memory, and the memory's general gain
    context   cl_32k.npz, cl_128k.npz (``tools.j_lens.context_learning``): share = recall / ceiling per task and distance,
              and the answers exactly right under the memory
    bound     elbo.npz (``tools.elbo_eval``): the likelihood bound with the write on and off and the memory's part
    noise     noise_*.json (``tools.grad_noise``): B_simple as recorded (not paired)

A run is ``NAME=DIR[@STEP]``; files are looked up in ``DIR`` or in its newest ``posteval_*`` sub-directory; a missing file
skips its section.  Sequences are aligned per source in order (the shared ones are compared).  Pure numpy.  Role of
the reference's ``tools/round_compare.py:1-235``.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import evalstats as S

READS = ("own", "write", "ctx", "isolated")          # last axis of gain_copy / gain_none in the distance files


def parse_run(spec: str, default_step: int) -> Tuple[str, str, int]:
    name, rest = spec.split("=", 1)
    if "@" in rest:
        d, st = rest.rsplit("@", 1)
        return name, d, int(st)
    return name, rest, default_step


def align(a: Dict[str, np.ndarray], b: Dict[str, np.ndarray]):
    """Index arrays picking, per source and in order, the sequences both files scored."""
    sa, sb = a["sources"].astype(str), b["sources"].astype(str)
    ia, ib = [], []
    for s in dict.fromkeys(sa):
        xa, xb = np.where(sa == s)[0], np.where(sb == s)[0]
        n = min(len(xa), len(xb))
        ia.append(xa[:n]); ib.append(xb[:n])
    return np.concatenate(ia), np.concatenate(ib)


def boot_se(x: np.ndarray, n_boot: int = S.N_BOOT) -> float:
    return S.cluster_se(x, np.arange(len(x)), None, n_boot)


def section_eval(title, rel, runs, pairs, steps, out):
    files = {n: S.find_file(d, rel.format(step=steps[n])) for n, d in runs.items()}
    if not any(files.values()):
        return
    out(f"\n## {title}")
    data = {n: S.load_npz(p) for n, p in files.items() if p}
    for a, b in pairs:
        if a not in data or b not in data:
            continue
        ia, ib = align(data[a], data[b])
        w = S.mix_weights(runs[b]) or {s: 1.0 for s in np.unique(data[b]["sources"].astype(str))}
        src, docs = data[b]["sources"][ib], data[b]["doc_ids"][ib] if "doc_ids" in data[b] else np.arange(len(ib))
        tok = data[b]["mask"][ib] if "mask" in data[a] and "mask" in data[b] else None
        cells = []
        for k, label in (("loss_1.0", "headline"), ("loss_0.0", "no-write twin"), ("gain", "write gain")):
            if k in data[a] and k in data[b]:
                m, _, se = S.mix_stat(data[a][k][ia] - data[b][k][ib], src, docs, w, tok)
                cells.append(f"{label} {m:+.4f} ±{se:.4f}")
        out(f"  {a} - {b} ({len(ia)} sequences): " + " | ".join(cells))
        for s in dict.fromkeys(src.astype(str)):
            if w.get(s, 0) == 0 and "loss_1.0" in data[a]:
                m_ = src.astype(str) == s
                d = data[a]["loss_1.0"][ia][m_] - data[b]["loss_1.0"][ib][m_]
                out(f"    {s} (evaluation only): {d.mean():+.4f} ±{S.cluster_se(d, docs[m_]):.4f}")


def section_distance(rel, runs, pairs, out):
    data = {n: S.load_npz(p) for n, d in runs.items() if (p := S.find_file(d, rel))}
    if not data:
        return
    out(f"\n## distance ({rel})")
    for a, b in pairs:
        if a not in data or b not in data:
            continue
        da, db = data[a], data[b]
        n = min(len(da["gain_copy"]), len(db["gain_copy"]))
        for ri in (0, 3):
            sa = 100 * da["gain_copy"][:n, :, ri] / np.maximum(da["ceiling"][:n], 1e-9)
            sb = 100 * db["gain_copy"][:n, :, ri] / np.maximum(db["ceiling"][:n], 1e-9)
            row = " ".join(f"d={int(dd)}: {(sa[:, j] - sb[:, j]).mean():+.1f}±{boot_se(sa[:, j] - sb[:, j], 500):.1f}" for j, dd in enumerate(da["dist"]))
            out(f"  {a} - {b} recall, % of copy ceiling ({READS[ri]}): {row}")
        if "general_gain" in da and "general_gain" in db:
            g = da["general_gain"][:n] - db["general_gain"][:n]
            out(f"  {a} - {b} memory's general gain: {g.mean():+.4f} ±{boot_se(g, 500):.4f} nats")


def section_context(rel, runs, pairs, out):
    data = {n: S.load_npz(p) for n, d in runs.items() if (p := S.find_file(d, rel))}
    if not data:
        return
    out(f"\n## context ({rel})")
    for a, b in pairs:
        if a not in data or b not in data:
            continue
        da, db = data[a], data[b]
        n = min(len(da["recall"]), len(db["recall"]))
        for ti, task in enumerate(da["tasks"].astype(str)):
            sa = 100 * da["recall"][:n, ti] / np.maximum(da["ceiling"][:n, ti], 1e-9)
            sb = 100 * db["recall"][:n, ti] / np.maximum(db["ceiling"][:n, ti], 1e-9)
            row = " ".join(f"d={int(dd)}: {(sa[:, j] - sb[:, j]).mean():+.1f}±{boot_se(sa[:, j] - sb[:, j], 500):.1f}" for j, dd in enumerate(da["dist"]))
            ex = (da["exact"][:n, ti].mean() - db["exact"][:n, ti].mean()) * 100 if "exact" in da and "exact" in db else float("nan")
            out(f"  {a} - {b} {task}: share % {row} | exactly right {ex:+.1f} points")


def section_bound(runs, pairs, out):
    data = {n: S.load_npz(p) for n, d in runs.items() if (p := S.find_file(d, "elbo.npz"))}
    if not data:
        return
    out("\n## bound (elbo.npz)")
    per_seq = lambda d, si: (d["ce"][:, si] / np.maximum(d["count"][:, si], 1)).mean(0)            # [n_seq]
    for a, b in pairs:
        if a not in data or b not in data:
            continue
        da, db = data[a], data[b]
        n = min(da["ce"].shape[-1], db["ce"].shape[-1])
        on = per_seq(da, 0)[:n] - per_seq(db, 0)[:n]
        line = f"  {a} - {b}: write on {on.mean():+.4f} ±{boot_se(on, 500):.4f}"
        if da["ce"].shape[1] > 1 and db["ce"].shape[1] > 1:
            off = per_seq(da, 1)[:n] - per_seq(db, 1)[:n]
            mem = (per_seq(da, 1) - per_seq(da, 0))[:n] - (per_seq(db, 1) - per_seq(db, 0))[:n]
            line += f" | off {off.mean():+.4f} ±{boot_se(off, 500):.4f} | memory's part {mem.mean():+.4f} ±{boot_se(mem, 500):.4f}"
        out(line)


def section_noise(runs, out):
    rows = []
    for n, d in runs.items():
        for p in sorted(glob.glob(os.path.join(d, "noise_*.json")) + glob.glob(os.path.join(d, "posteval_*", "noise_*.json"))):
            r = json.load(open(p))
            rows.append(f"  {n} {os.path.basename(p)}: " + " | ".join(f"{k} B_simple {v['total']['B_simple']:.1f} share {v['total']['share']:.2f}"
                                                                   for k, v in r.items() if k.startswith("views_")))
    if rows:
        out("\n## noise (as recorded, not paired)")
        for r in rows:
            out(r)


def main(argv=None, out=print) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.round_compare")
    ap.add_argument("runs", nargs="+", help="NAME=DIR[@STEP]")
    ap.add_argument("--step", type=int, default=0)
    ap.add_argument("--pairs", default="", help="comma-separated A-B; default: every later run against the first")
    a = ap.parse_args(argv)
    parsed = [parse_run(r, a.step) for r in a.runs]
    runs = {n: d for n, d, _ in parsed}
    steps = {n: s for n, _, s in parsed}
    names = list(runs)
    pairs = [tuple(p.split("-", 1)) for p in a.pairs.split(",") if p] or [(n, names[0]) for n in names[1:]]
    section_eval("8K (training-time evaluation)", "eval_{step}.npz", runs, pairs, steps, out)
    section_eval("32K", os.path.join("eval32k", "eval_0.npz"), runs, pairs, steps, out)
    for rel in ("distance_32k.npz", "distance_128k.npz"):
        section_distance(rel, runs, pairs, out)
    for rel in ("cl_32k.npz", "cl_128k.npz"):
        section_context(rel, runs, pairs, out)
    section_bound(runs, pairs, out)
    section_noise(runs, out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
