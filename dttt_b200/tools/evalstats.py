"""Statistics shared by the offline comparison tools: weighted means with their standard errors, the
document-cluster bootstrap, the recipe-mix weighting of per-source means, run-directory lookup.

The functionals follow the reference's ``tools/paired_diff.py`` (weighted SE ``:44-47``, cluster bootstrap ``:50-63``,
mix statistic ``:66-91``) so numbers are comparable, but the bootstrap is vectorised: per cluster the sums
``sum(w x)`` and ``sum(w)`` are formed once and every replicate is a multinomial count vector times those sums.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Optional, Tuple

import numpy as np

N_BOOT = 2000
SEED = 12345


def weighted_mean(x: np.ndarray, w: Optional[np.ndarray] = None) -> float:
    x = np.asarray(x, np.float64)
    w = np.ones_like(x) if w is None else np.asarray(w, np.float64)
    return float((x * w).sum() / w.sum())


def weighted_se(x: np.ndarray, w: Optional[np.ndarray] = None) -> float:
    """Standard error of the ``w``-weighted mean of independent draws ``x``."""
    x = np.asarray(x, np.float64)
    w = np.ones_like(x) if w is None else np.asarray(w, np.float64)
    n = len(x)
    if n < 2:
        return float("nan")
    p = w / w.sum()
    mu = (p * x).sum()
    return float(np.sqrt((p ** 2 * (x - mu) ** 2).sum() * n / (n - 1)))


def _cluster_sums(x, w, clusters):
    ids, inv = np.unique(clusters, return_inverse=True)
    sx = np.bincount(inv, weights=x * w, minlength=len(ids))
    sw = np.bincount(inv, weights=w, minlength=len(ids))
    return sx, sw


def bootstrap_means(x, clusters, w=None, n_boot: int = N_BOOT, rng=None) -> np.ndarray:
    """``n_boot`` replicates of the weighted mean of ``x`` with whole clusters resampled with replacement.  A single
    cluster has no between-cluster spread: its members are resampled instead."""
    x = np.asarray(x, np.float64)
    w = np.ones_like(x) if w is None else np.asarray(w, np.float64)
    clusters = np.asarray(clusters)
    if len(np.unique(clusters)) < 2:
        clusters = np.arange(len(x))
    sx, sw = _cluster_sums(x, w, clusters)
    rng = np.random.default_rng(SEED) if rng is None else rng
    k = len(sx)
    counts = rng.multinomial(k, np.full(k, 1.0 / k), size=n_boot).astype(np.float64)
    return (counts @ sx) / (counts @ sw)


def cluster_se(x, clusters, w=None, n_boot: int = N_BOOT) -> float:
    if len(x) < 2:
        return float("nan")
    return float(bootstrap_means(x, clusters, w, n_boot).std(ddof=1))


def mix_stat(x, sources, docs, weights: Dict[str, float], tokw=None, n_boot: int = N_BOOT) -> Tuple[float, float, float]:
    """Mix-weighted mean over the training sources (weight > 0) of the per-source weighted means of ``x``; its naive SE
    (independent sequences) and its SE under resampling of documents within every source."""
    x = np.asarray(x, np.float64)
    sources = np.asarray(sources).astype(str)
    tw = np.ones_like(x) if tokw is None else np.asarray(tokw, np.float64)
    names = [s for s in dict.fromkeys(sources) if weights.get(s, 0.0) > 0]
    if not names:
        return float("nan"), float("nan"), float("nan")
    tot = sum(weights[s] for s in names)
    rng = np.random.default_rng(SEED)
    mean, var, boots = 0.0, 0.0, np.zeros(n_boot)
    for s in names:
        m = sources == s
        share = weights[s] / tot
        mean += share * weighted_mean(x[m], tw[m])
        se = weighted_se(x[m], tw[m])
        var += (share * (0.0 if np.isnan(se) else se)) ** 2
        boots += share * bootstrap_means(x[m], np.asarray(docs)[m], tw[m], n_boot, rng)
    return mean, float(np.sqrt(var)), float(boots.std(ddof=1))


def mix_weights(run_dir: str) -> Dict[str, float]:
    """Source weights of a run: from ``train_config.json`` when the directory has one, else from the
    ``[ttt] config ... sources=name=path:weight,...`` line of ``train_main.log``."""
    for name in ("train_config.json",):
        p = os.path.join(run_dir, name)
        if os.path.exists(p):
            spec = json.load(open(p)).get("sources", "")
            if spec:
                return parse_sources(spec)
    log = os.path.join(run_dir, "train_main.log")
    if os.path.exists(log):
        m = re.search(r"\[ttt\] config .*?sources=(\S+)", open(log, errors="replace").read())
        if m:
            return parse_sources(m.group(1))
    return {}


def parse_sources(spec: str) -> Dict[str, float]:
    out = {}
    for item in spec.split(","):
        if "=" not in item:
            continue
        name, rest = item.split("=", 1)
        try:
            out[name] = float(rest.rsplit(":", 1)[1])
        except (IndexError, ValueError):
            out[name] = 1.0
    return out


def load_npz(path: str) -> Dict[str, np.ndarray]:
    d = np.load(path, allow_pickle=True)
    return {k: d[k] for k in d.files}


def find_file(run_dir: str, rel: str) -> Optional[str]:
    """``rel`` inside ``run_dir`` or inside its newest ``posteval_*`` directory."""
    p = os.path.join(run_dir, rel)
    if os.path.exists(p):
        return p
    subs = sorted(d for d in os.listdir(run_dir) if d.startswith("posteval_")) if os.path.isdir(run_dir) else []
    for d in reversed(subs):
        p = os.path.join(run_dir, d, rel)
        if os.path.exists(p):
            return p
    return None


# ------------------------------------------------------------------------------------------------ paired agreement tables
def agreement(x, y) -> Dict[str, float]:
    """How two measurements of the same items agree: both means, the mean shift, quantiles of the absolute difference and
    the correlation (NaN when either side is constant)."""
    x, y = np.asarray(x, np.float64), np.asarray(y, np.float64)
    gap = np.abs(y - x)
    varies = x.std() > 0 and y.std() > 0
    return {"mean A": x.mean(), "mean B": y.mean(), "B - A": (y - x).mean(), "|d| p50": np.median(gap), "|d| p99": np.quantile(gap, 0.99),
            "|d| max": gap.max(), "corr": np.corrcoef(x, y)[0, 1] if varies else float("nan")}


def text_table(rows: Dict[str, Dict[str, float]], first: str = "", digits: int = 5, signed=("B - A",)) -> str:
    """Rows of named numbers as an aligned text table; ``rows`` maps a label to ``{column: value}`` (same columns each)."""
    if not rows:
        return ""
    cols = list(next(iter(rows.values())))
    wide = max([len(first)] + [len(k) for k in rows]) + 2
    cell = lambda c, v: f"{v:+.{digits}f}" if c in signed else f"{v:.{digits}f}"
    lines = [first.ljust(wide) + "".join(c.rjust(digits + 8) for c in cols)]
    lines += [label.ljust(wide) + "".join(cell(c, r[c]).rjust(digits + 8) for c in cols) for label, r in rows.items()]
    return "\n".join(lines)
