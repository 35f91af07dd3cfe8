"""Evaluation probes on the host: which tokens does the memory help?

Given per-token cross-entropies of the write-on and write-off twins, every scored token gets a class and the
write gain ``CE_off - CE_on`` is aggregated per class (reference ``src/ttt/probes.py``):

* P1 recurrence (``recurrence_classes``): did the token's 4-gram occur earlier in the same document -
  ``within`` the attention window of its chunk, ``beyond`` it (inside the sequence), only before the sequence
  (``pre_seq``), or never (``novel``)?  Only the most recent earlier occurrence matters: if it is outside the
  window so is every older one, so the class is read off one "previous occurrence" array without a chain walk.
* P2 rarity (``rarity_bins``): terciles of the unigram token mass.
* P3 neighbours (``neighbour_classes``): left / right neighbour visible or masked in the outer stream.

``planted_probe_batch`` / ``recall_train_batch`` build the planted-recall inputs (a span copied beyond the
attention window, its tail after a visible cue scored); draws are keyed ``(seed, 7, j)`` / ``(seed, 11, j)`` as
in the reference so all variants and checkpoints are paired.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import numpy as np

P1_CLASSES = ("beyond", "within", "novel", "pre_seq")
P2_CLASSES = ("frequent", "mid", "rare")
P3_CLASSES = ("Lv_Rv", "Lv_Rm", "Lm_Rv", "Lm_Rm")
PLANT_PLACEMENTS = ("beyond", "within", "none")
PLANT_MODES = ("block", "alt")


def rarity_bins(counts: np.ndarray) -> np.ndarray:
    order = np.argsort(-counts.astype(np.int64), kind="stable")
    sc = counts[order].astype(np.float64)
    before = np.cumsum(sc) - sc
    total = sc.sum() if sc.sum() > 0 else 1.0
    out = np.empty(len(counts), np.int8)
    out[order] = np.where(before < total / 3, 0, np.where(before < 2 * total / 3, 1, 2)).astype(np.int8)
    out[counts == 0] = 2
    return out


def ngram_hash(tokens: np.ndarray, n: int = 4) -> np.ndarray:
    t = tokens.astype(np.int64)
    h = np.zeros_like(t)
    for k in range(n):
        h = h * 1_000_003 + np.concatenate([np.full(k, -7, np.int64), t[:len(t) - k]])
    h &= 0x7FFFFFFFFFFFFFFF
    h[:n - 1] = -1
    return h


def recurrence_classes(context: np.ndarray, seq_start: int, seq_len: int, doc_starts: np.ndarray, chunk: int,
                       window_chunks: int, n: int = 4) -> np.ndarray:
    """``[seq_len]`` int8 P1 class (0 beyond, 1 within, 2 novel, 3 pre_seq) of ``context[seq_start : seq_start+seq_len]``."""
    h = ngram_hash(context, n)
    L = len(context)
    order = np.lexsort((np.arange(L), h))
    prev = np.full(L, -1, np.int64)
    same = h[order][1:] == h[order][:-1]
    prev[order[1:][same]] = order[:-1][same]
    ds = np.sort(doc_starts)
    doc_of = ds[np.searchsorted(ds, np.arange(L), side="right") - 1]
    pos = seq_start + np.arange(seq_len)
    j = prev[pos]
    has = (h[pos] >= 0) & (j >= 0) & (j >= doc_of[pos])
    win = seq_start + (np.arange(seq_len) // chunk - window_chunks) * chunk
    within = has & (j >= win) & (j >= seq_start)
    beyond = has & ~within & (j >= seq_start)
    pre = has & ~within & ~beyond
    cls = np.full(seq_len, 2, np.int8)
    cls[within], cls[beyond], cls[pre] = 1, 0, 3
    return cls


def neighbour_classes(scored: np.ndarray) -> np.ndarray:
    s = scored.astype(bool)
    left, right = np.ones_like(s), np.ones_like(s)
    left[:, 1:], right[:, :-1] = s[:, :-1], s[:, 1:]
    return (2 * left + right).astype(np.int8)


def aggregate(ce_on: np.ndarray, ce_off: np.ndarray, scored: np.ndarray, labels: np.ndarray, n_classes: int,
              chunk: int) -> Dict[str, np.ndarray]:
    B, T = ce_on.shape
    nc = T // chunk
    g = ce_off - ce_on
    out = {"n": np.zeros(n_classes, np.int64), "loss": np.zeros(n_classes), "gain": np.zeros(n_classes),
           "seq_gain": np.full((n_classes, B), np.nan), "gain_by_chunk": np.zeros((n_classes, nc)),
           "n_by_chunk": np.zeros((n_classes, nc), np.int64)}
    for k in range(n_classes):
        m = scored & (labels == k)
        n = int(m.sum())
        out["n"][k] = n
        if not n:
            continue
        out["loss"][k], out["gain"][k] = float(ce_on[m].mean()), float(g[m].mean())
        per = m.sum(1)
        out["seq_gain"][k] = np.where(per > 0, (g * m).sum(1) / np.maximum(per, 1), np.nan)
        mc = m.reshape(B, nc, chunk)
        cnt = mc.sum((0, 2))
        out["n_by_chunk"][k] = cnt
        out["gain_by_chunk"][k] = np.where(cnt > 0, (g.reshape(B, nc, chunk) * mc).sum((0, 2)) / np.maximum(cnt, 1), 0.0)
    return out


def se_over_sequences(seq_gain: np.ndarray) -> float:
    v = seq_gain[~np.isnan(seq_gain)]
    return float(v.std(ddof=1) / np.sqrt(len(v))) if len(v) > 1 else float("nan")


def planted_chunks(n_chunks: int, window: int, target: Optional[int] = None) -> Tuple[int, int, int]:
    ct = window + 3 if target is None else int(target)
    if ct < window + 3:
        raise ValueError(f"planted recall: the target chunk {ct} must be >= window + 3 = {window + 3}")
    if n_chunks < ct + 1:
        raise ValueError(f"planted recall needs >= {ct + 1} chunks (window {window}), the sequence has {n_chunks}")
    return 1, ct, ct - 1


def planted_probe_batch(local: np.ndarray, j_global: Sequence[int], seed: int, chunk: int, window: int, length: int, cue: int,
                        placement: str, mode: str, eos: Optional[int] = None, tries: int = 8,
                        target: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    if placement not in PLANT_PLACEMENTS or mode not in PLANT_MODES:
        raise ValueError(f"placement {placement!r} / mode {mode!r}")
    if not 0 < cue < length <= chunk:
        raise ValueError(f"need 0 < cue ({cue}) < length ({length}) <= chunk ({chunk})")
    B, T = local.shape
    cs, ct, cw = planted_chunks(T // chunk, window, target)
    ids = np.array(local, dtype=np.int32, copy=True)
    lm = np.zeros((B, T), bool)
    for r, j in enumerate(j_global):
        gen = np.random.default_rng([seed, 7, int(j)])
        for _ in range(tries):
            a, b, w = (c * chunk + int(gen.integers(0, chunk - length + 1)) for c in (cs, ct, cw))
            if eos is None or not any((local[r, o:o + length] == eos).any() for o in (a, b, w)):
                break
        span = local[r, a:a + length]
        if placement != "none":
            ids[r, b:b + length] = span
        if placement == "within":
            ids[r, w:w + length] = span
        scored = np.arange(b + cue, b + length)
        lm[r, scored if mode == "block" else scored[1::2]] = True
    return ids, lm


def recall_train_batch(local: np.ndarray, j_global: Sequence[int], seed: int, chunk: int, window: int, len_min: int,
                       len_max: int, cue: int, eos: Optional[int] = None, tries: int = 8) -> Tuple[np.ndarray, np.ndarray]:
    B, T = local.shape
    nc = T // chunk
    if nc < window + 2 or not 0 < cue < len_min <= len_max <= chunk:
        raise ValueError("recall_train_batch: need >= window + 2 chunks and 0 < cue < len_min <= len_max <= chunk")
    ids = np.array(local, dtype=np.int32, copy=True)
    lm = np.zeros((B, T), bool)
    for r, j in enumerate(j_global):
        gen = np.random.default_rng([seed, 11, int(j)])
        block = gen.random() < 0.5
        for _ in range(tries):
            L = int(gen.integers(len_min, len_max + 1))
            cs = int(gen.integers(0, nc - window - 1))
            ct = int(gen.integers(cs + window + 1, nc))
            a = cs * chunk + int(gen.integers(0, chunk - L + 1))
            b = ct * chunk + int(gen.integers(0, chunk - L + 1))
            if eos is None or not ((local[r, a:a + L] == eos).any() or (local[r, b:b + L] == eos).any()):
                ids[r, b:b + L] = local[r, a:a + L]
                scored = np.arange(b + cue, b + L)
                lm[r, scored if block else scored[1::2]] = True
                break
    return ids, lm
