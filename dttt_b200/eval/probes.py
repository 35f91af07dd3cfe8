"""Evaluation probes on the host: which tokens does the memory help?

From the per-token cross-entropies of the write-on and write-off twins, every scored token gets a class and the write gain
``CE_off - CE_on`` is aggregated per class.  The three classifications and the record layout are those of the reference's
``src/ttt/probes.py`` (so that evaluation records of both code bases can be compared), computed here with vectorised numpy:

* P1 recurrence (``recurrence_classes``): has the 4-gram ending at the token occurred earlier in the same document, and where
  is its most recent earlier occurrence: ``within`` the attention window of the token's chunk, ``beyond`` the window but inside
  the sequence, only before the sequence (``pre_seq``), or nowhere (``novel``)?  Only the most recent occurrence matters: when it
  is outside the window, so is every older one.
* P2 rarity (``rarity_bins``): thirds of the unigram token mass, most frequent tokens first.
* P3 neighbours (``neighbour_classes``): is the left / right neighbour visible or masked in the outer stream?

``planted_probe_batch`` / ``recall_train_batch`` build the planted-recall inputs (a span copied to a chunk beyond the attention
window; after a visible cue its tail is scored).  Their random draws are keyed by ``(seed, 7, j)`` / ``(seed, 11, j)`` with the
global row index ``j`` and consume the generator in a fixed order, so every variant and checkpoint sees the same plants.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import numpy as np

P1_CLASSES = ("beyond", "within", "novel", "pre_seq")
P2_CLASSES = ("frequent", "mid", "rare")
P3_CLASSES = ("Lv_Rv", "Lv_Rm", "Lm_Rv", "Lm_Rm")
PLANT_PLACEMENTS = ("beyond", "within", "none")
PLANT_MODES = ("block", "alt")

_BEYOND, _WITHIN, _NOVEL, _PRE_SEQ = range(4)


# ---------------------------------------------------------------------------------------------------- classifications
def rarity_bins(counts: np.ndarray) -> np.ndarray:
    """Per vocabulary entry 0 / 1 / 2 = frequent / mid / rare: walking the vocabulary from the most frequent token down, an entry
    belongs to the third of the total mass in which its own mass STARTS; tokens that never occur are rare."""
    c = np.asarray(counts).astype(np.float64)
    rank = np.argsort(-np.asarray(counts).astype(np.int64), kind="stable")
    mass_before = np.concatenate([[0.0], np.cumsum(c[rank])[:-1]])
    total = float(c.sum()) or 1.0
    third = np.searchsorted(np.array([total / 3.0, 2.0 * total / 3.0]), mass_before, side="right")
    bins = np.empty(len(c), np.int8)
    bins[rank] = third.astype(np.int8)
    bins[np.asarray(counts) == 0] = 2
    return bins


def ngram_hash(tokens: np.ndarray, n: int = 4) -> np.ndarray:
    """A 63-bit fingerprint of the ``n``-gram ending at every position (``-1`` where fewer than ``n`` tokens precede it)."""
    t = np.asarray(tokens).astype(np.uint64)
    L = len(t)
    out = np.full(L, -1, np.int64)
    if L < n:
        return out
    grams = np.lib.stride_tricks.sliding_window_view(t, n)                      # [L - n + 1, n], oldest token first
    mult = np.uint64(0x9E3779B97F4A7C15)
    acc = np.zeros(len(grams), np.uint64)
    with np.errstate(over="ignore"):
        for k in range(n):
            acc = (acc ^ (grams[:, k] + np.uint64(k + 1))) * mult
            acc ^= acc >> np.uint64(29)
    out[n - 1:] = (acc & np.uint64(0x7FFFFFFFFFFFFFFF)).astype(np.int64)
    return out


def _previous_equal(keys: np.ndarray) -> np.ndarray:
    """For every position the largest earlier position holding the same key, else ``-1``."""
    idx = np.argsort(keys, kind="stable")                                       # equal keys keep their order of appearance
    sorted_keys = keys[idx]
    prev = np.full(len(keys), -1, np.int64)
    repeat = np.flatnonzero(sorted_keys[1:] == sorted_keys[:-1]) + 1
    prev[idx[repeat]] = idx[repeat - 1]
    return prev


def recurrence_classes(context: np.ndarray, seq_start: int, seq_len: int, doc_starts: np.ndarray, chunk: int,
                       window_chunks: int, n: int = 4) -> np.ndarray:
    """``[seq_len]`` int8 P1 class (0 beyond, 1 within, 2 novel, 3 pre_seq) of ``context[seq_start : seq_start + seq_len]``;
    ``context`` may start before the sequence (so that ``pre_seq`` can be told from ``novel``), ``doc_starts`` are the offsets in
    ``context`` at which documents begin."""
    fp = ngram_hash(context, n)
    last_seen = _previous_equal(fp)
    starts = np.sort(np.asarray(doc_starts))
    here = seq_start + np.arange(seq_len)
    doc_begin = starts[np.searchsorted(starts, here, side="right") - 1]
    earlier = last_seen[here]
    found = (fp[here] >= 0) & (earlier >= 0) & (earlier >= doc_begin)
    window_begin = seq_start + (np.arange(seq_len) // chunk - window_chunks) * chunk
    in_sequence = earlier >= seq_start
    cls = np.full(seq_len, _NOVEL, np.int8)
    cls[found & ~in_sequence] = _PRE_SEQ
    cls[found & in_sequence & (earlier < window_begin)] = _BEYOND
    cls[found & in_sequence & (earlier >= window_begin)] = _WITHIN
    return cls


def neighbour_classes(scored: np.ndarray) -> np.ndarray:
    """``[B, T]`` int8: ``2 * left_masked + right_masked`` (a neighbour outside the sequence counts as masked)."""
    padded = np.pad(np.asarray(scored).astype(bool), ((0, 0), (1, 1)), constant_values=True)
    return (2 * padded[:, :-2].astype(np.int8) + padded[:, 2:].astype(np.int8)).astype(np.int8)


# ---------------------------------------------------------------------------------------------------- aggregation
def aggregate(ce_on: np.ndarray, ce_off: np.ndarray, scored: np.ndarray, labels: np.ndarray, n_classes: int,
              chunk: int) -> Dict[str, np.ndarray]:
    """Per class: token count ``n``, mean write-on loss, mean gain, per-sequence mean gain ``seq_gain [classes, B]`` (NaN where
    a sequence has no token of the class) and the gain / count by chunk position ``[classes, T / chunk]``."""
    B, T = ce_on.shape
    nc = T // chunk
    gain = np.asarray(ce_off, np.float64) - np.asarray(ce_on, np.float64)
    rows, cols = np.nonzero(scored)
    lab = np.asarray(labels)[rows, cols].astype(np.int64)
    keep = (lab >= 0) & (lab < n_classes)
    rows, cols, lab = rows[keep], cols[keep], lab[keep]
    g, on = gain[rows, cols], np.asarray(ce_on, np.float64)[rows, cols]

    def by(index: np.ndarray, size: int, weights=None) -> np.ndarray:
        return np.bincount(index, weights=weights, minlength=size)[:size]

    n = by(lab, n_classes).astype(np.int64)
    safe = np.maximum(n, 1)
    seq_key, chunk_key = lab * B + rows, lab * nc + cols // chunk
    seq_n = by(seq_key, n_classes * B).reshape(n_classes, B)
    chunk_n = by(chunk_key, n_classes * nc).reshape(n_classes, nc)
    with np.errstate(invalid="ignore", divide="ignore"):
        seq_gain = by(seq_key, n_classes * B, g).reshape(n_classes, B) / seq_n
    seq_gain[seq_n == 0] = np.nan
    chunk_gain = by(chunk_key, n_classes * nc, g).reshape(n_classes, nc) / np.maximum(chunk_n, 1)
    return {"n": n, "loss": np.where(n > 0, by(lab, n_classes, on) / safe, 0.0), "gain": np.where(n > 0, by(lab, n_classes, g) / safe, 0.0),
            "seq_gain": seq_gain, "gain_by_chunk": np.where(chunk_n > 0, chunk_gain, 0.0), "n_by_chunk": chunk_n.astype(np.int64)}


def se_over_sequences(seq_gain: np.ndarray) -> float:
    """Standard error of the mean over the sequences that have a value."""
    have = np.asarray(seq_gain)[np.isfinite(seq_gain)]
    if have.size < 2:
        return float("nan")
    return float(np.std(have, ddof=1) / np.sqrt(have.size))


# ---------------------------------------------------------------------------------------------------- planted recall
def planted_chunks(n_chunks: int, window: int, target: Optional[int] = None) -> Tuple[int, int, int]:
    """Chunk indices ``(source, target, within-window copy)``: the source is chunk 1, the target at least ``window + 3`` (so the
    source has left the attention window with a margin), the optional visible copy sits in the chunk before the target."""
    first_allowed = window + 3
    tgt = first_allowed if target is None else int(target)
    if tgt < first_allowed:
        raise ValueError(f"planted recall: the target chunk {tgt} must be >= window + 3 = {first_allowed}")
    if tgt + 1 > n_chunks:
        raise ValueError(f"planted recall needs >= {tgt + 1} chunks (window {window}), the sequence has {n_chunks}")
    return 1, tgt, tgt - 1


def _contains(row: np.ndarray, start: int, length: int, token: Optional[int]) -> bool:
    return token is not None and bool(np.any(row[start:start + length] == token))


def _mark_scored(mask_row: np.ndarray, start: int, stop: int, every_other: bool) -> None:
    """Score ``[start, stop)``, or with ``every_other`` its second, fourth, ... slot."""
    if every_other:
        mask_row[start + 1:stop:2] = True
    else:
        mask_row[start:stop] = True


def planted_probe_batch(local: np.ndarray, j_global: Sequence[int], seed: int, chunk: int, window: int, length: int, cue: int,
                        placement: str, mode: str, eos: Optional[int] = None, tries: int = 8,
                        target: Optional[int] = None) -> Tuple[np.ndarray, np.ndarray]:
    """``(ids, scored)`` for the evaluation probe: a span of ``length`` tokens from the source chunk is written into the target
    chunk (``placement`` ``beyond``; ``within`` also copies it into the chunk before the target; ``none`` plants nothing and only
    marks the slots).  The first ``cue`` tokens of the plant stay visible, the rest is scored: all of it (``block``) or every
    other token (``alt``).  Offsets are redrawn up to ``tries`` times while a span touches a document boundary (``eos``)."""
    if placement not in PLANT_PLACEMENTS or mode not in PLANT_MODES:
        raise ValueError(f"placement {placement!r} / mode {mode!r}")
    if not (0 < cue < length <= chunk):
        raise ValueError(f"need 0 < cue ({cue}) < length ({length}) <= chunk ({chunk})")
    rows, T = local.shape
    chunks = planted_chunks(T // chunk, window, target)
    ids = np.asarray(local).astype(np.int32, copy=True)
    scored = np.zeros((rows, T), bool)
    room = chunk - length + 1
    for r, j in enumerate(j_global):
        gen = np.random.default_rng([seed, 7, int(j)])
        offsets = (0, 0, 0)
        for _ in range(tries):
            offsets = tuple(c * chunk + int(gen.integers(0, room)) for c in chunks)            # source, target, window copy
            if not any(_contains(local[r], o, length, eos) for o in offsets):
                break
        src, dst, near = offsets
        plant = local[r, src:src + length]
        if placement in ("beyond", "within"):
            ids[r, dst:dst + length] = plant
        if placement == "within":
            ids[r, near:near + length] = plant
        _mark_scored(scored[r], dst + cue, dst + length, every_other=(mode == "alt"))
    return ids, scored


def recall_train_batch(local: np.ndarray, j_global: Sequence[int], seed: int, chunk: int, window: int, len_min: int,
                       len_max: int, cue: int, eos: Optional[int] = None, tries: int = 8) -> Tuple[np.ndarray, np.ndarray]:
    """``(ids, scored)`` for recall training: per row one span of random length copied from a random chunk to a random chunk more
    than ``window`` chunks later, scored after ``cue`` visible tokens (block or every other token, chosen per row); a row whose
    draws all touch a document boundary is left unplanted."""
    rows, T = local.shape
    n_chunks = T // chunk
    if n_chunks < window + 2 or not (0 < cue < len_min <= len_max <= chunk):
        raise ValueError("recall_train_batch: need >= window + 2 chunks and 0 < cue < len_min <= len_max <= chunk")
    ids = np.asarray(local).astype(np.int32, copy=True)
    scored = np.zeros((rows, T), bool)
    for r, j in enumerate(j_global):
        gen = np.random.default_rng([seed, 11, int(j)])
        whole_block = gen.random() < 0.5
        for _ in range(tries):
            span = int(gen.integers(len_min, len_max + 1))
            from_chunk = int(gen.integers(0, n_chunks - window - 1))
            to_chunk = int(gen.integers(from_chunk + window + 1, n_chunks))
            src = from_chunk * chunk + int(gen.integers(0, chunk - span + 1))
            dst = to_chunk * chunk + int(gen.integers(0, chunk - span + 1))
            if _contains(local[r], src, span, eos) or _contains(local[r], dst, span, eos):
                continue
            ids[r, dst:dst + span] = local[r, src:src + span]
            _mark_scored(scored[r], dst + cue, dst + span, every_other=not whole_block)
            break
    return ids, scored
