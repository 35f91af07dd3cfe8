"""Deterministic inner targets chosen on the host from the tokens themselves.

``rare``: per chunk the ``target_frac`` least frequent tokens (corpus unigram counts), ties by a position
hash.  ``docaware``: tokens whose 3-gram already occurred earlier in the same document first, then the rare
tercile, then the rest, with a ``generic_floor`` share of slots reserved for hash-chosen tokens.  Pad and
EOS are never targets.  ``split_perm`` gives the split task's per-chunk physical order
``[context (natural order) | targets (shuffled)]`` (reference ``src/ttt/inner_masks.py:30-120``; the scores,
hashes and generators are the reference's so both implementations choose the same targets).
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np

MODES = ("random", "rare", "docaware")
_U = np.uint64


def position_hash(n: int, seed: int) -> np.ndarray:
    x = (np.arange(n, dtype=np.uint64) + _U(seed) * _U(0x9E3779B97F4A7C15)) & _U(0xFFFFFFFFFFFFFFFF)
    x ^= x >> _U(33)
    x *= _U(0xFF51AFD7ED558CCD)
    x ^= x >> _U(33)
    return (x & _U(0xFFFFFF)).astype(np.float64) / float(1 << 24)


def trigram_recurs(tokens: np.ndarray, eos: int, prefix: Optional[np.ndarray] = None) -> np.ndarray:
    """``[T]`` bool: the 3-gram ending here occurred earlier in the same document."""
    seq = tokens.astype(np.int64) if prefix is None else np.concatenate([prefix.astype(np.int64), tokens.astype(np.int64)])
    n, off = len(seq), (0 if prefix is None else len(prefix))
    h = seq.copy()
    h = h * 1_000_003 + np.concatenate([[-7], seq[:-1]])
    h = h * 1_000_003 + np.concatenate([[-7, -7], seq[:-2]])
    key = (h & 0x7FFFFFFFFFFFFFFF) * 4099 + np.cumsum(seq == eos)
    order = np.lexsort((np.arange(n), key))
    ks = key[order]
    seen = np.zeros(n, bool)
    seen[order[1:][ks[1:] == ks[:-1]]] = True
    seen[:2] = False
    return seen[off:]


def _topk_per_chunk(score: np.ndarray, chunk: int, k: int) -> np.ndarray:
    T = len(score)
    mask = np.zeros(T, bool)
    for c in range(T // chunk):
        sl = score[c * chunk:(c + 1) * chunk]
        idx = np.argsort(-sl, kind="stable")[:k]
        mask[c * chunk + idx[np.isfinite(sl[idx])]] = True
    return mask


def inner_mask_rule(tokens: np.ndarray, mode: str, chunk: int, eos: int, pad: int, unigram: Optional[np.ndarray] = None,
                    target_frac: float = 0.5, generic_floor: float = 0.1, seed: int = 0,
                    prefix: Optional[np.ndarray] = None) -> np.ndarray:
    if mode == "random":
        raise ValueError("random masks are drawn from the step key, not on the host")
    T = len(tokens)
    h01 = position_hash(T, seed)
    score = h01 * 0.1
    if unigram is not None:
        ids = np.clip(tokens, 0, len(unigram) - 1)
        rank = np.argsort(np.argsort(unigram[ids].astype(np.float64)))
        score += 1.0 - rank / max(T - 1, 1)
        if mode == "docaware":
            order = np.argsort(-unigram)
            before = np.cumsum(unigram[order]) - unigram[order]
            rare = np.zeros(len(unigram), bool)
            rare[order[before >= 2 * unigram.sum() / 3]] = True
            score += 1.0 * rare[ids]
    if mode == "docaware":
        score += 3.0 * trigram_recurs(tokens, eos, prefix)
    if generic_floor > 0:
        score += 10.0 * (h01 < generic_floor * target_frac)
    score = np.where((tokens == pad) | (tokens == eos), -np.inf, score)
    return _topk_per_chunk(score, chunk, int(round(target_frac * chunk)))


def split_perm(tokens: np.ndarray, mode: str, chunk: int, eos: int, pad: int, context_frac: float = 0.5,
               unigram: Optional[np.ndarray] = None, generic_floor: float = 0.1, seed: int = 0,
               prefix: Optional[np.ndarray] = None) -> np.ndarray:
    T = len(tokens)
    K = int(round(context_frac * chunk))
    if mode == "random":
        targets = _topk_per_chunk(position_hash(T, seed), chunk, chunk - K)
    else:
        targets = inner_mask_rule(tokens, mode, chunk, eos, pad, unigram, 1.0 - K / chunk, generic_floor, seed, prefix)
    gen = np.random.default_rng([seed, int(np.bitwise_xor.reduce(tokens.astype(np.int64)[:min(T, 64)]) & 0x7FFFFFFF)])
    perm = np.zeros(T, np.int32)
    for c in range(T // chunk):
        base = c * chunk
        t = np.flatnonzero(targets[base:base + chunk])
        ctx = np.setdiff1d(np.arange(chunk), t)
        while len(t) < chunk - K:                       # pad/eos-only chunks: fill from the context's tail
            t, ctx = np.append(t, ctx[-1]), ctx[:-1]
        perm[base:base + chunk] = base + np.concatenate([ctx, gen.permutation(t)])
    return perm


class MaskMaker:
    """Host-side inner masks (mask task) or permutations (split task) for a batch; ``None`` when the masks are
    the random ones drawn from the step key (reference data.py:852-877)."""

    def __init__(self, mode: str, chunk: int, eos: int, pad: int, unigram_path: str = "", target_frac: float = 0.5,
                 generic_floor: float = 0.1, seed: int = 0, task: str = "mask"):
        self.mode, self.chunk, self.eos, self.pad, self.task = mode, chunk, eos, pad, task
        self.target_frac, self.generic_floor, self.seed = target_frac, generic_floor, seed
        self.unigram = None
        if (mode != "random" or task == "split") and unigram_path and os.path.exists(unigram_path):
            self.unigram = np.fromfile(unigram_path, dtype=np.int64)

    @property
    def active(self) -> bool:
        return self.task == "split" or self.mode != "random"

    def __call__(self, ids: np.ndarray) -> Optional[np.ndarray]:
        if self.task == "split":
            return np.stack([split_perm(r, self.mode, self.chunk, self.eos, self.pad, 1.0 - self.target_frac, self.unigram,
                                        self.generic_floor, self.seed) for r in ids])
        if self.mode == "random":
            return None
        return np.stack([inner_mask_rule(r, self.mode, self.chunk, self.eos, self.pad, self.unigram, self.target_frac,
                                         self.generic_floor, self.seed) for r in ids])
