"""Inner targets chosen on the host from the tokens themselves, identically in training, evaluation and decoding.

A ``TargetRule`` ranks the positions of a sequence and takes the best ``round(target_frac * C)`` of every chunk:

``rare``      the least frequent tokens of the sequence by corpus unigram count;
``docaware``  first the tokens whose 3-gram already occurred earlier in the same document, then tokens of the rare third
              of the corpus mass, then the rest by rarity;

always with a small position-hash jitter as the tie-break and a ``generic_floor`` share of the slots forced to hash-chosen
positions, so that the write is never blind to ordinary tokens.  Pad and EOS are never targets.  The split task's
physical order of a chunk is ``[context in natural order | targets shuffled]``.

The ranking terms, their weights (0.1 jitter, 1 rarity, 1 rare third, 3 recurrence, 10 floor), the 3-gram hash and the
shuffle generator's seeding are those of the reference (``src/ttt/inner_masks.py:30-120``): both implementations must pick
the same targets for the same tokens, which ``tests`` check against recorded vectors.  Everything is computed on whole
``[chunks, C]`` views; nothing loops over chunks except the shuffle, whose generator is consumed chunk by chunk.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

MODES = ("random", "rare", "docaware")
_GOLDEN, _MIX, _LOW24 = np.uint64(0x9E3779B97F4A7C15), np.uint64(0xFF51AFD7ED558CCD), np.uint64(0xFFFFFF)


def position_hash(n: int, seed: int) -> np.ndarray:
    """``[n]`` floats in [0, 1): a pure function of (position, seed)."""
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64) + np.uint64(seed) * _GOLDEN
        x ^= x >> np.uint64(33)
        x *= _MIX
        x ^= x >> np.uint64(33)
    return (x & _LOW24).astype(np.float64) * 2.0 ** -24


def trigram_recurs(tokens: np.ndarray, eos: int, prefix: Optional[np.ndarray] = None) -> np.ndarray:
    """``[T]`` bool: the 3-gram ending at a position was already seen in the same document (documents end at EOS; ``prefix``
    holds what is known before ``tokens``, e.g. the committed blocks while decoding).  Every position is keyed by a 63-bit
    hash of its 3-gram joined with its document number; a position recurs when it is not the first holder of its key."""
    body = np.asarray(tokens, np.int64)
    lead = 0 if prefix is None else len(prefix)
    seq = body if prefix is None else np.concatenate([np.asarray(prefix, np.int64), body])
    back1 = np.concatenate([[-7], seq[:-1]])
    back2 = np.concatenate([[-7, -7], seq[:-2]])
    with np.errstate(over="ignore"):
        gram = (seq * 1_000_003 + back1) * 1_000_003 + back2
        key = (gram & 0x7FFFFFFFFFFFFFFF) * 4099 + np.cumsum(seq == eos)
    _, first, member = np.unique(key, return_index=True, return_inverse=True)
    again = first[member] != np.arange(len(seq))
    again[:2] = False                                             # no complete 3-gram ends at the first two positions
    return again[lead:]


def best_per_chunk(score: np.ndarray, chunk: int, k: int) -> np.ndarray:
    """``[T]`` bool: in every chunk the ``k`` highest finite scores (earlier position first among equals)."""
    table = score.reshape(-1, chunk)
    top = np.argsort(-table, axis=1, kind="stable")[:, :k]
    chosen = np.zeros(table.shape, bool)
    np.put_along_axis(chosen, top, np.isfinite(np.take_along_axis(table, top, axis=1)), axis=1)
    return chosen.reshape(-1)


@dataclass
class TargetRule:
    mode: str
    chunk: int
    eos: int
    pad: int
    unigram: Optional[np.ndarray] = None
    target_frac: float = 0.5
    generic_floor: float = 0.1
    seed: int = 0
    _rare_third: Optional[np.ndarray] = field(default=None, repr=False)

    def rare_third(self) -> np.ndarray:
        """Vocabulary flags: the ids that, taken from the rarest upward, make up the last third of the corpus mass."""
        if self._rare_third is None:
            by_count = np.argsort(-self.unigram)
            mass_before = np.cumsum(self.unigram[by_count]) - self.unigram[by_count]
            flags = np.zeros(len(self.unigram), bool)
            flags[by_count[mass_before >= 2 * self.unigram.sum() / 3]] = True
            self._rare_third = flags
        return self._rare_third

    def scores(self, tokens: np.ndarray, prefix: Optional[np.ndarray] = None, frac: Optional[float] = None) -> np.ndarray:
        if self.mode == "random":
            raise ValueError("random masks are drawn from the step key, not on the host")
        frac = self.target_frac if frac is None else frac
        T = len(tokens)
        jitter = position_hash(T, self.seed)
        total = 0.1 * jitter
        if self.unigram is not None:
            ids = np.clip(tokens, 0, len(self.unigram) - 1)
            commonness = np.argsort(np.argsort(self.unigram[ids].astype(np.float64)))       # 0 = rarest token of the sequence
            total = total + (1.0 - commonness / max(T - 1, 1))
            if self.mode == "docaware":
                total = total + 1.0 * self.rare_third()[ids]
        if self.mode == "docaware":
            total = total + 3.0 * trigram_recurs(tokens, self.eos, prefix)
        if self.generic_floor > 0:
            total = total + 10.0 * (jitter < self.generic_floor * frac)
        return np.where((tokens == self.pad) | (tokens == self.eos), -np.inf, total)

    def targets(self, tokens: np.ndarray, prefix: Optional[np.ndarray] = None, frac: Optional[float] = None) -> np.ndarray:
        frac = self.target_frac if frac is None else frac
        return best_per_chunk(self.scores(tokens, prefix, frac), self.chunk, int(round(frac * self.chunk)))

    def split_order(self, tokens: np.ndarray, context_frac: float, prefix: Optional[np.ndarray] = None) -> np.ndarray:
        """``[T]`` int32 absolute positions: per chunk the ``K = round(context_frac * C)`` context slots in natural order, then
        the ``C - K`` targets in an order drawn from a generator seeded by (seed, the first tokens)."""
        T, C = len(tokens), self.chunk
        K = int(round(context_frac * C))
        if self.mode == "random":
            chosen = best_per_chunk(position_hash(T, self.seed), C, C - K)
        else:
            chosen = self.targets(tokens, prefix, 1.0 - K / C)
        head = np.asarray(tokens, np.int64)[:min(T, 64)]
        draw = np.random.default_rng([self.seed, int(np.bitwise_xor.reduce(head) & 0x7FFFFFFF)])
        order = np.empty(T, np.int32)
        slots = np.arange(C)
        for c, row in enumerate(chosen.reshape(-1, C)):
            tgt, ctx = slots[row], slots[~row]
            short = (C - K) - len(tgt)
            if short > 0:                                          # a chunk of pad / EOS: take the missing targets from the context's end
                tgt, ctx = np.concatenate([tgt, ctx[::-1][:short]]), ctx[:len(ctx) - short]
            order[c * C:(c + 1) * C] = c * C + np.concatenate([ctx, draw.permutation(tgt)])
        return order


def inner_mask_rule(tokens: np.ndarray, mode: str, chunk: int, eos: int, pad: int, unigram: Optional[np.ndarray] = None,
                    target_frac: float = 0.5, generic_floor: float = 0.1, seed: int = 0,
                    prefix: Optional[np.ndarray] = None) -> np.ndarray:
    """``[T]`` bool mask of the inner targets of one sequence (``T`` a multiple of ``chunk``)."""
    return TargetRule(mode, chunk, eos, pad, unigram, target_frac, generic_floor, seed).targets(np.asarray(tokens), prefix)


def split_perm(tokens: np.ndarray, mode: str, chunk: int, eos: int, pad: int, context_frac: float = 0.5,
               unigram: Optional[np.ndarray] = None, generic_floor: float = 0.1, seed: int = 0,
               prefix: Optional[np.ndarray] = None) -> np.ndarray:
    return TargetRule(mode, chunk, eos, pad, unigram, 0.5, generic_floor, seed).split_order(np.asarray(tokens), context_frac, prefix)


class MaskMaker:
    """Host-side inner masks (mask task) or orders (split task) for a batch ``[B, T]``; ``None`` when the masks are the
    random ones drawn from the step key (reference data.py:852-877)."""

    def __init__(self, mode: str, chunk: int, eos: int, pad: int, unigram_path: str = "", target_frac: float = 0.5,
                 generic_floor: float = 0.1, seed: int = 0, task: str = "mask"):
        self.mode, self.task, self.target_frac = mode, task, target_frac
        table = None
        if (mode != "random" or task == "split") and unigram_path and os.path.exists(unigram_path):
            table = np.fromfile(unigram_path, dtype=np.int64)
        self.unigram = table
        self.rule = TargetRule(mode, chunk, eos, pad, table, target_frac, generic_floor, seed)

    @property
    def active(self) -> bool:
        return self.task == "split" or self.mode != "random"

    def __call__(self, ids: np.ndarray) -> Optional[np.ndarray]:
        if self.task == "split":
            return np.stack([self.rule.split_order(row, 1.0 - self.target_frac) for row in ids])
        if self.mode == "random":
            return None
        return np.stack([self.rule.targets(row) for row in ids])
