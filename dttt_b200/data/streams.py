"""Token streams on disk and the stateless multi-source sampler.

On-disk form (shared with the reference, ``src/ttt/data.py:5-24``): one directory per source holding
``tokens.u32`` (flat little-endian uint32, documents separated by one EOS, no BOS), ``meta.json``
(``num_tokens``, ``num_docs``, tokenizer fingerprint, ...) and optional ``windows_<T>_<holdout>.npy``.

``Sampler.batch(step)`` is a pure function of ``(seed, step)`` (``data.py:620-770``): global sample
``g = step * G + j``; its source is drawn per block of 65 536 samples from
``default_rng([seed, 1, block])``; its rank within the source is the count of earlier samples of that
source; source epoch ``e`` reads the permutation ``default_rng([seed, 2, source, e])``.  The generators,
seeds and the path-free data hash are the reference's, so both implementations read the same sequences
in the same order and accept each other's checkpoints' data check.  What differs is the execution: the
choices and ranks of a whole batch are resolved with vectorised numpy instead of one ``locate`` call per
sample, and the rows are gathered into a caller-provided (pinned) buffer.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

BLOCK = 1 << 16


@dataclass(frozen=True)
class Source:
    name: str
    path: str
    weight: float
    num_tokens: int
    vocab_len: int = 0
    eos_token_id: int = 128001

    def open(self) -> np.memmap:
        return np.memmap(os.path.join(self.path, "tokens.u32"), dtype="<u4", mode="r")


def split_sources(spec: str, root: str = "") -> List[Tuple[str, str, float]]:
    """``"a=dir:0.7,b=dir:0.3"`` -> ``[(name, dir, weight)]``; relative dirs are taken under ``root``."""
    out = []
    for item in (s.strip() for s in spec.split(",")):
        if not item:
            continue
        name, rest = item.split("=", 1)
        path, w = rest.rsplit(":", 1) if ":" in rest else (rest, "1.0")
        out.append((name, os.path.join(root, path) if root else path, float(w)))
    return out


def parse_sources(spec: str, root: str = "") -> List[Source]:
    rows = []
    for name, path, w in split_sources(spec, root):
        with open(os.path.join(path, "meta.json")) as fh:
            meta = json.load(fh)
        tok = meta.get("tokenizer", {})
        tok = tok if isinstance(tok, dict) else {}
        eos = tok.get("eos_token_id", meta.get("eos_token_id"))
        rows.append(Source(name, path, w, int(meta["num_tokens"]), int(tok.get("len", 0)), int(eos) if eos is not None else 128001))
    if not rows:
        raise ValueError("no sources")
    z = sum(s.weight for s in rows)
    return [Source(s.name, s.path, s.weight / z, s.num_tokens, s.vocab_len, s.eos_token_id) for s in rows]


def check_vocab(sources: Sequence[Source], vocab_size: int) -> None:
    for s in sources:
        if s.vocab_len and s.vocab_len > vocab_size:
            raise ValueError(f"source {s.name}: tokenizer length {s.vocab_len} exceeds model vocab_size {vocab_size}")


def sources_hash(sources: Sequence[Source], seed: int, seq_len: int, step_batch: int, holdout_tokens: int = 0,
                 extra: Optional[list] = None, paths: Optional[Sequence[str]] = None) -> str:
    """Identity of a training stream, path-free (``data_hash_version`` 2); with ``paths`` the version-1 form."""
    if paths is None:
        rows = [(s.name, round(s.weight, 9), s.num_tokens) for s in sources]
    else:
        rows = [(s.name, os.path.abspath(p), round(s.weight, 9), s.num_tokens) for s, p in zip(sources, paths)]
    payload = rows + [seed, seq_len, step_batch, holdout_tokens] + (list(extra) if extra else [])
    return hashlib.sha256(json.dumps(payload, sort_keys=True).encode()).hexdigest()[:16]


@dataclass(frozen=True)
class Plant:
    """Planted recall: a fraction of the training sequences gets one span copied from an early chunk to a
    chunk beyond the attention window of the copy (reference data.py:585-617)."""
    frac: float
    len_min: int
    len_max: int
    chunk: int
    window: int


def plant_copy(row: np.ndarray, rng: np.random.Generator, len_min: int, len_max: int, chunk: int, window: int,
               eos: Optional[int] = None, tries: int = 8) -> Optional[Tuple[int, int, int]]:
    nc = len(row) // chunk
    if nc < window + 2:
        return None
    for _ in range(tries):
        L = int(rng.integers(len_min, len_max + 1))
        cs = int(rng.integers(0, nc - window - 1))
        ct = int(rng.integers(cs + window + 1, nc))
        a = cs * chunk + int(rng.integers(0, chunk - L + 1))
        b = ct * chunk + int(rng.integers(0, chunk - L + 1))
        if eos is not None and ((row[a:a + L] == eos).any() or (row[b:b + L] == eos).any()):
            continue
        row[b:b + L] = row[a:a + L]
        return a, b, L
    return None


class Sampler:
    def __init__(self, sources: Sequence[Source], seq_len: int, global_batch: int, seed: int, rank: int = 0, world: int = 1,
                 holdout_tokens: int = 0, eos: Optional[int] = None, eval_only: bool = False, plant: Optional[Plant] = None,
                 windows: Optional[Sequence[np.ndarray]] = None, accum: int = 1):
        if global_batch % world:
            raise ValueError(f"global_batch {global_batch} not divisible by {world} hosts")
        self.sources = list(sources)
        self.T, self.G, self.seed = seq_len, global_batch, seed
        self.rank, self.world, self.local = rank, world, global_batch // world
        self.accum, self.step_batch = accum, global_batch * accum
        self.holdout_tokens = self.holdout = holdout_tokens
        self.eval_only, self.eos = eval_only, eos
        S = len(self.sources)
        self.w = np.array([s.weight for s in self.sources], np.float64)
        tokens = np.array([s.num_tokens for s in self.sources], np.int64)
        if eval_only:
            self.n_seq = np.zeros(S, np.int64)
        else:
            self.n_seq = np.maximum(0, tokens - max(holdout_tokens, 0)) // seq_len
        self.windows = None if windows is None else [np.asarray(w, np.int64) for w in windows]
        if self.windows is not None and not eval_only:
            if len(self.windows) != S:
                raise ValueError("windows: one array per source")
            self.n_seq = np.array([len(w) for w in self.windows], np.int64)
        if not eval_only and (self.n_seq <= 0).any():
            raise ValueError("a source is shorter than one training sequence after the holdout")
        self._mm = [s.open() for s in self.sources]
        self._choice: Dict[int, np.ndarray] = {}
        self._before: Dict[int, np.ndarray] = {0: np.zeros(S, np.int64)}
        self._perm: Dict[Tuple[int, int], np.ndarray] = {}
        self.plant = plant if plant is not None and plant.frac > 0 else None
        extra: list = []
        if self.plant is not None:
            p = self.plant
            extra += ["plant", p.frac, p.len_min, p.len_max, p.chunk, p.window]
        if self.windows is not None:
            extra += ["windows"] + [hashlib.sha256(w.tobytes()).hexdigest()[:16] for w in self.windows]
        self._extra = extra or None
        self.hash = sources_hash(self.sources, seed, seq_len, self.step_batch, holdout_tokens, extra=self._extra)
        # held-out tail: starts at the first EOS at or after num_tokens - holdout
        self.eval_start = np.zeros(S, np.int64)
        self.n_eval_seq = np.zeros(S, np.int64)
        for i, s in enumerate(self.sources):
            raw = 0 if eval_only else (max(0, s.num_tokens - holdout_tokens) if holdout_tokens > 0 else s.num_tokens)
            start = raw
            if raw < s.num_tokens:
                e = s.eos_token_id if s.eos_token_id else (eos if eos is not None else 128001)
                start = self._first_eos_after(self._mm[i], raw, e)
            self.eval_start[i] = start
            self.n_eval_seq[i] = max(0, (s.num_tokens - start) // seq_len)

    @staticmethod
    def _first_eos_after(mm: np.ndarray, raw: int, eos: int) -> int:
        for span in (1_048_576, None):
            sub = np.asarray(mm[raw:raw + span] if span else mm[raw:])
            hit = np.flatnonzero(sub == eos)
            if len(hit):
                return raw + int(hit[0]) + 1
        return raw

    # ---- counter-based streams
    def _choices(self, blk: int) -> np.ndarray:
        c = self._choice.get(blk)
        if c is None:
            gen = np.random.default_rng([self.seed, 1, blk])
            c = self._choice[blk] = gen.choice(len(self.sources), size=BLOCK, p=self.w).astype(np.int32)
        return c

    def _counts_before(self, blk: int) -> np.ndarray:
        have = max(b for b in self._before if b <= blk)
        for b in range(have, blk):
            self._before[b + 1] = self._before[b] + np.bincount(self._choices(b), minlength=len(self.sources))
        return self._before[blk]

    def _permutation(self, s: int, epoch: int) -> np.ndarray:
        key = (s, epoch)
        p = self._perm.get(key)
        if p is None:
            p = self._perm[key] = np.random.default_rng([self.seed, 2, s, epoch]).permutation(self.n_seq[s])
            if len(self._perm) > 8:
                self._perm.pop(next(iter(self._perm)))
        return p

    def locate_many(self, g0: int, n: int) -> List[Tuple[int, int]]:
        """``(source, sequence index)`` of global samples ``g0 .. g0+n-1``."""
        out: List[Tuple[int, int]] = []
        g = g0
        while g < g0 + n:
            blk, off = divmod(g, BLOCK)
            take = min(g0 + n - g, BLOCK - off)
            ch = self._choices(blk)
            before = self._counts_before(blk)
            onehot = (ch[:off + take, None] == np.arange(len(self.sources))[None, :])
            csum = np.cumsum(onehot, axis=0)
            for j in range(off, off + take):
                s = int(ch[j])
                rank = int(before[s] + csum[j, s] - 1)
                epoch, r = divmod(rank, int(self.n_seq[s]))
                out.append((s, int(self._permutation(s, epoch)[r])))
            g += take
        return out

    def locate(self, g: int) -> Tuple[int, int]:
        return self.locate_many(g, 1)[0]

    def _offset(self, s: int, i: int) -> int:
        return i * self.T if self.windows is None else int(self.windows[s][i])

    def _plant(self, row: np.ndarray, g: int) -> None:
        p = self.plant
        if p is not None:
            gen = np.random.default_rng([self.seed, 3, g])
            if gen.random() < p.frac:
                plant_copy(row, gen, p.len_min, p.len_max, p.chunk, p.window, self.eos)

    def _rows(self, g0: int, n: int, out: Optional[np.ndarray]) -> np.ndarray:
        if out is None:
            out = np.empty((n, self.T), np.int32)
        for j, (s, i) in enumerate(self.locate_many(g0, n)):
            off = self._offset(s, i)
            out[j] = self._mm[s][off:off + self.T]
            self._plant(out[j], g0 + j)
        return out

    def batch(self, step: int, out: Optional[np.ndarray] = None) -> np.ndarray:
        """This rank's ``[local, T]`` int32 rows of global batch ``step`` (optionally into ``out``)."""
        return self._rows(step * self.G + self.rank * self.local, self.local, out)

    def global_batch(self, step: int) -> np.ndarray:
        return self._rows(step * self.G, self.G, None)

    def hash_at(self, step_batch: int) -> str:
        return sources_hash(self.sources, self.seed, self.T, step_batch, self.holdout_tokens, extra=self._extra)

    def legacy_hash(self, paths: Sequence[str], global_batch: int) -> str:
        return sources_hash(self.sources, self.seed, self.T, global_batch, self.holdout_tokens, extra=self._extra, paths=paths)

    # ---- held-out evaluation
    def eval_batches(self, source: int) -> int:
        return int(self.n_eval_seq[source] // self.G)

    def eval_step_batches(self, source: int) -> int:
        return int(self.n_eval_seq[source] // self.step_batch)

    def eval_batch(self, source: int, k: int) -> np.ndarray:
        if not 0 <= k < self.eval_batches(source):
            raise IndexError(f"eval batch {k} of source {source}: only {self.eval_batches(source)}")
        base = int(self.eval_start[source]) + (k * self.G + self.rank * self.local) * self.T
        mm = self._mm[source]
        return np.stack([np.asarray(mm[base + j * self.T: base + (j + 1) * self.T]) for j in range(self.local)]).astype(np.int32)

    def eval_doc_info(self, source: int, k: int, eos: int, window_tokens: int):
        """Per sequence of held-out batch ``k`` (all ``G``): the length of the document it starts in, how many of
        its tokens belong to that document beyond the attention window, and the document's start offset."""
        T = self.T
        base = int(self.eval_start[source]) + k * self.G * T
        mm = self._mm[source]
        step0 = int(self.eval_start[source]) + (k * self.G // self.step_batch) * self.step_batch * T
        lo = max(0, step0 - 64 * T)
        hi = min(len(mm), step0 + self.step_batch * T + 64 * T)
        eos_pos = np.flatnonzero(np.asarray(mm[lo:hi]) == eos) + lo
        starts_of = base + np.arange(self.G) * T
        i = np.searchsorted(eos_pos, starts_of)
        start = np.where(i > 0, eos_pos[np.maximum(i - 1, 0)] + 1, lo) if len(eos_pos) else np.full(self.G, lo)
        end = np.where(i < len(eos_pos), eos_pos[np.minimum(i, max(len(eos_pos) - 1, 0))], hi) if len(eos_pos) else np.full(self.G, hi)
        doc_len = (end - start + 1).astype(np.int64)
        beyond = np.maximum(0, np.minimum(end, starts_of + T) - (starts_of + window_tokens)).astype(np.int64)
        return doc_len, beyond, start.astype(np.int64)

    def eval_context(self, source: int, k: int, eos: int, lookback: int):
        T = self.T
        base = int(self.eval_start[source]) + k * self.G * T
        mm = self._mm[source]
        out = []
        for j in range(self.G):
            o = base + j * T
            lo = max(0, o - lookback)
            ctx = np.asarray(mm[lo:o + T])
            starts = np.concatenate([[0], np.flatnonzero(ctx == eos) + 1])
            out.append((ctx, o - lo, starts[starts < len(ctx)]))
        return out
