"""Token streams on disk and the stateless multi-source sampler.

A source is a directory with ``tokens.u32`` (flat little-endian uint32, documents separated by one EOS, no BOS), ``meta.json``
(``num_tokens``, ``num_docs``, tokenizer fingerprint, ...) and optionally ``windows_<T>_<holdout>.npy``: the on-disk form of the
reference (src/ttt/data.py:5-24), so prepared data is interchangeable.

What is read at a training step is a pure function of ``(seed, step)``; nothing is carried between steps, which makes restarts
exact.  The mapping is the reference's (data.py:620-770), so both code bases read the same sequences in the same order and their
checkpoints pass each other's data check:

* the mixture: global sample ``g`` takes its source from ``default_rng([seed, 1, g // 65536]).choice(sources, 65536, p=weights)``;
* the sample's rank inside its source = how many earlier samples chose that source; rank ``r`` of a source with ``n`` sequences
  reads entry ``r % n`` of the epoch permutation ``default_rng([seed, 2, source, r // n]).permutation(n)``;
* plants: ``default_rng([seed, 3, g])`` decides and draws;
* the stream's identity: a path-free hash of (name, weight, size) per source, seed, sequence length, sequences per optimiser
  step, hold-out, plant and window settings.

Three classes share the work: ``MixtureIndex`` (sample number -> source and sequence, resolved for a whole batch at once with
numpy), ``HeldOut`` (the evaluation tail of every source: starts after an EOS, read in order) and ``Sampler`` (the rows).
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

BLOCK = 1 << 16                      # samples per block of the mixture stream
DEFAULT_EOS = 128001


# ------------------------------------------------------------------------------------------------------------ sources
@dataclass(frozen=True)
class Source:
    name: str
    path: str
    weight: float
    num_tokens: int
    vocab_len: int = 0
    eos_token_id: int = DEFAULT_EOS

    def open(self) -> np.memmap:
        return np.memmap(os.path.join(self.path, "tokens.u32"), dtype="<u4", mode="r")


def split_sources(spec: str, root: str = "") -> List[Tuple[str, str, float]]:
    """``"a=dir:0.7,b=dir"`` -> ``[(name, directory, weight)]`` (weight 1 when absent; relative directories under ``root``)."""
    triples = []
    for entry in filter(None, (part.strip() for part in spec.split(","))):
        name, _, where = entry.partition("=")
        if not _:
            raise ValueError(f"source {entry!r}: expected name=directory[:weight]")
        directory, sep, weight = where.rpartition(":")
        if not sep:
            directory, weight = where, "1.0"
        triples.append((name, os.path.join(root, directory) if root else directory, float(weight)))
    return triples


def _read_meta(directory: str) -> dict:
    with open(os.path.join(directory, "meta.json")) as fh:
        return json.load(fh)


def parse_sources(spec: str, root: str = "") -> List[Source]:
    """The sources of ``spec`` with their sizes read from ``meta.json`` and their weights normalised to sum 1."""
    found = []
    for name, directory, weight in split_sources(spec, root):
        meta = _read_meta(directory)
        tokenizer = meta.get("tokenizer")
        tokenizer = tokenizer if isinstance(tokenizer, dict) else {}
        eos = tokenizer.get("eos_token_id", meta.get("eos_token_id"))
        found.append(Source(name, directory, weight, int(meta["num_tokens"]), int(tokenizer.get("len", 0)),
                            DEFAULT_EOS if eos is None else int(eos)))
    if not found:
        raise ValueError("no sources")
    total = sum(s.weight for s in found)
    return [Source(s.name, s.path, s.weight / total, s.num_tokens, s.vocab_len, s.eos_token_id) for s in found]


def check_vocab(sources: Sequence[Source], vocab_size: int) -> None:
    for s in sources:
        if s.vocab_len and s.vocab_len > vocab_size:
            raise ValueError(f"source {s.name}: tokenizer length {s.vocab_len} exceeds model vocab_size {vocab_size}")


def sources_hash(sources: Sequence[Source], seed: int, seq_len: int, step_batch: int, holdout_tokens: int = 0,
                 extra: Optional[list] = None, paths: Optional[Sequence[str]] = None) -> str:
    """Identity of a training stream (16 hex digits).  Without ``paths`` the path-free form (``data_hash_version`` 2); with the
    stream directories given, the older form that includes their absolute paths (version 1)."""
    if paths is None:
        per_source = [(s.name, round(s.weight, 9), s.num_tokens) for s in sources]
    else:
        per_source = [(s.name, os.path.abspath(p), round(s.weight, 9), s.num_tokens) for s, p in zip(sources, paths)]
    record = per_source + [seed, seq_len, step_batch, holdout_tokens] + list(extra or [])
    return hashlib.sha256(json.dumps(record, sort_keys=True).encode()).hexdigest()[:16]


# ------------------------------------------------------------------------------------------------------------ plants
@dataclass(frozen=True)
class Plant:
    """Planted recall in training: a fraction ``frac`` of the sequences gets one span (``len_min .. len_max`` tokens) copied from
    an early chunk to a chunk more than ``window`` chunks later (reference data.py:585-617)."""
    frac: float
    len_min: int
    len_max: int
    chunk: int
    window: int


def plant_copy(row: np.ndarray, rng: np.random.Generator, len_min: int, len_max: int, chunk: int, window: int,
               eos: Optional[int] = None, tries: int = 8) -> Optional[Tuple[int, int, int]]:
    """Copy one span inside ``row`` in place; returns ``(source offset, target offset, length)`` or ``None`` when the row is too
    short or every draw touched a document boundary.  The generator is consumed in a fixed order per try: length, source chunk,
    target chunk, offset in the source chunk, offset in the target chunk."""
    n_chunks = len(row) // chunk
    if n_chunks < window + 2:
        return None

    def touches_boundary(start: int, length: int) -> bool:
        return eos is not None and bool(np.any(row[start:start + length] == eos))

    for _ in range(tries):
        span = int(rng.integers(len_min, len_max + 1))
        src_chunk = int(rng.integers(0, n_chunks - window - 1))
        dst_chunk = int(rng.integers(src_chunk + window + 1, n_chunks))
        src = src_chunk * chunk + int(rng.integers(0, chunk - span + 1))
        dst = dst_chunk * chunk + int(rng.integers(0, chunk - span + 1))
        if touches_boundary(src, span) or touches_boundary(dst, span):
            continue
        row[dst:dst + span] = row[src:src + span]
        return src, dst, span
    return None


# ------------------------------------------------------------------------------------------------------------ the mixture
class MixtureIndex:
    """Global sample number -> ``(source, sequence index)``, with small caches of the block choices, the per-source counts before
    each block and the epoch permutations."""

    def __init__(self, weights: np.ndarray, n_seq: np.ndarray, seed: int, keep_permutations: int = 8):
        self.weights, self.n_seq, self.seed = weights, n_seq, seed
        self.n_sources = len(weights)
        self._keep = keep_permutations
        self._choices: Dict[int, np.ndarray] = {}
        self._counts_at: Dict[int, np.ndarray] = {0: np.zeros(self.n_sources, np.int64)}
        self._perms: Dict[Tuple[int, int], np.ndarray] = {}

    def choices(self, block: int) -> np.ndarray:
        """The source of each of the ``BLOCK`` samples of ``block``."""
        got = self._choices.get(block)
        if got is None:
            draw = np.random.default_rng([self.seed, 1, block]).choice(self.n_sources, size=BLOCK, p=self.weights)
            got = self._choices[block] = draw.astype(np.int32)
        return got

    def counts_before(self, block: int) -> np.ndarray:
        """Per source, how many samples of blocks ``0 .. block - 1`` chose it."""
        known = max(b for b in self._counts_at if b <= block)
        for b in range(known, block):
            self._counts_at[b + 1] = self._counts_at[b] + np.bincount(self.choices(b), minlength=self.n_sources)
        return self._counts_at[block]

    def permutation(self, source: int, epoch: int) -> np.ndarray:
        key = (source, epoch)
        perm = self._perms.get(key)
        if perm is None:
            perm = self._perms[key] = np.random.default_rng([self.seed, 2, source, epoch]).permutation(self.n_seq[source])
            while len(self._perms) > self._keep:
                del self._perms[next(iter(self._perms))]
        return perm

    def locate(self, first: int, count: int) -> List[Tuple[int, int]]:
        """``(source, sequence index)`` of samples ``first .. first + count - 1``."""
        found: List[Tuple[int, int]] = []
        g, end = first, first + count
        while g < end:
            block, at = divmod(g, BLOCK)
            n = min(end - g, BLOCK - at)
            picked = self.choices(block)
            here = picked[at:at + n].astype(np.int64)
            # rank inside the source = samples of that source in earlier blocks + earlier in this block
            earlier_in_block = np.bincount(picked[:at], minlength=self.n_sources)
            running = np.zeros(self.n_sources, np.int64)
            base = self.counts_before(block) + earlier_in_block
            for s in here:
                rank = int(base[s] + running[s])
                running[s] += 1
                epoch, slot = divmod(rank, int(self.n_seq[s]))
                found.append((int(s), int(self.permutation(int(s), epoch)[slot])))
            g += n
        return found


# ------------------------------------------------------------------------------------------------------------ held-out tails
class HeldOut:
    """The evaluation region of every source: the last ``holdout`` tokens, moved forward to start right after an EOS, read as
    consecutive sequences (never sampled for training)."""

    SEARCH = 1 << 20

    def __init__(self, sources: Sequence[Source], maps: Sequence[np.ndarray], seq_len: int, holdout: int, whole: bool,
                 fallback_eos: Optional[int]):
        self.start = np.zeros(len(sources), np.int64)
        self.n_seq = np.zeros(len(sources), np.int64)
        for i, (s, mm) in enumerate(zip(sources, maps)):
            if whole:
                cut = 0
            elif holdout > 0:
                cut = max(0, s.num_tokens - holdout)
            else:
                cut = s.num_tokens
            begin = cut
            if cut < s.num_tokens:
                eos = s.eos_token_id or (DEFAULT_EOS if fallback_eos is None else fallback_eos)
                begin = self._after_next_eos(mm, cut, eos)
            self.start[i] = begin
            self.n_seq[i] = max(0, (s.num_tokens - begin) // seq_len)

    @classmethod
    def _after_next_eos(cls, mm: np.ndarray, at: int, eos: int) -> int:
        """The offset after the first EOS at or after ``at`` (a bounded look first, then the rest); ``at`` when there is none."""
        for stop in (at + cls.SEARCH, None):
            hits = np.flatnonzero(np.asarray(mm[at:stop]) == eos)
            if hits.size:
                return at + int(hits[0]) + 1
        return at


# ------------------------------------------------------------------------------------------------------------ the sampler
class Sampler:
    """Rows of the training stream (``batch``, ``global_batch``) and of the held-out tails (``eval_*``) for one data rank."""

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
        self._mm = [s.open() for s in self.sources]
        n_sources = len(self.sources)
        self.windows = None if windows is None else [np.asarray(w, np.int64) for w in windows]
        if eval_only:
            self.n_seq = np.zeros(n_sources, np.int64)
        elif self.windows is not None:
            if len(self.windows) != n_sources:
                raise ValueError("windows: one array per source")
            self.n_seq = np.array([len(w) for w in self.windows], np.int64)
        else:
            sizes = np.array([s.num_tokens for s in self.sources], np.int64)
            self.n_seq = np.maximum(0, sizes - max(holdout_tokens, 0)) // seq_len
        if not eval_only and np.any(self.n_seq <= 0):
            raise ValueError("a source is shorter than one training sequence after the holdout")
        self.w = np.array([s.weight for s in self.sources], np.float64)
        self._index = MixtureIndex(self.w, self.n_seq, seed)
        self.plant = plant if (plant is not None and plant.frac > 0) else None
        self._extra = self._identity_extras()
        self.hash = self.hash_at(self.step_batch)
        tail = HeldOut(self.sources, self._mm, seq_len, holdout_tokens, eval_only, eos)
        self.eval_start, self.n_eval_seq = tail.start, tail.n_seq

    def _identity_extras(self) -> Optional[list]:
        parts: list = []
        if self.plant is not None:
            p = self.plant
            parts += ["plant", p.frac, p.len_min, p.len_max, p.chunk, p.window]
        if self.windows is not None:
            parts += ["windows"] + [hashlib.sha256(w.tobytes()).hexdigest()[:16] for w in self.windows]
        return parts or None

    # ---- identity
    def hash_at(self, step_batch: int) -> str:
        """The stream's identity if an optimiser step took ``step_batch`` sequences."""
        return sources_hash(self.sources, self.seed, self.T, step_batch, self.holdout_tokens, extra=self._extra)

    def legacy_hash(self, paths: Sequence[str], global_batch: int) -> str:
        return sources_hash(self.sources, self.seed, self.T, global_batch, self.holdout_tokens, extra=self._extra, paths=paths)

    # ---- training rows
    def locate_many(self, g0: int, n: int) -> List[Tuple[int, int]]:
        return self._index.locate(g0, n)

    def locate(self, g: int) -> Tuple[int, int]:
        return self._index.locate(g, 1)[0]

    def _read(self, first: int, count: int, out: Optional[np.ndarray]) -> np.ndarray:
        rows = np.empty((count, self.T), np.int32) if out is None else out
        for j, (s, i) in enumerate(self._index.locate(first, count)):
            at = i * self.T if self.windows is None else int(self.windows[s][i])
            rows[j] = self._mm[s][at:at + self.T]
            if self.plant is not None:
                gen = np.random.default_rng([self.seed, 3, first + j])
                if gen.random() < self.plant.frac:
                    p = self.plant
                    plant_copy(rows[j], gen, p.len_min, p.len_max, p.chunk, p.window, self.eos)
        return rows

    def batch(self, step: int, out: Optional[np.ndarray] = None) -> np.ndarray:
        """This rank's ``[local, T]`` int32 rows of global batch ``step`` (written into ``out`` when given, e.g. pinned memory)."""
        return self._read(step * self.G + self.rank * self.local, self.local, out)

    def global_batch(self, step: int) -> np.ndarray:
        return self._read(step * self.G, self.G, None)

    # ---- held-out rows
    def eval_batches(self, source: int) -> int:
        return int(self.n_eval_seq[source] // self.G)

    def eval_step_batches(self, source: int) -> int:
        return int(self.n_eval_seq[source] // self.step_batch)

    def _eval_origin(self, source: int, k: int) -> int:
        """Offset of the first sequence of held-out batch ``k`` (all ranks)."""
        return int(self.eval_start[source]) + k * self.G * self.T

    def eval_batch(self, source: int, k: int) -> np.ndarray:
        """This rank's rows of held-out batch ``k`` of ``source``."""
        if not 0 <= k < self.eval_batches(source):
            raise IndexError(f"eval batch {k} of source {source}: only {self.eval_batches(source)}")
        first = self._eval_origin(source, k) + self.rank * self.local * self.T
        block = np.asarray(self._mm[source][first:first + self.local * self.T])
        return block.reshape(self.local, self.T).astype(np.int32)

    def eval_doc_info(self, source: int, k: int, eos: int, window_tokens: int):
        """For each of the ``G`` sequences of held-out batch ``k``: the length of the document its first token belongs to, how many
        of the sequence's tokens of that document lie beyond the attention window, and the document's start offset.  Documents are
        delimited inside a neighbourhood of 64 sequences around the optimiser-step batch that contains ``k``."""
        T, mm = self.T, self._mm[source]
        seq_at = self._eval_origin(source, k) + np.arange(self.G) * T
        step_at = int(self.eval_start[source]) + (k * self.G // self.step_batch) * self.step_batch * T
        lo, hi = max(0, step_at - 64 * T), min(len(mm), step_at + (self.step_batch + 64) * T)
        boundaries = lo + np.flatnonzero(np.asarray(mm[lo:hi]) == eos)
        if boundaries.size == 0:
            doc_start, doc_end = np.full(self.G, lo), np.full(self.G, hi)
        else:
            nxt = np.searchsorted(boundaries, seq_at)                              # first boundary at or after the sequence start
            doc_start = np.where(nxt > 0, boundaries[np.maximum(nxt - 1, 0)] + 1, lo)
            doc_end = np.where(nxt < boundaries.size, boundaries[np.minimum(nxt, boundaries.size - 1)], hi)
        doc_len = (doc_end - doc_start + 1).astype(np.int64)
        beyond = np.clip(np.minimum(doc_end, seq_at + T) - (seq_at + window_tokens), 0, None).astype(np.int64)
        return doc_len, beyond, doc_start.astype(np.int64)

    def eval_context(self, source: int, k: int, eos: int, lookback: int):
        """Per sequence of held-out batch ``k``: ``(tokens from up to lookback before the sequence to its end, where the sequence
        starts inside them, offsets at which documents begin)`` -- what the recurrence probe needs."""
        T, mm = self.T, self._mm[source]
        rows = []
        for j in range(self.G):
            at = self._eval_origin(source, k) + j * T
            lo = max(0, at - lookback)
            tokens = np.asarray(mm[lo:at + T])
            begins = np.concatenate([[0], np.flatnonzero(tokens == eos) + 1])
            rows.append((tokens, at - lo, begins[begins < len(tokens)]))
        return rows
