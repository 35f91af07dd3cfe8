"""Word n-gram overlap with a reference set of books: the measure used to keep evaluation books out of training data.

A text's signature is the set of 64-bit hashes of its word 13-grams (lower-cased runs of ``[a-z0-9]``, every
``stride``-th position); its overlap with the reference set is the share of those hashes found there.  The reference
set is held as one sorted ``uint64`` array and membership is a vectorised ``searchsorted``.  Definition of the measure:
reference ``tools/convert_dolma.py:44-64``.
"""
from __future__ import annotations

import hashlib
import re
from typing import Iterable, Optional

import numpy as np

WORD = re.compile(r"[a-z0-9]+")
N = 13


def gram_hashes(text: str, stride: int = 1, n: int = N) -> np.ndarray:
    words = WORD.findall(text.lower())
    if len(words) < n:
        return np.empty(0, np.uint64)
    out = np.empty((len(words) - n) // stride + 1, np.uint64)
    for j, i in enumerate(range(0, len(words) - n + 1, stride)):
        out[j] = int.from_bytes(hashlib.blake2b(" ".join(words[i:i + n]).encode(), digest_size=8).digest(), "little")
    return out


class BookSet:
    """The 13-grams (and, when known, the Project Gutenberg numbers) of a set of books."""

    def __init__(self, texts: Iterable[str], gutenberg_ids: Optional[Iterable[int]] = None, names: Optional[Iterable[str]] = None):
        per = [np.unique(gram_hashes(t)) for t in texts]
        self.names = list(names) if names is not None else [str(i) for i in range(len(per))]
        allh = np.concatenate(per) if per else np.empty(0, np.uint64)
        owner = np.concatenate([np.full(len(h), i, np.int32) for i, h in enumerate(per)]) if per else np.empty(0, np.int32)
        order = np.argsort(allh, kind="stable")
        self.hashes, self.owner = allh[order], owner[order]
        self.ids = set(int(i) for i in (gutenberg_ids or ()))

    @classmethod
    def from_parquet(cls, path: str) -> "BookSet":
        import pyarrow.parquet as pq
        cols = pq.ParquetFile(path).schema_arrow.names
        t = pq.read_table(path, columns=[c for c in ("url", "text", "title") if c in cols])
        urls = t.column("url").to_pylist() if "url" in cols else []
        ids = [int(u.rstrip("/").split("/")[-1]) for u in urls if u and u.rstrip("/").split("/")[-1].isdigit()]
        names = t.column("title").to_pylist() if "title" in cols else (urls or None)
        return cls(t.column("text").to_pylist(), ids, names)

    def _find(self, h: np.ndarray):
        if not len(self.hashes) or not len(h):
            return np.zeros(len(h), bool), np.zeros(len(h), np.int64)
        pos = np.searchsorted(self.hashes, h)
        pos = np.minimum(pos, len(self.hashes) - 1)
        return self.hashes[pos] == h, pos

    def overlap(self, text: str, stride: int = 1) -> float:
        h = gram_hashes(text, stride)
        if not len(h):
            return 0.0
        hit, _ = self._find(h)
        return float(hit.mean())

    def best_book(self, text: str, stride: int = 1):
        """``(overlap, name of the book most of the hits come from)``."""
        h = gram_hashes(text, stride)
        if not len(h):
            return 0.0, None
        hit, pos = self._find(h)
        if not hit.any():
            return 0.0, None
        owners = self.owner[pos[hit]]
        return float(hit.mean()), self.names[int(np.bincount(owners).argmax())]


def gutenberg_number(record: dict) -> Optional[int]:
    m = re.search(r"gutenberg\.org/ebooks/(\d+)", str((record.get("metadata") or {}).get("url", "")))
    return int(m.group(1)) if m else None
