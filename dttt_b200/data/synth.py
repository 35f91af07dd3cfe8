"""Synthetic token streams: Zipf-distributed tokens with EOS at geometric document boundaries.

``zipf_tokens`` draws ids from ``p(rank) ~ rank^-s`` over the vocabulary (special ids excluded) and
inserts ``eos`` after documents whose lengths are geometric with the given mean.  ``write_stream``
writes them in the on-disk stream format of the reference (``src/ttt/data.py:5-24``): a directory with
``tokens.u32`` (little-endian uint32, one EOS per document, no BOS) and ``meta.json``, so either
implementation can train on the same synthetic data.
"""
from __future__ import annotations

import json
import os
from typing import Iterable, Optional

import numpy as np


def zipf_tokens(n: int, vocab: int, seed: int, s: float = 1.1, eos: Optional[int] = None, mean_doc: int = 2048,
                exclude: Iterable[int] = ()) -> np.ndarray:
    """``[n]`` uint32 token ids."""
    rng = np.random.default_rng([seed, 0x5A1F])
    banned = set(int(x) for x in exclude)
    if eos is not None:
        banned.add(int(eos))
    usable = np.array([i for i in range(vocab) if i not in banned], dtype=np.int64) if len(banned) < 64 else \
        np.setdiff1d(np.arange(vocab), np.fromiter(banned, dtype=np.int64))
    ranks = np.arange(1, len(usable) + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    # a fixed permutation so that frequent ids are spread over the vocabulary
    perm = np.random.default_rng([seed, 0xBEEF]).permutation(len(usable))
    idx = np.searchsorted(cdf, rng.random(n), side="left").clip(0, len(usable) - 1)
    toks = usable[perm[idx]].astype(np.uint32)
    if eos is not None and mean_doc > 0:
        pos, p = 0, 1.0 / mean_doc
        while True:
            pos += int(rng.geometric(p))
            if pos >= n:
                break
            toks[pos] = eos
    return toks


def write_stream(path: str, tokens: np.ndarray, eos: int, name: str = "synthetic", vocab: int = 0) -> str:
    os.makedirs(path, exist_ok=True)
    tokens.astype("<u4").tofile(os.path.join(path, "tokens.u32"))
    vocab = int(vocab or int(tokens.max()) + 1)
    meta = {"name": name, "files": [], "min_doc_tokens": 0, "bos": False, "sep": "eos", "clean": "",
            "tokenizer": {"class": "synthetic-zipf", "len": vocab, "vocab_size": vocab, "eos_token_id": int(eos),
                          "bos_token_id": None},
            "num_docs": int((tokens == eos).sum()), "dropped_docs": 0, "num_tokens": int(tokens.size)}
    with open(os.path.join(path, "meta.json"), "w") as fh:
        json.dump(meta, fh, indent=2)
    return path
