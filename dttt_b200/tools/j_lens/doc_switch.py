"""A document switch in front of a memory trained on single-document windows (the packing question): document A
(``--n_a`` chunks, its last token replaced by EOS) followed by document B (``--n_b`` chunks), both whole documents from the
held-out tails of their sources, B starting at a chunk boundary, positions running on.  Every chunk is read first (i.i.d.
masks at each ``--t``, the same masks for every variant), then written with the run's own write, against

    carry   the memory as written so far (A, then B): what a packed sequence gives the model
    reset   the memory reset to W_0 at the switch, the windows unchanged: carry - reset isolates A's content left in the memory
    off     W_0 with the carry state's windows: no memory

Per chunk offset after the switch: stale = carry - reset (A's leftover content; > 0 hurts), gain = off - reset (B's own
memory), net = off - carry.  Pairs: A from source i and B from source i + 1 (``cross``), and two documents of source i
(``same``).  The file holds ``ce [n_pairs, n_t, n_a + n_b, 3]`` (carry, reset, off), ``kind [n_pairs]``, ``ts``.

    python -m dttt_b200.tools.j_lens.doc_switch --ckpt <step dir> --sources a=dir:1.0,b=dir:1.0 --n_a 8 --n_b 8 --n_per_pair 3 --t 0.3,0.6,0.9

Role of the reference's ``tools/j_lens/doc_switch.py:1-213``.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

from . import _cli
from .core import Reader

VARIANTS = ("carry", "reset", "off")


def held_out_docs(src_dir: str, holdout: int, eos: int, need: int, count: int):
    """The first ``count`` whole documents of at least ``need`` tokens in a stream's held-out tail (its last ``holdout`` tokens,
    from the first EOS on), each cut to its first ``need`` tokens."""
    mm = np.memmap(os.path.join(src_dir, "tokens.u32"), dtype="<u4", mode="r")
    tail = np.asarray(mm[max(0, len(mm) - holdout):])
    ends = np.flatnonzero(tail == eos)
    docs = []
    for s, e in zip(ends[:-1] + 1, ends[1:]):
        if e - s >= need:
            docs.append(tail[s:s + need].astype(np.int64))
            if len(docs) == count:
                break
    return docs


def pairs_from(docs_by_source, n_per_pair: int):
    names = list(docs_by_source)
    out = []
    for i, n in enumerate(names):
        d = docs_by_source[n]
        for k in range(min(n_per_pair, len(d) // 2)):
            out.append(("same", d[2 * k][0], d[2 * k + 1][1]))
        nxt = docs_by_source[names[(i + 1) % len(names)]]
        if len(names) > 1:
            for k in range(min(n_per_pair, len(d), len(nxt))):
                out.append(("cross", d[k][0], nxt[k][1]))
    return out


def measure(reader: Reader, pairs, n_a: int, n_b: int, ts, eos: int, log=print) -> np.ndarray:
    C = reader.C
    nc = n_a + n_b
    ce = np.zeros((len(pairs), len(ts), nc, 3))
    g = torch.Generator().manual_seed(777)
    u = torch.rand(nc, C, generator=g)                                        # one uniform draw per slot: the masks are nested in t
    for p, (kind, A_, B_) in enumerate(pairs):
        a = A_.copy()
        a[-1] = eos
        seq = torch.as_tensor(np.concatenate([a, B_])[None], device=reader.dev)
        carry = reader.fresh(1)
        reset = None
        for c in range(nc):
            x = seq[:, c * C:(c + 1) * C]
            if c == n_a:
                reset = reader.reset_memory(carry)                             # W_0 at the switch, the windows as they are
            states = {"carry": carry, "reset": carry if reset is None else reader.with_memory(carry, reset.W), "off": reader.reset_memory(carry)}
            for ti, t in enumerate(ts):
                m = (u[c] < t)[None].to(reader.dev)
                for vi, v in enumerate(VARIANTS):
                    ce[p, ti, c, vi] = float(reader.mean_ce(reader.read(x, m, states[v]), x, m))
            nxt = reader.write(carry, x)
            if reset is not None:
                reset = reader.write(reader.with_memory(carry, reset.W), x)
            carry = nxt
        off_b = ce[p, :, n_a:].mean(0)
        log(f"[switch] pair {p + 1}/{len(pairs)} ({kind}): stale by offset " + " ".join(f"{v:+.3f}" for v in off_b[:, 0] - off_b[:, 1]))
    return ce


def summarise(ce: np.ndarray, kinds, n_a: int, log=print) -> None:
    for kind in dict.fromkeys(kinds):
        sel = np.array(kinds) == kind
        m = ce[sel].mean((0, 1))                                                # [chunks, 3]
        b = m[n_a:]
        log(f"[switch] {kind}: A's gain (off - carry) {np.mean(m[:n_a, 2] - m[:n_a, 0]):+.4f} | after the switch, by offset: stale "
            + " ".join(f"{v:+.3f}" for v in b[:, 0] - b[:, 1]) + " | gain " + " ".join(f"{v:+.3f}" for v in b[:, 2] - b[:, 1])
            + " | net " + " ".join(f"{v:+.3f}" for v in b[:, 2] - b[:, 0]))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.j_lens.doc_switch")
    _cli.add_common(ap)
    ap.add_argument("--n_a", type=int, default=8)
    ap.add_argument("--n_b", type=int, default=8)
    ap.add_argument("--n_per_pair", type=int, default=3)
    ap.add_argument("--t", default="0.3,0.6,0.9")
    ap.add_argument("--holdout", type=int, default=4_194_304)
    a = ap.parse_args(argv)
    a.seq_len = a.seq_len if a.synthetic else 0
    reader, ids, names = _cli.load(a)
    C, eos = reader.C, reader.mc.eos_token_id
    ts = [float(x) for x in a.t.split(",")]
    if a.synthetic:
        g = np.random.default_rng(a.seed)
        mk = lambda n: g.integers(3, a.synthetic, size=n * C).astype(np.int64)
        docs = {"synthetic": [(mk(a.n_a), mk(a.n_b)) for _ in range(2 * a.n_per_pair)]}
    else:
        from ...data.streams import parse_sources
        docs = {}
        for s in parse_sources(reader.cfg.sources, reader.cfg.data_root):
            ds = held_out_docs(s.path, a.holdout, eos, max(a.n_a, a.n_b) * C, 2 * a.n_per_pair)
            docs[s.name] = [(d[:a.n_a * C], d[:a.n_b * C]) for d in ds]
    pairs = pairs_from(docs, a.n_per_pair)
    if not pairs:
        raise SystemExit("no held-out document is long enough for the requested chunks")
    ce = measure(reader, pairs, a.n_a, a.n_b, ts, eos)
    kinds = [p[0] for p in pairs]
    summarise(ce, kinds, a.n_a)
    if a.out:
        np.savez_compressed(a.out, ce=ce, kind=np.array(kinds), ts=np.array(ts), variants=np.array(VARIANTS), n_a=a.n_a, n_b=a.n_b)
    return 0


if __name__ == "__main__":
    sys.exit(main())
