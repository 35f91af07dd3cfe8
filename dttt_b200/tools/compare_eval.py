"""Reproduction check between two evaluations of the same weights (two ``eval_<step>.npz`` / ``eval_<step>_planted.npz``
files written on different machines or builds).

    python -m dttt_b200.tools.compare_eval A/eval_4000.npz B/eval_4000.npz

First whether both scored the same sequences (sources, document ids and lengths, tokens beyond the window), then for
every per-sequence array they share: both means, the mean difference, quantiles of ``|B - A|`` and the correlation;
for the losses also the mean difference per source.  Role of the reference's ``tools/compare_eval.py:1-48``.
"""
from __future__ import annotations

import sys

import numpy as np

from . import evalstats as S

IDENTITY = ("sources", "doc_ids", "doc_lens", "beyond")


def compare(a, b, out=print) -> bool:
    paired = True
    for k in IDENTITY:
        if k in a or k in b:
            same = k in a and k in b and a[k].shape == b[k].shape and bool(np.all(a[k] == b[k]))
            paired &= same
            out(f"  {k:10s} {'identical' if same else 'DIFFERENT'}")
    if not paired:
        out("  the files did not score the same sequences: what follows is not a paired comparison")
    out(f"  {'array':16s} {'mean A':>10s} {'mean B':>10s} {'B - A':>10s} {'|d| p50':>10s} {'p99':>10s} {'max':>10s} {'corr':>8s}")
    for k in sorted((set(a) & set(b)) - set(IDENTITY)):
        x, y = np.asarray(a[k], np.float64), np.asarray(b[k], np.float64)
        if x.ndim != 1 or x.shape != y.shape or not len(x):
            continue
        d = np.abs(y - x)
        corr = np.corrcoef(x, y)[0, 1] if x.std() > 0 and y.std() > 0 else float("nan")
        out(f"  {k:16s} {x.mean():10.5f} {y.mean():10.5f} {(y - x).mean():+10.5f} {np.median(d):10.5f} {np.quantile(d, 0.99):10.5f} "
            f"{d.max():10.5f} {corr:8.4f}")
    if paired and "sources" in a:
        src = a["sources"].astype(str)
        for k in ("loss_1.0", "loss_0.0"):
            if k in a and k in b:
                out(f"  {k} B - A by source: " + " | ".join(f"{s} {(b[k][src == s] - a[k][src == s]).mean():+.5f}" for s in dict.fromkeys(src)))
    return paired


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__)
        return 2
    compare(S.load_npz(argv[0]), S.load_npz(argv[1]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
