"""Did two builds (or two machines) evaluate the same weights to the same numbers?

    python -m dttt_b200.tools.compare_eval A/eval_4000.npz B/eval_4000.npz

Works on the ``eval_<step>.npz`` / ``eval_<step>_planted.npz`` files a run writes.  Step one decides whether the two files are
about the same items at all: the identity arrays (sources, document ids and lengths, tokens beyond the window) must be
equal element for element.  Step two is one agreement table (``evalstats.agreement``) over every per-sequence array both
files hold, and, when the items pair up, the per-source shift of the losses with the write on and off.  Same purpose as
the reference's ``tools/compare_eval.py``.
"""
from __future__ import annotations

import sys

import numpy as np

from . import evalstats as S

IDENTITY = ("sources", "doc_ids", "doc_lens", "beyond")
BY_SOURCE = ("loss_1.0", "loss_0.0")


def same_items(a, b) -> dict:
    """Identity array -> whether both files hold it with equal contents (arrays neither file has are left out)."""
    held = [k for k in IDENTITY if k in a or k in b]
    return {k: k in a and k in b and a[k].shape == b[k].shape and bool((a[k] == b[k]).all()) for k in held}


def comparable(a, b):
    """Names of the 1-D arrays of equal, non-zero length that both files share (identity arrays excluded)."""
    for k in sorted(set(a).intersection(b).difference(IDENTITY)):
        if np.ndim(a[k]) == 1 and np.shape(a[k]) == np.shape(b[k]) and len(a[k]):
            yield k


def compare(a, b, out=print) -> bool:
    verdicts = same_items(a, b)
    for k, ok in verdicts.items():
        out(f"  {k:10s} {'identical' if ok else 'DIFFERENT'}")
    paired = all(verdicts.values())
    if not paired:
        out("  the files did not score the same sequences: what follows is not a paired comparison")
    table = S.text_table({k: S.agreement(a[k], b[k]) for k in comparable(a, b)}, first="array")
    for line in table.splitlines():
        out("  " + line)
    if paired and "sources" in a:
        src = a["sources"].astype(str)
        for k in (k for k in BY_SOURCE if k in a and k in b):
            shift = {s: float((np.asarray(b[k])[src == s] - np.asarray(a[k])[src == s]).mean()) for s in dict.fromkeys(src)}
            out(f"  {k} B - A by source: " + " | ".join(f"{s} {v:+.5f}" for s, v in shift.items()))
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
