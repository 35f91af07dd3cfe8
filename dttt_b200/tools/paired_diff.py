"""Paired differences between runs from their per-sequence evaluation arrays (``eval_<step>.npz``).

    python -m dttt_b200.tools.paired_diff --step 1000 A=log/run_a B=log/run_b [C=...]

The first run is the reference.  For every other run: the recipe-mix-weighted difference (run - reference) of the
headline loss (write on), of the no-write twin and of the write gain, each with the naive paired standard error and the
document-cluster bootstrap one (sequences cut from one document are not independent); then every run's own levels and
the per-source headline differences.  Means are token-weighted when every file carries the ``mask`` counts.  Purpose and
functionals as the reference's ``tools/paired_diff.py:1-143``.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np

from . import evalstats as S

KEYS = (("loss_1.0", "headline (write on)"), ("loss_0.0", "no-write twin"), ("gain", "write gain"))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.paired_diff")
    ap.add_argument("runs", nargs="+", help="NAME=DIR")
    ap.add_argument("--step", type=int, default=1000)
    ap.add_argument("--n_boot", type=int, default=S.N_BOOT)
    a = ap.parse_args(argv)
    runs = [tuple(r.split("=", 1)) for r in a.runs]
    data = {n: S.load_npz(os.path.join(d, f"eval_{a.step}.npz")) for n, d in runs}
    ref_name, ref_dir = runs[0]
    ref = data[ref_name]
    for n, d in data.items():
        if not (np.array_equal(d["sources"], ref["sources"]) and np.array_equal(d["doc_ids"], ref["doc_ids"])):
            raise SystemExit(f"{n}: scored other sequences than {ref_name}; the differences would not be paired")
    weights = S.mix_weights(ref_dir) or {str(s): 1.0 for s in np.unique(ref["sources"])}
    tokw = ref.get("mask") if all("mask" in d for d in data.values()) else None
    print(f"step {a.step}; reference {ref_name}; {len(ref['sources'])} sequences of {len(np.unique(ref['doc_ids']))} documents; "
          f"{'token' if tokw is not None else 'sequence'}-weighted; mix over {sum(w > 0 for w in weights.values())} sources")
    print("\n| run - ref | " + " | ".join(t for _, t in KEYS) + " |\n|:--|" + "--:|" * len(KEYS))
    for n, d in data.items():
        if n == ref_name:
            continue
        cells = []
        for k, _ in KEYS:
            if k not in d or k not in ref:
                cells.append("-")
                continue
            m, se_n, se_c = S.mix_stat(d[k] - ref[k], ref["sources"], ref["doc_ids"], weights, tokw, a.n_boot)
            cells.append(f"{m:+.4f} (naive ±{se_n:.4f}, cluster ±{se_c:.4f}, {abs(m) / se_c if se_c > 0 else float('nan'):.1f}σ)")
        print(f"| {n} - {ref_name} | " + " | ".join(cells) + " |")
    print("\n| run | " + " | ".join(t for _, t in KEYS) + " |\n|:--|" + "--:|" * len(KEYS))
    for n, d in data.items():
        cells = []
        for k, _ in KEYS:
            if k not in d:
                cells.append("-")
                continue
            m, _, se_c = S.mix_stat(d[k], d["sources"], d["doc_ids"], weights, d.get("mask") if tokw is not None else None, a.n_boot)
            cells.append(f"{m:.4f} ±{se_c:.4f}")
        print(f"| {n} | " + " | ".join(cells) + " |")
    print("\nper-source headline differences (run - ref), naive ± / cluster ±:")
    for n, d in data.items():
        if n == ref_name:
            continue
        parts = []
        for s in dict.fromkeys(ref["sources"].astype(str)):
            m = ref["sources"].astype(str) == s
            diff = (d["loss_1.0"][m] - ref["loss_1.0"][m]).astype(np.float64)
            w = None if tokw is None else tokw[m]
            parts.append(f"{s} {S.weighted_mean(diff, w):+.4f} ±{S.weighted_se(diff, w):.4f}/±{S.cluster_se(diff, ref['doc_ids'][m], w, a.n_boot):.4f}"
                         f" (n={int(m.sum())})")
        print(f"  {n}: " + "; ".join(parts))
    return 0


if __name__ == "__main__":
    sys.exit(main())
