"""How much of the training gradient's noise comes from the mask draw and how much from the data.

    python -m dttt_b200.tools.grad_noise --ckpt <step dir> --n_seq 16 --n_masks 4 [--views 2] --out grad_noise.json

At a checkpoint, with the run's own training loss, ``n_seq`` training sequences each get ``n_masks`` gradients of their
loss, one per key (the key draws the noise level, the mask and the self-prior read).  The loss is the sequence's CE SUM
over its scored tokens: one sequence's share of a batch gradient.  With g_dm the gradient of sequence d under key m, per
parameter group (embedding, prefix, suffix, fast-weight template, rest) and in total:

    mask    W = mean_d [ sum_m |g_dm - g_d.|^2 / (M - 1) ]        noise of the draw, per sequence
    data    D = var_d(g_d.) - W / M                                 noise of the sequence
    signal  |G|^2 = |g_..|^2 - var_d(g_d.) / n_seq                  (unbiased)
    share   W / (W + D)          B_simple = (W + D) / |G|^2  in sequences (McCandlish et al. 2018)

``--views V`` repeats the measurement with V noisy reads per step and times both, so the cost ratio can be set against
the noise cut.  Role of the reference's ``tools/grad_noise.py:1-190``.  Only sums and squared norms are kept, so the
memory cost is three gradient-sized f32 buffers whatever ``n_seq`` and ``n_masks`` are.
"""
from __future__ import annotations

import argparse
import dataclasses as dc
import json
import sys
import time
from typing import Dict

import numpy as np
import torch


def group_slices(store):
    """name of group -> list of (space, start, end) ranges of the flat gradient buffers."""
    from ..optim import group_of
    out: Dict[str, list] = {}
    for name, (space, off, n, _) in store.slots.items():
        out.setdefault(group_of(name), []).append((space, off, off + n))
    return out


def sq_by_group(bufs, groups) -> Dict[str, float]:
    res = {}
    for g, rs in groups.items():
        res[g] = float(sum(bufs[sp][a:b].double().pow(2).sum() for sp, a, b in rs))
    res["total"] = sum(res.values())
    return res


def measure(ctx, ids: np.ndarray, n_masks: int, lcfg, seed: int, log=print):
    from ..utils import rng
    eng = ctx.engine
    st = eng.store
    groups = group_slices(st)
    n = len(ids)
    sum_all = {k: torch.zeros_like(v) for k, v in st.grad.items()}          # sum_d g_d.
    acc_W = {g: 0.0 for g in list(groups) + ["total"]}
    acc_sq_d = {g: 0.0 for g in acc_W}                                        # sum_d |g_d.|^2
    t_grad = []
    for d in range(n):
        sum_d = {k: torch.zeros_like(v) for k, v in st.grad.items()}
        sq_m = {g: 0.0 for g in acc_W}
        b = ctx.make_batch(ids[d:d + 1])
        for m in range(n_masks):
            key = rng.fold_in(rng.fold_in(rng.key(seed), d), m)
            if eng.device.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.time()
            eng.grad_of(b, key, ctx.step, lcfg, weight="sum")
            if eng.device.type == "cuda":
                torch.cuda.synchronize()
            t_grad.append(time.time() - t0)
            for k in sum_d:
                sum_d[k] += st.grad[k]
            for g, v in sq_by_group(st.grad, groups).items():
                sq_m[g] += v
        mean_d = {k: v / n_masks for k, v in sum_d.items()}
        sq_mean = sq_by_group(mean_d, groups)
        for g in acc_W:
            acc_W[g] += (sq_m[g] - n_masks * sq_mean[g]) / max(n_masks - 1, 1)
            acc_sq_d[g] += sq_mean[g]
        for k in sum_all:
            sum_all[k] += mean_d[k]
        log(f"[noise] sequence {d + 1}/{n}: {np.mean(t_grad[-n_masks:]):.2f} s per gradient")
    mean_all = {k: v / n for k, v in sum_all.items()}
    sq_all = sq_by_group(mean_all, groups)
    out = {}
    for g in acc_W:
        W = acc_W[g] / n
        var_d = (acc_sq_d[g] - n * sq_all[g]) / max(n - 1, 1)
        D = var_d - W / n_masks
        G2 = sq_all[g] - var_d / n
        out[g] = {"W": W, "D": D, "G2": G2, "share": W / (W + D) if W + D > 0 else float("nan"),
                  "B_simple": (W + D) / G2 if G2 > 0 else float("inf")}
    return out, float(np.median(t_grad))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.grad_noise")
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--n_seq", type=int, default=16)
    ap.add_argument("--n_masks", type=int, default=4)
    ap.add_argument("--views", type=int, default=1)
    ap.add_argument("--self_prior", type=float, default=-1.0)
    ap.add_argument("--seq_len", type=int, default=0)
    ap.add_argument("--sources", default="")
    ap.add_argument("--data_root", default="")
    ap.add_argument("--seed", type=int, default=4321)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    from .runctx import open_run
    ctx = open_run(a.ckpt, seq_len=a.seq_len, batch_size=1, sources=a.sources, data_root=a.data_root, trainable=True)
    lc = ctx.lcfg if a.self_prior < 0 else dc.replace(ctx.lcfg, self_prior=a.self_prior)
    # training sequences of the run's own sampler, a step far past the run
    far = ctx.step + 10_000_000
    ids = np.concatenate([ctx.sampler.batch(far + i) for i in range(a.n_seq)])[:a.n_seq]
    res = {"ckpt": a.ckpt, "n_seq": a.n_seq, "n_masks": a.n_masks}
    res["views_1"], res["seconds_per_gradient_views_1"] = measure(ctx, ids, a.n_masks, dc.replace(lc, outer_views=1), a.seed)
    if a.views > 1:
        res[f"views_{a.views}"], res[f"seconds_per_gradient_views_{a.views}"] = measure(ctx, ids, a.n_masks, dc.replace(lc, outer_views=a.views), a.seed)
        res["cost_ratio"] = res[f"seconds_per_gradient_views_{a.views}"] / res["seconds_per_gradient_views_1"]
    for k in [k for k in res if k.startswith("views_")]:
        t = res[k]["total"]
        print(f"[noise] {k}: W {t['W']:.4g}  D {t['D']:.4g}  |G|^2 {t['G2']:.4g}  share {t['share']:.3f}  B_simple {t['B_simple']:.1f} sequences")
        print("        " + " | ".join(f"{g} share {v['share']:.2f} B {v['B_simple']:.1f}" for g, v in res[k].items() if g != "total"))
    if a.out:
        with open(a.out, "w") as fh:
            json.dump(res, fh, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
