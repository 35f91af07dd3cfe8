"""The masked-diffusion likelihood bound of a checkpoint and its cross-entropy at every noise level, on held-out
sequences: the unweighted counterpart of the CART-weighted headline.

    python -m dttt_b200.tools.elbo_eval --ckpt <step dir> --n_per_source 6 [--n_t 10] --out log/<dir>/elbo.npz

For ``n_t`` noise levels (the midpoints of equal bins of [0, 1]) the CE of the masked tokens with the write on and with
the write off (the no-write twin; inner-lr scale 0), everything else as in the run's own training loss.  Every
checkpoint scores the same sequences with the same per-sequence keys, so differences between checkpoints are paired.
With i.i.d. masking at rate t the continuous-time bound per token is the integral of CE(t) over [0, 1] (the 1 / t weight
and the t masked tokens cancel): the mean of the CE at the bin midpoints.  Role of the reference's
``tools/elbo_eval.py:1-136``.

The file holds ``ts [n_t]``, ``scales [2]``, ``ce [n_t, 2, n_seq]`` (CE sums), ``count [n_t, 2, n_seq]`` (masked tokens),
``sources [n_seq]`` and ``bound [2]`` (nats per token, write on / off).
"""
from __future__ import annotations

import argparse
import dataclasses as dc
import sys
import time

import numpy as np
import torch


def measure(ctx, ids: np.ndarray, keys: torch.Tensor, ts, scales=(1.0, 0.0), batch: int = 0, log=print):
    """``(ce, count)`` of shape ``[n_t, n_scales, n_seq]``."""
    from ..train import at_scale
    n = len(ids)
    B = batch or ctx.cfg.batch_size
    lc = dc.replace(ctx.lcfg, per_sequence=True, per_token=False, time_reweighting="none", mtp_weight=0.0, aux_causal_weight=0.0,
                    window_drop=0.0, self_prior=0.0, outer_views=1)
    ce = np.zeros((len(ts), len(scales), n))
    cnt = np.zeros_like(ce)
    t0 = time.time()
    for ti, t in enumerate(ts):
        for si, sc in enumerate(scales):
            lcs = at_scale(lc, sc)
            for a in range(0, n, B):
                sl = slice(a, min(n, a + B))
                b = ctx.make_batch(ids[sl], outer_t=np.full(sl.stop - sl.start, t, np.float32))
                with torch.no_grad():
                    _, st = ctx.engine.eval_step(b, keys[sl], ctx.step, lcs)
                m = st["mask_by_seq"].float().cpu().numpy()
                ce[ti, si, sl] = st["loss_by_seq"].float().cpu().numpy() * m
                cnt[ti, si, sl] = m
        log(f"[elbo] t={t:.3f}: CE on {ce[ti, 0].sum() / max(cnt[ti, 0].sum(), 1):.4f}  off {ce[ti, -1].sum() / max(cnt[ti, -1].sum(), 1):.4f}"
            f"  ({time.time() - t0:.0f}s)")
    return ce, cnt


def bound(ce: np.ndarray, cnt: np.ndarray) -> np.ndarray:
    """``[n_scales]``: mean over the noise levels of the token-weighted CE."""
    return (ce.sum(-1) / np.maximum(cnt.sum(-1), 1)).mean(0)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.elbo_eval")
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--n_per_source", type=int, default=6)
    ap.add_argument("--n_t", type=int, default=10)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq_len", type=int, default=0)
    ap.add_argument("--sources", default="")
    ap.add_argument("--data_root", default="")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--out", default="")
    a = ap.parse_args(argv)
    from ..utils import rng
    from .runctx import heldout_sequences, open_run
    ctx = open_run(a.ckpt, seq_len=a.seq_len, batch_size=a.batch, sources=a.sources, data_root=a.data_root)
    ids, names = heldout_sequences(ctx, a.n_per_source)
    keys = rng.split(rng.key(a.seed), len(ids))                    # one key per sequence, the same in every call
    ts = (np.arange(a.n_t) + 0.5) / a.n_t
    scales = (1.0,) if ctx.cfg.no_write else (1.0, 0.0)
    ce, cnt = measure(ctx, ids, keys, ts, scales, a.batch)
    bd = bound(ce, cnt)
    print(f"[elbo] bound (nats/token): write on {bd[0]:.4f}" + (f"  off {bd[-1]:.4f}  memory's part {bd[-1] - bd[0]:+.4f}" if len(scales) > 1 else ""))
    if a.out:
        np.savez_compressed(a.out, ts=ts, scales=np.array(scales), ce=ce, count=cnt, sources=names, bound=bd)
    return 0


if __name__ == "__main__":
    sys.exit(main())
