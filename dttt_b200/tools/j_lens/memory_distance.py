"""Recall over distance: how much of a one-off span does the memory still return when its copy is read ``d`` chunks after
the span's chunk, with every chunk in between written too?

The planted-recall probe with the copy in chunk ``1 + d`` for every ``d`` of ``--distances``: the same draws at every
distance (paired).  The chunks before a target are natural text whatever the target, so each sequence is written once,
chunk by chunk, with the run's own write; every target chunk is read before it is written.  Per distance, in nats (and in
the summary as % of the ceiling = attention's copy: the span also in the chunk before the target, memory off),
recall = the copy's gain minus the same memory's gain on the unplanted text at the same slots, for the reads

    own       the memory as it is
    write     the memory's contribution at the copy's slots taken at the source slots' inputs (the write's keys)
    ctx       the read chunk's own clean causal inputs (the copy unmasked, causal attention)
    isolated  W_0 + the source chunk's own write (the windows as they are): what the source chunk wrote alone;
              own / isolated is how much of it survives the other writes
    den_iso   the memory as it is with every fast branch normalised by the RMS of the isolated memory's output
    num_iso   the isolated memory normalised by the full memory's RMS

plus the memory's drift ``|W - W_0| / |W_0|`` at the read and, on an i.i.d.-masked read (ratio 0.5, fixed draws) of the target
chunk's natural text, the memory's general gain.  The file holds ``dist [n_d]``, ``gain_copy`` / ``gain_none``
``[n_seq, n_d, 6]`` (memory-off CE minus the read's CE, planted / unplanted), ``ceiling [n_seq, n_d]``, ``drift [n_seq, n_d]``,
``general_gain [n_seq]``, ``sources``.

    python -m dttt_b200.tools.j_lens.memory_distance --ckpt <step dir> --sources name=dir:1.0 --seq_len 32768 \\
        --distances 5,9,17,30 --n_per_source 8 --out distance_32k.npz

Role of the reference's ``tools/j_lens/memory_distance.py:1-236``.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch

from . import _cli
from .core import Reader, Transplant
from .key_transplant import PLANT_SEED, plant, source_inputs

KEYS = ("own", "write", "ctx", "isolated", "den_iso", "num_iso")


def drift(W, W0) -> float:
    num = sum((a.float() - b.float()).pow(2).sum() for w, w0 in zip(W, W0) for a, b in zip(w, w0))
    den = sum(b.float().pow(2).sum() for w0 in W0 for b in w0)
    return float(torch.sqrt(num / den))


def measure(reader: Reader, ids: np.ndarray, distances, length: int, cue: int, log=print) -> dict:
    C = reader.C
    n, nd = len(ids), len(distances)
    out = {"gain_copy": np.zeros((n, nd, len(KEYS))), "gain_none": np.zeros((n, nd, len(KEYS))), "ceiling": np.zeros((n, nd)),
           "drift": np.zeros((n, nd)), "general_gain": np.zeros(n)}
    shift = 1 if reader.outer_shift else 0
    src_c = 1
    g = torch.Generator().manual_seed(PLANT_SEED)
    iid = torch.rand(C, generator=g) < 0.5                                   # the general-gain read: fixed draws
    for i in range(n):
        seq = torch.as_tensor(ids[i:i + 1], device=reader.dev)
        chunk = lambda t_, c: t_[:, c * C:(c + 1) * C]
        targets = [src_c + d for d in distances]
        _, snaps = reader.write_pass(seq, max(targets), keep=[src_c, src_c + 1] + targets + [t - 1 for t in targets])
        W0 = reader.reset_memory(snaps[src_c]).W
        one = reader.write(reader.with_memory(snaps[src_c], W0), chunk(seq, src_c))
        for j, (d, tc) in enumerate(zip(distances, targets)):
            planted, masked, dst_slots, src_slots = plant(ids[i:i + 1], C, src_c, tc, length, cue, PLANT_SEED)
            pl = torch.as_tensor(planted, device=reader.dev)
            m = torch.as_tensor(masked, device=reader.dev)
            st = snaps[tc]
            x_src = source_inputs(reader, snaps[src_c], chunk(seq, src_c), src_slots, shift)
            tx = Transplant(torch.as_tensor(dst_slots - shift, device=reader.dev), x_src)
            iso = reader.with_memory(st, one.W)
            off = reader.reset_memory(st)
            reads = {"own": (st, {}), "write": (st, {"transplant": tx}), "ctx": (st, {"own": "causal"}), "isolated": (iso, {}),
                     "den_iso": (st, {"den_W": one.W}), "num_iso": (iso, {"den_W": st.W})}
            for arr, key in ((pl, "gain_copy"), (seq, "gain_none")):
                x = chunk(arr, tc)
                ce_off = float(reader.mean_ce(reader.read(x, m, off), x, m))
                for k, (state, kw) in reads.items():
                    mm = m if k != "ctx" else torch.zeros_like(m)                # ctx: the copy unmasked, causal inputs
                    lg = reader.read(x, mm, state, **kw)
                    out[key][i, j, KEYS.index(k)] = ce_off - float(reader.mean_ce(lg, x, m))
            # ceiling: the span also in the chunk before the target, memory off
            within, _, _, _ = plant(planted, C, src_c, tc - 1, length, cue, PLANT_SEED + 1)
            wst, _ = reader.write_pass(torch.as_tensor(within, device=reader.dev), tc)
            x = chunk(pl, tc)
            out["ceiling"][i, j] = float(reader.mean_ce(reader.read(x, m, off), x, m)) - \
                float(reader.mean_ce(reader.read(x, m, reader.reset_memory(wst)), x, m))
            out["drift"][i, j] = drift(st.W, W0)
        tc = targets[-1]
        x = chunk(seq, tc)
        mi = iid[None].to(reader.dev)
        out["general_gain"][i] = float(reader.mean_ce(reader.read(x, mi, reader.reset_memory(snaps[tc])), x, mi)) - \
            float(reader.mean_ce(reader.read(x, mi, snaps[tc]), x, mi))
        rec = out["gain_copy"][i, :, 0] - out["gain_none"][i, :, 0]
        log(f"[distance] sequence {i + 1}/{n}: own recall by distance " + " ".join(f"{r:+.3f}" for r in rec) +
            f" | general gain {out['general_gain'][i]:+.4f}")
    return out


def summarise(out: dict, distances, log=print) -> None:
    rec = out["gain_copy"] - out["gain_none"]
    ceil = np.maximum(out["ceiling"], 1e-9)
    for k, name in enumerate(KEYS):
        log(f"[distance] {name:9s} % of ceiling: " + " ".join(f"d={d}: {100 * (rec[:, j, k] / ceil[:, j]).mean():6.1f}" for j, d in enumerate(distances)))
    log(f"[distance] drift |W - W0| / |W0|: " + " ".join(f"d={d}: {out['drift'][:, j].mean():.4f}" for j, d in enumerate(distances)) +
        f" | general gain {out['general_gain'].mean():+.4f} nats")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.j_lens.memory_distance")
    _cli.add_common(ap)
    ap.add_argument("--distances", default="5,9,17,30")
    ap.add_argument("--length", type=int, default=64)
    ap.add_argument("--cue", type=int, default=16)
    a = ap.parse_args(argv)
    reader, ids, names = _cli.load(a)
    dist = [int(x) for x in a.distances.split(",")]
    if ids.shape[1] < (2 + max(dist)) * reader.C:
        raise SystemExit(f"--seq_len must cover chunk {1 + max(dist)}: at least {(2 + max(dist)) * reader.C} tokens")
    out = measure(reader, ids, dist, a.length, a.cue)
    summarise(out, dist)
    if a.out:
        np.savez_compressed(a.out, dist=np.array(dist), sources=names, keys=np.array(KEYS), **out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
