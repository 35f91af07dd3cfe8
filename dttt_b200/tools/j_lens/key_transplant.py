"""Key transplant: is one-off recall beyond the attention window lost at the read's keys, or in what the memory holds?

The planted-recall probe: a span of ``--length`` tokens from chunk 1 is copied into chunk ``window + 3``; its first ``--cue``
tokens stay visible, then every other token is masked and scored (each scored token has a visible predecessor).  Chunks
before the copy are written with the run's own write; the copy's chunk is read in the outer stream's condition.  Per
sequence the mean CE of the scored slots with

    off / on        the memory reset at the read / the memory after all the writes
    on_tx           "on", but every fast layer's memory contribution at the scored slots is taken at the WRITE's input of
                    the source slot holding the same token (``core.Transplant``): the memory queried with the write's keys
    src, src_tx     only chunks 0 .. 1 written (the later writes removed)
    one, one_tx     W_0 + the source chunk's write alone
    off_within      the copy also inside the window (chunk window + 2), memory off: attention's copy (the ceiling)
    off_none / on_none   nothing planted, the same slots: the memory's generic gain there

recall = (off - on) - (off_none - on_none), ceiling = off - off_within.  ``on_tx >> on``: the read's keys do not match the
write's; ``on_tx ~ on``: what is stored is too weak or drowned (``src`` / ``one``: by the other chunks' writes or not).

    python -m dttt_b200.tools.j_lens.key_transplant --ckpt <step dir> --sources name=dir:1.0 --n_per_source 8 --out kt.npz

Role of the reference's ``tools/j_lens/key_transplant.py:1-218``.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np
import torch

from . import _cli
from .core import Reader, Transplant

VARIANTS = ("off", "on", "on_tx", "src", "src_tx", "one", "one_tx", "off_within", "off_none", "on_none")
PLANT_SEED = 12345


def plant(ids: np.ndarray, C: int, src_chunk: int, dst_chunk: int, length: int, cue: int, seed: int):
    """Copy a span of chunk ``src_chunk`` into ``dst_chunk`` (same draw for every target chunk: paired).  Returns the
    planted ids, the scored mask of the target chunk ``[n, C]``, and per scored slot its source slot ``[n, n_scored]``."""
    g = np.random.default_rng(seed)
    n = len(ids)
    out = ids.copy()
    masked = np.zeros((n, C), bool)
    dst_slots, src_slots = [], []
    for i in range(n):
        a = int(g.integers(0, C - length + 1))          # offset within the source chunk
        b = int(g.integers(0, C - length + 1))          # offset within the target chunk
        span = ids[i, src_chunk * C + a: src_chunk * C + a + length]
        out[i, dst_chunk * C + b: dst_chunk * C + b + length] = span
        sc = np.arange(cue + 1, length, 2)              # every other later token
        masked[i, b + sc] = True
        dst_slots.append(b + sc)
        src_slots.append(a + sc)
    return out, masked, np.array(dst_slots), np.array(src_slots)


def source_inputs(reader: Reader, state, ids_chunk: torch.Tensor, slots: np.ndarray, shift: int):
    """The fast branches' inputs of the (clean) source chunk at ``slots - shift`` (the slot whose output predicts that token)."""
    with torch.no_grad():
        _, cap = reader.forward(ids_chunk, state, capture=[("mem_in", i) for i in range(reader.mc.suffix_len)],
                                own="causal" if reader.task == "causal" else "full", shift=reader.task == "causal")
    idx = torch.as_tensor(slots - shift, device=reader.dev).clamp_min(0)
    return [torch.gather(cap[("mem_in", i)], 1, idx[..., None].expand(-1, -1, cap[("mem_in", i)].shape[-1]))
            for i in range(reader.mc.suffix_len) if ("mem_in", i) in cap]


def measure(reader: Reader, ids: np.ndarray, length: int, cue: int, seed: int = PLANT_SEED, log=print) -> dict:
    C, Wn = reader.C, reader.Wn
    src_c, dst_c = 1, Wn + 3
    if ids.shape[1] < (dst_c + 1) * C:
        raise SystemExit(f"sequences of at least {(dst_c + 1) * C} tokens are needed (window {Wn})")
    planted, masked, dst_slots, src_slots = plant(ids, C, src_c, dst_c, length, cue, seed)
    within, _, _, _ = plant(planted, C, src_c, dst_c - 1, length, cue, seed + 1)
    res = {v: [] for v in VARIANTS}
    shift = 1 if reader.outer_shift else 0
    for i in range(len(ids)):
        t = lambda arr: torch.as_tensor(arr[i:i + 1], device=reader.dev)
        chunk = lambda arr, c: t(arr)[:, c * C:(c + 1) * C]
        m = torch.as_tensor(masked[i:i + 1], device=reader.dev)
        dsl = torch.as_tensor(dst_slots[i:i + 1] - shift, device=reader.dev)
        full, snaps = reader.write_pass(t(planted), dst_c, keep=(src_c, src_c + 1))
        x_src = source_inputs(reader, snaps[src_c], chunk(planted, src_c), src_slots[i:i + 1], shift)
        tx = Transplant(dsl, x_src)
        ce = lambda st, arr=planted, **kw: float(reader.mean_ce(reader.read(chunk(arr, dst_c), m, st, **kw), chunk(arr, dst_c), m))
        res["on"].append(ce(full)); res["on_tx"].append(ce(full, transplant=tx)); res["off"].append(ce(reader.reset_memory(full)))
        src_only = reader.with_memory(full, snaps[src_c + 1].W)                       # chunks 0..1 written, the windows as they are
        res["src"].append(ce(src_only)); res["src_tx"].append(ce(src_only, transplant=tx))
        one = reader.write(reader.with_memory(snaps[src_c], reader.reset_memory(full).W), chunk(planted, src_c))
        one_st = reader.with_memory(full, one.W)
        res["one"].append(ce(one_st)); res["one_tx"].append(ce(one_st, transplant=tx))
        w_full, _ = reader.write_pass(t(within), dst_c)
        res["off_within"].append(ce(reader.reset_memory(w_full), within))
        n_full, _ = reader.write_pass(t(ids), dst_c)
        res["on_none"].append(ce(n_full, ids)); res["off_none"].append(ce(reader.reset_memory(n_full), ids))
        log(f"[transplant] sequence {i + 1}/{len(ids)}: off {res['off'][-1]:.3f} on {res['on'][-1]:.3f} on_tx {res['on_tx'][-1]:.3f} "
            f"within {res['off_within'][-1]:.3f}")
    return {k: np.array(v) for k, v in res.items()}


def summarise(res: dict, log=print) -> None:
    ceiling = (res["off"] - res["off_within"]).mean()
    generic = (res["off_none"] - res["on_none"]).mean()
    for k in ("on", "on_tx", "src", "src_tx", "one", "one_tx"):
        gain = (res["off"] - res[k]).mean() - generic
        log(f"[transplant] {k:7s} recall {gain:+.4f} nats = {100 * gain / ceiling if ceiling > 0 else float('nan'):5.1f}% of the ceiling ({ceiling:.4f})")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.j_lens.key_transplant")
    _cli.add_common(ap)
    ap.add_argument("--length", type=int, default=64)
    ap.add_argument("--cue", type=int, default=16)
    a = ap.parse_args(argv)
    reader, ids, names = _cli.load(a)
    res = measure(reader, ids, a.length, a.cue)
    summarise(res)
    if a.out:
        np.savez_compressed(a.out, sources=names, **res)
    return 0


if __name__ == "__main__":
    sys.exit(main())
