"""The evaluation programmes of a training run, built once and run at every evaluation step.

A programme is ``Engine.eval_step`` under one ``LossConfig``.  The suite holds (reference src/ttt/train.py:270-672, 1071-1083):

* the held-out loss with the write at each requested inner-rate scale (scale 0 = the write ablation, always included when the
  model writes), optionally with the first chunks re-read (``eval_reread_chunks``);
* the same at fixed masking rates (``eval_fixed_t``: the bound's terms);
* the planted-recall probe (write on / off).
"""
from __future__ import annotations

import dataclasses as dc
from typing import Callable, Dict, List, Optional, Tuple

from ..eval import evaluate as EV
from ..eval import probes as PR
from ..schema import ModelConfig, TrainConfig


def parse_write_plan(spec: str, n_chunks: int) -> Tuple[int, ...]:
    """``"c:k,c:k"`` -> writes per chunk (1 everywhere else); ``()`` for an empty spec."""
    if not spec:
        return ()
    steps = [1] * n_chunks
    for item in filter(None, (s.strip() for s in spec.split(","))):
        chunk, k = (int(v) for v in item.split(":"))
        if chunk >= n_chunks:
            raise ValueError(f"eval_write_plan: chunk {chunk} >= {n_chunks} chunks per sequence")
        steps[chunk] = k
    return tuple(steps)


def at_scale(lc, scale: float):
    """``lc`` with the inner rate multiplied by ``scale``; at 0 the write schemes collapse to the single (inert) step."""
    scaled = dc.replace(lc, inner_lr=scale * lc.inner_lr)
    if scale == 0:
        scaled = dc.replace(scaled, write=dc.replace(scaled.write, steps=1), write_plan=())
    return scaled


def _floats(csv: str) -> List[float]:
    return [float(x) for x in csv.split(",") if x.strip()]


class EvalSuite:
    def __init__(self, cfg: TrainConfig, mcfg: ModelConfig, eng, lc_base, groups, make_batch: Callable, log: Callable, is_main: bool,
                 all_reduce: Optional[Callable]):
        self.cfg, self.mcfg, self.groups, self.make_batch, self.log, self.is_main, self.all_reduce = \
            cfg, mcfg, groups, make_batch, log, is_main, all_reduce
        self.on_result: Optional[Callable[[dict, int], None]] = None          # e.g. the experiment tracker
        self.main: Optional[Dict] = None
        self.fixed_t: Dict[float, Dict] = {}
        self.planted: Optional[Dict] = None
        if not (cfg.holdout and cfg.eval_batches):
            return
        programme = lambda lc: (lambda batch, keys, step: eng.eval_step(batch, keys, step, lc))
        n_chunks = cfg.seq_len // mcfg.chunk_size
        plan = parse_write_plan(cfg.eval_write_plan, n_chunks)
        quiet = dict(mtp_weight=0.0, aux_causal_weight=0.0, window_drop=0.0, self_prior=0.0, outer_views=1)   # training-only terms off
        lc = dc.replace(lc_base, per_sequence=True, per_token=cfg.eval_probes, write_plan=plan, **quiet)
        if cfg.eval_reread_chunks:
            n = cfg.eval_reread_chunks
            seg = lc.segment_chunks or n
            if n % seg:
                raise ValueError(f"eval_reread_chunks {n} must be a multiple of segment_chunks {seg}")
            lc = dc.replace(lc, score_from_chunk=n if cfg.eval_score_from_chunk < 0 else cfg.eval_score_from_chunk, segment_chunks=seg)
        ablation = () if cfg.no_write else (0.0,)
        scales = {1.0, *_floats(cfg.eval_inner_lr_scales), *ablation}
        self.main = {sc: programme(at_scale(lc, sc)) for sc in scales}
        if cfg.eval_reread_chunks:
            self.main["reread"] = programme(dc.replace(lc, reread_chunks=cfg.eval_reread_chunks))
        on_off = (*ablation, 1.0)
        for t in _floats(cfg.eval_fixed_t):
            lc_t = dc.replace(lc, outer_t=t, time_reweighting="none", per_token=False, reread_chunks=0, score_from_chunk=0)
            self.fixed_t[t] = {sc: programme(at_scale(lc_t, sc)) for sc in on_off}
        if cfg.eval_planted_recall:
            PR.planted_chunks(n_chunks, mcfg.window_chunks)                   # refuses sequences too short for a plant
            if cfg.eval_planted_len > mcfg.chunk_size:
                raise ValueError(f"eval_planted_len {cfg.eval_planted_len} > chunk_size {mcfg.chunk_size}")
            lc_p = dc.replace(lc_base, per_sequence=True, per_token=True, time_reweighting="none", outer_t=-1.0, write_plan=plan, **quiet)
            self.planted = {sc: programme(at_scale(lc_p, sc)) for sc in on_off}

    def run(self, step: int) -> dict:
        if self.main is None:
            return {}
        common = dict(is_main=self.is_main)
        res = EV.evaluate(self.main, self.groups, self.cfg, self.mcfg, self.make_batch, step, self.log, all_reduce=self.all_reduce, **common)
        for t, fns in self.fixed_t.items():
            res.update(EV.evaluate(fns, self.groups, self.cfg, self.mcfg, self.make_batch, step, self.log, tag=f" t={t:g}",
                                   all_reduce=self.all_reduce, **common))
        if self.planted is not None:
            res.update(EV.evaluate_planted(self.planted, self.groups, self.cfg, self.mcfg, self.make_batch, step, self.log, **common))
        if self.on_result is not None:
            self.on_result(res, step)
        return res
