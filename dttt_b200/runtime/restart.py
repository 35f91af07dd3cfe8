"""Where a run starts from and which part of its data stream it reads.

Three ways in (semantics of the reference's ``resume`` / ``continue_from`` / ``init_from``, src/ttt/train.py:170-197 and docs/config.md):

* **resume**: the newest complete checkpoint of this run's own directory: weights, optimiser state, step, data position.  The data
  stream must be the one the checkpoint was written on (a hash of sources, sampling and batch geometry), else the run refuses.
* **continue**: another run's checkpoint as the start of a NEW run (own directory): weights, optimiser state and step are taken;
  the data stream is this run's.  If it is the same stream the reading position carries over, otherwise the new stream starts at
  its first sample.
* **init**: weights only.
"""
from __future__ import annotations

import dataclasses as dc
import json
import os
from typing import Callable, Optional

from ..ckpt import store as ckpt
from ..data.streams import Sampler, split_sources
from ..schema import TrainConfig


@dc.dataclass
class Restart:
    start_step: int = 0
    state: dict = dc.field(default_factory=dict)
    resumed: Optional[str] = None              # checkpoint directory this run resumes
    continued: Optional[str] = None            # checkpoint directory of the run this one continues

    @property
    def source(self) -> Optional[str]:
        return self.resumed or self.continued


def _recorded_config(step_dir: str) -> dict:
    with open(os.path.join(step_dir, "train_config.json")) as fh:
        return json.load(fh)


def _sequences_per_step(recorded: dict) -> int:
    return recorded["batch_size"] * recorded.get("grad_accum", 1)


def refuse_unknown_schedule(step_dir: str) -> None:
    """Checkpoints written before the warm-up-stable-decay schedule carry no ``decay_start``; a run that decayed under the older
    schedule cannot be resumed exactly."""
    old = _recorded_config(step_dir)
    if "decay_start" not in old and old["lr"] != old["end_lr"]:
        raise ValueError(f"--resume {step_dir}: the run decayed lr {old['lr']} -> end_lr {old['end_lr']} on a warmup-cosine schedule, "
                         "which does not exist here; --continue_from it or --init_from it")


def restore(cfg: TrainConfig, eng, log: Callable) -> Restart:
    """Load what the configuration asks for into ``eng`` and say where the step counter starts."""
    resumed = ckpt.resolve_resume(cfg.ckpt_dir, "auto" if cfg.continue_from else cfg.resume)
    continued = None
    if not resumed and cfg.continue_from:
        continued = ckpt.resolve_resume(cfg.ckpt_dir, cfg.continue_from)
    plan = Restart(resumed=resumed, continued=continued)
    if resumed:
        refuse_unknown_schedule(resumed)
    if plan.source:
        plan.state = ckpt.read_state(plan.source)
        ckpt.load_weights(plan.source, eng, log)
        ckpt.load_opt(plan.source, eng)
        eng.store.sync_compute()
        plan.start_step = int(plan.state["step"]) + 1
        if resumed:
            log(f"[ttt] resumed {resumed} at step {plan.start_step}")
        else:
            log(f"[ttt] continuing {continued} at step {plan.start_step}: its weights, optimiser state and step; this run's data and settings")
    elif cfg.init_from:
        ckpt.load_weights(cfg.init_from, eng, log)
        eng.store.sync_compute()
        log(f"[ttt] initialised weights from {cfg.init_from}; fresh optimiser and schedule")
    return plan


def verify_same_stream(plan: Restart, sampler: Sampler, cfg: TrainConfig, log: Callable) -> None:
    """A resumed run must read the stream its checkpoint was written on.  Version-2 hashes are independent of file paths;
    version-1 hashes are recomputed in their own form from the stream paths the checkpoint recorded."""
    want = plan.state.get("data_hash")
    version = plan.state.get("data_hash_version", 1)
    if version >= 2:
        got = sampler.hash
    else:
        old = _recorded_config(plan.resumed)
        if _sequences_per_step(old) != sampler.step_batch:
            raise RuntimeError(f"checkpoint {plan.resumed}: {_sequences_per_step(old)} sequences per step, this run {sampler.step_batch}")
        paths_then = {name: path for name, path, _ in split_sources(old["sources"])}
        root = cfg.resume_legacy_root or os.getcwd()
        got = sampler.legacy_hash([os.path.join(root, paths_then.get(s.name, s.path)) for s in sampler.sources], old["batch_size"])
    if got != want:
        raise RuntimeError(f"data configuration changed since checkpoint ({want} != {got}, hash version {version}); use --init_from instead")
    log(f"[ttt] resume data check: hash {want} (version {version}) reproduced")


def data_offset(plan: Restart, sampler: Sampler, cfg: TrainConfig, log: Callable) -> int:
    """The step whose batch is the stream's first sample (``step - offset`` indexes the stream)."""
    if plan.resumed:
        verify_same_stream(plan, sampler, cfg, log)
        return int(plan.state.get("data_offset", 0))
    if not plan.continued:
        return 0
    hashed = plan.state.get("data_hash_version", 1) >= 2
    same = hashed and plan.state.get("data_hash") == sampler.hash
    if hashed and not same:
        then = _sequences_per_step(_recorded_config(plan.continued))
        if then != sampler.step_batch and plan.state.get("data_hash") == sampler.hash_at(then):
            raise ValueError(f"--continue_from {plan.continued}: the same data at another step batch ({then} -> {sampler.step_batch} "
                             "sequences) would read the stream again from its first sample; keep batch_size x grad_accum")
    if same:
        log("[ttt] data: the continued run's stream, read on")
        return int(plan.state.get("data_offset", 0))
    log(f"[ttt] data: a new stream (hash {sampler.hash}), its first batch at step {plan.start_step}")
    return plan.start_step
