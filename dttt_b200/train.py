"""Training entry point: ``python -m dttt_b200.train --config runs/trunk_8k.json [--flag value ...]``
(one process per GPU: ``torchrun --nproc-per-node N -m dttt_b200.train ...``).

Every flag is a ``TrainConfig`` field (``runtime.cliargs``).  A run is a ``Trainer``: it builds the engine, restores what the
configuration asks for (``runtime.restart``), opens the data stream at the right position, builds the evaluation suite
(``runtime.evalsuite``) and then loops ``batch -> Engine.train_step -> log / checkpoint / operator requests / evaluation``.

Operator controls (``runtime.signals``): ``touch <trigger_dir>/TRIGGER_SAVE`` writes a checkpoint at the end of the current step,
``TRIGGER_STOP`` does the same and exits cleanly (``--resume auto`` continues); SIGUSR1 / SIGUSR2 do the same by signal.

Failure handling: a rank that stops answering ends every collective of the others with an error after the heartbeat timeout
(``parallel.mesh.init_distributed``); after any stop the same command is run again and resumes from the newest complete
checkpoint, which is exact because sampling and step keys are functions of ``(seed, step)`` and the data hash is checked.
The reference's counterpart is src/ttt/train.py:810-1199; the log lines keep its format so that its log readers work here.
"""
from __future__ import annotations

import dataclasses as dc
import os
import socket
import sys
import time
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .ckpt import store as ckpt
from .data.host_masks import MaskMaker
from .data.prefetch import Prefetcher
from .data.prep import windows_path
from .data.streams import Plant, Sampler, check_vocab, parse_sources
from .engine import Engine, loss_config
from .eval import probes as PR
from .parallel.mesh import init_distributed, make_mesh
from .runtime import restart as RS
from .runtime.cliargs import train_config_from_argv
from .runtime.evalsuite import EvalSuite, at_scale, parse_write_plan  # noqa: F401  (at_scale: used by the tools)
from .runtime.signals import OperatorSignals, Request
from .schema import ModelConfig, TrainConfig
from .ttt.scan import Batch
from .utils import prof

parse_args = train_config_from_argv


class Trainer:
    """One training run on this rank."""

    def __init__(self, cfg: TrainConfig, rank: int, world: int, local: int):
        self.rank, self.world, self.is_main = rank, world, rank == 0
        self.log = (lambda *a, **k: print(*a, **k, flush=True)) if self.is_main else (lambda *a, **k: None)
        self.device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        elif cfg.compute_dtype == "bfloat16":
            cfg = cfg.replace(compute_dtype="float32")           # CPU runs are the f32 reference path
        self.cfg = cfg
        self.mcfg = ModelConfig.load(cfg.model_config)
        self.signals = OperatorSignals()
        self.signals.clear()
        self.mesh = make_mesh(cfg.fsdp_size, cfg.tp_size, self.device)
        self.data_ranks = self.mesh.batch_ranks
        if cfg.batch_size % self.data_ranks:
            raise ValueError(f"batch_size {cfg.batch_size} must be divisible by {self.data_ranks} data ranks")
        if cfg.grad_accum < 1:
            raise ValueError(f"grad_accum {cfg.grad_accum} must be >= 1")
        self.accum = cfg.grad_accum
        self._announce()
        self.eng = Engine(self.mcfg, cfg, self.mesh, self.device)
        self.log(f"[ttt] {self.eng.n_params / 1e9:.3f}B params")
        self.restart = RS.restore(cfg, self.eng, self.log)
        self._open_data()
        self.cfg = cfg = self.eng.tc                              # "as many as fit" knobs are numbers from here on
        self.lc_base = loss_config(cfg)
        self.lc_train = dc.replace(self.lc_base, time_reweighting="none") if cfg.train_recall else self.lc_base
        self.evals = self._build_evals()
        self.tracker = None
        self.tracker_id = None

    # ------------------------------------------------------------------------------------------------ set-up
    def _announce(self) -> None:
        cfg, m, n = self.cfg, self.mcfg, self.accum
        per_rank = cfg.batch_size // self.data_ranks
        micro = f" x {n} micro-batches = {cfg.batch_size * n} sequences/step" if n > 1 else ""
        self.log(f"[ttt] {self.world} ranks (mesh {self.mesh.shape()}); batch {cfg.batch_size} ({per_rank}/rank){micro}, "
                 f"seq {cfg.seq_len}, steps {cfg.steps}")
        self.log(f"[ttt] model {cfg.model_config}: L={m.num_hidden_layers} H={m.hidden_size} suffix={m.suffix_len} "
                 f"chunk={m.chunk_size} window={m.window_chunks} memory={m.memory}")
        self.log("[ttt] config " + " ".join(f"{k}={v}" for k, v in dc.asdict(cfg).items()))

    def _open_data(self) -> None:
        cfg, m = self.cfg, self.mcfg
        self.sources = parse_sources(cfg.sources, cfg.data_root)
        check_vocab(self.sources, m.vocab_size)
        plant = None
        if cfg.plant_frac > 0:
            if cfg.plant_len_max > m.chunk_size or cfg.seq_len // m.chunk_size < m.window_chunks + 2:
                raise ValueError(f"plant: span <= chunk_size ({m.chunk_size}) and >= window_chunks + 2 chunks per sequence")
            plant = Plant(cfg.plant_frac, cfg.plant_len_min, cfg.plant_len_max, m.chunk_size, m.window_chunks)
        windows = None
        if cfg.doc_windows:
            index_files = [windows_path(s.path, cfg.seq_len, cfg.holdout) for s in self.sources]
            absent = [p for p in index_files if not os.path.exists(p)]
            if absent:
                raise FileNotFoundError(f"doc_windows: build the window index first (python -m dttt_b200.data windows): {absent}")
            windows = [np.load(p) for p in index_files]
        self.sampler_kw = dict(rank=self.mesh.batch_index, world=self.data_ranks, holdout_tokens=cfg.holdout, eos=m.eos_token_id,
                               accum=self.accum)
        self.sampler = Sampler(self.sources, cfg.seq_len, cfg.batch_size, cfg.seed, plant=plant, windows=windows, **self.sampler_kw)
        self.data_offset = RS.data_offset(self.restart, self.sampler, cfg, self.log)
        self.log("[ttt] sources: " + ", ".join(f"{s.name}({s.num_tokens / 1e9:.2f}B, w={s.weight:.2f})" for s in self.sources))
        self.masks = MaskMaker(cfg.inner_mask_mode, m.chunk_size, m.eos_token_id, m.pad_token_id, cfg.data_path(cfg.unigram_path),
                               cfg.inner_target_frac, cfg.inner_generic_floor, cfg.seed, cfg.inner_task)

    def make_batch(self, ids, host=None, outer_t=None, loss_mask=None) -> Batch:
        """Token ids (+ the host-side inner mask / permutation, made here when the caller has none) as a ``Batch``."""
        tokens = ids if torch.is_tensor(ids) else torch.as_tensor(np.asarray(ids))
        if host is None and self.masks.active:
            host = self.masks(np.asarray(tokens))
        inner = {}
        if host is not None:
            inner["inner_perm" if self.cfg.inner_task == "split" else "inner_mask"] = torch.as_tensor(host)
        return Batch(input_ids=tokens, outer_t=None if outer_t is None else torch.as_tensor(outer_t, dtype=torch.float32),
                     loss_mask=None if loss_mask is None else torch.as_tensor(loss_mask), **inner)

    def _build_evals(self) -> EvalSuite:
        cfg = self.cfg
        groups = [(self.sampler, self.sources, True)]
        if cfg.eval_sources and cfg.holdout:
            held_out = parse_sources(cfg.eval_sources, cfg.data_root)
            check_vocab(held_out, self.mcfg.vocab_size)
            groups.append((Sampler(held_out, cfg.seq_len, cfg.batch_size, cfg.seed, eval_only=True, **self.sampler_kw), held_out, False))
        reduce = (lambda t: self.eng.store.all_reduce_scalar(t.to(self.device))) if self.data_ranks > 1 else None
        return EvalSuite(cfg, self.mcfg, self.eng, self.lc_base, groups, self.make_batch, self.log, self.is_main, reduce)

    def _start_tracker(self) -> None:
        """Optional experiment tracker on the main process.  The checkpoint's tracker run is continued only when this run writes
        into the same checkpoint directory; a branch into another directory is a new tracker run."""
        cfg = self.cfg
        if not (cfg.wandb_project and self.is_main):
            return
        try:
            import wandb
            resumed = self.restart.resumed
            same_run = bool(resumed) and os.path.dirname(os.path.abspath(resumed)) == os.path.abspath(cfg.ckpt_dir)
            self.tracker = wandb.init(project=cfg.wandb_project, config={**dc.asdict(cfg), **dc.asdict(self.mcfg)}, resume="allow",
                                      id=self.restart.state.get("wandb_run_id") if same_run else None)
            self.tracker_id = self.tracker.id
            self.evals.on_result = lambda res, step: self.tracker.log(
                {k: v for k, v in res.items() if isinstance(v, (int, float))}, step=step)
        except Exception as e:                                   # noqa: BLE001 - not installed, offline, no credentials
            self.log(f"[ttt] wandb_project={cfg.wandb_project} but the tracker is unavailable ({type(e).__name__}: {e}); "
                     "logging to stdout only")

    # ------------------------------------------------------------------------------------------------ one-off modes
    def probe_memory(self) -> int:
        """One dry step; report the allocator's peak."""
        batches = [self.make_batch(self.sampler.batch(i)) for i in range(self.accum)]
        on_gpu = self.device.type == "cuda"
        if on_gpu:
            torch.cuda.reset_peak_memory_stats()
        self.eng.train_step(batches, 0, self.lc_train)
        if on_gpu:
            gib = 2 ** 30
            self.log(f"[probe] peak allocated {torch.cuda.max_memory_allocated() / gib:.2f} GiB  reserved "
                     f"{torch.cuda.max_memory_reserved() / gib:.2f} GiB per GPU (one step: forward, backward, optimiser)")
        return 0

    # ------------------------------------------------------------------------------------------------ the loop
    def _step_batches(self, prefetch: Prefetcher, stream_step: int) -> List[Batch]:
        cfg, m = self.cfg, self.mcfg
        if not cfg.train_recall:
            out = []
            for i in range(self.accum):
                ids, host = prefetch.get_tensor(stream_step * self.accum + i)
                out.append(self.make_batch(ids.clone(), host))
            return out
        local_ids, host = prefetch.get(stream_step)
        first_row = stream_step * self.sampler.G + self.sampler.rank * self.sampler.local
        ids, scored = PR.recall_train_batch(local_ids, range(first_row, first_row + len(local_ids)), cfg.seed, m.chunk_size, m.window_chunks,
                                            cfg.plant_len_min, cfg.plant_len_max, cfg.train_recall_cue, eos=m.eos_token_id)
        return [self.make_batch(ids, host, outer_t=np.ones(len(ids), np.float32), loss_mask=scored)]

    def _log_step(self, step: int, m: dict, seconds: float) -> None:
        cfg = self.cfg
        tok_s = cfg.batch_size * cfg.seq_len * self.accum / max(seconds, 1e-9)
        extras = [(cfg.inner_feat != "off", lambda: f"feat {m['inner_feat']:.3f}"),
                  (cfg.distill, lambda: f"distill {m['inner_distill']:.3f}"),
                  (cfg.mtp, lambda: f"mtp {m['mtp_loss']:.3f}/{m['inner_mtp']:.3f}"),
                  (cfg.aux_causal_weight > 0, lambda: f"aux x{cfg.aux_causal_weight:g}"),
                  (cfg.inner_kvb_weight > 0, lambda: f"kvb {m['inner_kvb']:.3f}"),
                  ("grad_noise_scale" in m, lambda: f"noise {m['grad_noise_scale']:.0f}"),
                  (bool(m["overflow"]), lambda: f"overflow {m['overflow']}"),
                  (m["grad_norm"] > 2.0 or step < 2,
                   lambda: f"gn[e/p/s/w/o] {m['gnorm_embed']:.2f}/{m['gnorm_prefix']:.2f}/{m['gnorm_suffix']:.2f}/"
                           f"{m['gnorm_fast_weight']:.2f}/{m['gnorm_other']:.2f}")]
        line = (f"[{step:>7}] loss {m['main_loss']:.4f}  inner {m['inner_loss']:.4f}  drift {m['ttt_drift_rel']:.2e}  "
                f"gnorm {m['grad_norm']:.3f}  lr {m['lr']:.2e}  {seconds:.3f}s/step  {tok_s / 1e3:.0f}k tok/s")
        self.log(line + "".join("  " + text() for on, text in extras if on))
        if self.tracker:
            scalars = {f"train/{k}": v for k, v in m.items() if isinstance(v, (int, float))}
            self.tracker.log({**scalars, "train/s_per_step": seconds, "train/tokens_per_s": tok_s}, step=step)

    def _phase_profile(self, step: int, first_step: int, stop_at: int) -> int:
        """``--profile_dir``: phase ranges for two steps early in the run and whenever ``<dir>/TRIGGER`` appears."""
        cfg = self.cfg
        if not (cfg.profile_dir and self.is_main):
            return stop_at
        marker = os.path.join(cfg.profile_dir, "TRIGGER")
        asked = step % cfg.log_interval == 0 and os.path.exists(marker)
        if step == first_step + 2 or asked:
            if os.path.exists(marker):
                os.remove(marker)
            prof.enable(True)
            return step + 2
        if step == stop_at:
            report = prof.report()
            prof.enable(False)
            os.makedirs(cfg.profile_dir, exist_ok=True)
            with open(os.path.join(cfg.profile_dir, f"phases_step{step - 2}.txt"), "w") as fh:
                fh.write(prof.format_report(report) + "\n")
            self.log(f"[ttt] profile (steps {step - 2}-{step - 1}) -> {cfg.profile_dir}")
        return stop_at

    def _checkpoint(self, step: int) -> str:
        state = {"data_offset": self.data_offset}
        if self.tracker_id:
            state["wandb_run_id"] = self.tracker_id
        return ckpt.save(self.cfg.ckpt_dir, step, self.eng, self.sampler.hash, keep=self.cfg.keep_checkpoints, extra_state=state)

    def fit(self) -> int:
        cfg = self.cfg
        first = self.restart.start_step
        self._start_tracker()
        prefetch = Prefetcher(self.sampler, (first - self.data_offset) * self.accum, max(cfg.prefetch, self.accum),
                              self.masks if self.masks.active else None)
        eval_every = cfg.eval_interval or cfg.ckpt_interval
        last_step = cfg.steps - 1
        clock, logged_at = time.time(), first - 1
        profile_stop = -1
        try:
            if cfg.eval_only:
                self.evals.run(first)
                return 0
            if cfg.eval_step0 and (first == 0 or self.restart.continued):
                self.evals.run(first)
            for step in range(first, cfg.steps):
                profile_stop = self._phase_profile(step, first, profile_stop)
                metrics = self.eng.train_step(self._step_batches(prefetch, step - self.data_offset), step, self.lc_train)
                if step % cfg.log_interval == 0 or step == last_step:
                    now = time.time()
                    self._log_step(step, metrics, (now - clock) / max(1, step - logged_at))
                    clock, logged_at = now, step
                due = bool(cfg.ckpt_interval) and ((step + 1) % cfg.ckpt_interval == 0 or step == last_step)
                if due:
                    self.log(f"[ttt] checkpoint -> {self._checkpoint(step)}  (keeping the newest {cfg.keep_checkpoints})")
                request = self.signals.agreed(self.device, self.world)
                if request != Request.NONE:
                    if not due:
                        self.log(f"[ttt] triggered checkpoint -> {self._checkpoint(step)}")
                    self.signals.clear()
                    if request == Request.STOP:
                        self.log(f"[ttt] triggered stop after step {step}: checkpoint written, exiting (--resume auto continues)")
                        break
                if eval_every and ((step + 1) % eval_every == 0 or step == last_step):
                    self.evals.run(step + 1)
        finally:
            prefetch.close()
        return 0


def main(argv=None) -> int:
    rank, world, local = init_distributed()
    cfg = train_config_from_argv(argv)
    role = "main - training log follows" if rank == 0 else "worker - quiet"
    print(f"[ttt] process {rank}/{world} on {socket.gethostname()}: {role}", flush=True)
    try:
        trainer = Trainer(cfg, rank, world, local)
        return trainer.probe_memory() if cfg.probe_memory else trainer.fit()
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:                                    # noqa: BLE001 - a peer is already gone
                pass


if __name__ == "__main__":
    sys.exit(main())
