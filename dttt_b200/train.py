"""Training entry point: ``python -m dttt_b200.train --config runs/trunk_8k.json [--flag value ...]``
(one process per GPU: ``torchrun --nproc-per-node N -m dttt_b200.train ...``).

Every flag is a ``TrainConfig`` field; ``--config`` reads a run configuration (``schema.load_run_config``) and
the flags given replace its values (reference ``src/ttt/train.py:97-131``).  The loop is: build or load, then
``for step: batch -> Engine.train_step -> log / checkpoint / triggers / evaluation`` (``train.py:810-1199``).

Operator controls (``train.py:49-91``): ``touch <trigger_dir>/TRIGGER_SAVE`` writes a checkpoint at the end of
the current step, ``TRIGGER_STOP`` does the same and exits cleanly (``--resume auto`` continues); SIGUSR1 /
SIGUSR2 do the same by signal.  The per-rank flags are max-reduced once per step so one host's file is enough.
``<trigger_dir>`` is ``$DTTT_TRIGGER_DIR`` (or ``$TTT_TRIGGER_DIR``), else ``./log``.

Failure handling: a rank that stops answering ends every collective of the others with an error after the
heartbeat timeout (``parallel.mesh.init_distributed``); after any stop the same command is run again and resumes
from the newest complete checkpoint, which is exact because sampling and step keys are functions of
``(seed, step)`` and the data hash is checked (``train.py:170-197``).
"""
from __future__ import annotations

import argparse
import dataclasses as dc
import json
import os
import signal
import socket
import sys
import time
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .ckpt import store as ckpt
from .data.host_masks import MaskMaker
from .data.prefetch import Prefetcher
from .data.prep import windows_path
from .data.streams import Plant, Sampler, check_vocab, parse_sources, split_sources
from .engine import Engine, loss_config
from .eval import evaluate as EV
from .eval import probes as PR
from .parallel.mesh import init_distributed, make_mesh
from .schema import ModelConfig, TrainConfig, load_run_config
from .ttt.scan import Batch
from .utils import prof, rng

TRIGGER_DIR = os.environ.get("DTTT_TRIGGER_DIR") or os.environ.get("TTT_TRIGGER_DIR") or os.path.join(os.getcwd(), "log")
TRIGGER_SAVE, TRIGGER_STOP = 1, 2
_signal_flag = [0]


def install_trigger_signals() -> None:
    def handler(signum, _frame):
        _signal_flag[0] = max(_signal_flag[0], TRIGGER_STOP if signum == signal.SIGUSR2 else TRIGGER_SAVE)
    for sig in (signal.SIGUSR1, signal.SIGUSR2):
        try:
            signal.signal(sig, handler)
        except (ValueError, OSError):
            pass


def poll_trigger() -> int:
    flag = _signal_flag[0]
    if os.path.exists(os.path.join(TRIGGER_DIR, "TRIGGER_STOP")):
        return TRIGGER_STOP
    if os.path.exists(os.path.join(TRIGGER_DIR, "TRIGGER_SAVE")):
        flag = max(flag, TRIGGER_SAVE)
    return flag


def clear_trigger() -> None:
    _signal_flag[0] = 0
    for name in ("TRIGGER_SAVE", "TRIGGER_STOP"):
        try:
            os.remove(os.path.join(TRIGGER_DIR, name))
        except OSError:
            pass


def _coerce(default, v):
    if isinstance(default, float) and isinstance(v, int) and not isinstance(v, bool):
        return float(v)
    if isinstance(default, int) and not isinstance(default, bool) and isinstance(v, float) and v.is_integer():
        return int(v)
    return v


def parse_args(argv=None) -> TrainConfig:
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--config", default="")
    run = pre.parse_known_args(argv)[0].config
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.train", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("--config", default="", help="run configuration (JSON of these fields; 'base' inherits)")
    defaults = {}
    truthy = lambda s: s.lower() in ("1", "true", "yes")
    for f in dc.fields(TrainConfig):
        defaults[f.name] = f.default
        if isinstance(f.default, bool):
            ap.add_argument(f"--{f.name}", type=truthy, default=f.default, dest=f.name)
        elif isinstance(f.default, tuple):
            ap.add_argument(f"--{f.name}", type=type(f.default[0]), nargs=2, metavar=("LO", "HI"), default=f.default, dest=f.name)
        else:
            ap.add_argument(f"--{f.name}", type=type(f.default), default=f.default, dest=f.name)
    if run:
        ap.set_defaults(**{k: _coerce(defaults[k], v) for k, v in load_run_config(run).items()})
    d = vars(ap.parse_args(argv))
    d.pop("config")
    for name in ("inner_mask_range", "distill_t_range"):
        d[name] = tuple(d[name])
    return TrainConfig(**d)


def check_resume_data(d: str, st: dict, sampler: Sampler, cfg: TrainConfig, log=print) -> None:
    """Refuse to resume on another training stream (hash version 2 is path-free; version 1 is recomputed in its
    own form from the checkpoint's recorded stream paths; reference train.py:170-197)."""
    want, version = st.get("data_hash"), st.get("data_hash_version", 1)
    if version >= 2:
        got = sampler.hash
    else:
        with open(os.path.join(d, "train_config.json")) as fh:
            old = json.load(fh)
        old_step = old["batch_size"] * old.get("grad_accum", 1)
        if old_step != sampler.step_batch:
            raise RuntimeError(f"checkpoint {d}: {old_step} sequences per step, this run {sampler.step_batch}")
        recorded = {name: path for name, path, _ in split_sources(old["sources"])}
        root = cfg.resume_legacy_root or os.getcwd()
        got = sampler.legacy_hash([os.path.join(root, recorded.get(s.name, s.path)) for s in sampler.sources], old["batch_size"])
    if got != want:
        raise RuntimeError(f"data configuration changed since checkpoint ({want} != {got}, hash version {version}); use --init_from instead")
    log(f"[ttt] resume data check: hash {want} (version {version}) reproduced")


def check_resume_schedule(d: str) -> None:
    with open(os.path.join(d, "train_config.json")) as fh:
        old = json.load(fh)
    if "decay_start" not in old and old["lr"] != old["end_lr"]:
        raise ValueError(f"--resume {d}: the run decayed lr {old['lr']} -> end_lr {old['end_lr']} on a warmup-cosine schedule, "
                         "which does not exist here; --continue_from it or --init_from it")


def write_plan(cfg: TrainConfig, nc: int):
    if not cfg.eval_write_plan:
        return ()
    plan = [1] * nc
    for item in cfg.eval_write_plan.split(","):
        if item.strip():
            c, k = (int(v) for v in item.split(":"))
            if c >= nc:
                raise ValueError(f"eval_write_plan: chunk {c} >= {nc} chunks per sequence")
            plan[c] = k
    return tuple(plan)


def at_scale(lc, sc: float):
    lc = dc.replace(lc, inner_lr=sc * lc.inner_lr)
    return dc.replace(lc, write=dc.replace(lc.write, steps=1), write_plan=()) if sc == 0 else lc


def main(argv=None) -> int:
    rank, world, local = init_distributed()
    cfg = parse_args(argv)
    install_trigger_signals()
    clear_trigger()
    mcfg = ModelConfig.load(cfg.model_config)
    is_main = rank == 0
    print(f"[ttt] process {rank}/{world} on {socket.gethostname()}: " + ("main - training log follows" if is_main else "worker - quiet"), flush=True)
    log = (lambda *a, **k: print(*a, **k, flush=True)) if is_main else (lambda *a, **k: None)
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    elif cfg.compute_dtype == "bfloat16":
        cfg = cfg.replace(compute_dtype="float32")           # CPU runs are the f32 reference path
    mesh = make_mesh(cfg.fsdp_size, cfg.tp_size, device)
    nb = mesh.batch_ranks
    if cfg.batch_size % nb:
        raise ValueError(f"batch_size {cfg.batch_size} must be divisible by {nb} data ranks")
    if cfg.grad_accum < 1:
        raise ValueError(f"grad_accum {cfg.grad_accum} must be >= 1")
    N = cfg.grad_accum
    log(f"[ttt] {world} ranks (mesh {mesh.shape()}); batch {cfg.batch_size} ({cfg.batch_size // nb}/rank)"
        + (f" x {N} micro-batches = {cfg.batch_size * N} sequences/step" if N > 1 else "") + f", seq {cfg.seq_len}, steps {cfg.steps}")
    log(f"[ttt] model {cfg.model_config}: L={mcfg.num_hidden_layers} H={mcfg.hidden_size} suffix={mcfg.suffix_len} "
        f"chunk={mcfg.chunk_size} window={mcfg.window_chunks} memory={mcfg.memory}")
    log("[ttt] config " + " ".join(f"{k}={v}" for k, v in dc.asdict(cfg).items()))

    eng = Engine(mcfg, cfg, mesh, device)
    log(f"[ttt] {eng.n_params / 1e9:.3f}B params")
    start_step = 0
    resume_dir = ckpt.resolve_resume(cfg.ckpt_dir, "auto" if cfg.continue_from else cfg.resume)
    cont_dir = None if resume_dir or not cfg.continue_from else ckpt.resolve_resume(cfg.ckpt_dir, cfg.continue_from)
    st: dict = {}
    if resume_dir:
        check_resume_schedule(resume_dir)
    if resume_dir or cont_dir:
        from_dir = resume_dir or cont_dir
        st = ckpt.read_state(from_dir)
        ckpt.load_weights(from_dir, eng, log)
        ckpt.load_opt(from_dir, eng)
        eng.store.sync_compute()
        start_step = int(st["step"]) + 1
        log(f"[ttt] resumed {from_dir} at step {start_step}" if resume_dir else
            f"[ttt] continuing {from_dir} at step {start_step}: its weights, optimiser state and step; this run's data and settings")
    elif cfg.init_from:
        ckpt.load_weights(cfg.init_from, eng, log)
        eng.store.sync_compute()
        log(f"[ttt] initialised weights from {cfg.init_from}; fresh optimiser and schedule")

    # ---- data
    sources = parse_sources(cfg.sources, cfg.data_root)
    check_vocab(sources, mcfg.vocab_size)
    plant = None
    if cfg.plant_frac > 0:
        if cfg.plant_len_max > mcfg.chunk_size or cfg.seq_len // mcfg.chunk_size < mcfg.window_chunks + 2:
            raise ValueError(f"plant: span <= chunk_size ({mcfg.chunk_size}) and >= window_chunks + 2 chunks per sequence")
        plant = Plant(cfg.plant_frac, cfg.plant_len_min, cfg.plant_len_max, mcfg.chunk_size, mcfg.window_chunks)
    windows = None
    if cfg.doc_windows:
        paths = [windows_path(s.path, cfg.seq_len, cfg.holdout) for s in sources]
        missing = [p for p in paths if not os.path.exists(p)]
        if missing:
            raise FileNotFoundError(f"doc_windows: build the window index first (python -m dttt_b200.data windows): {missing}")
        windows = [np.load(p) for p in paths]
    skw = dict(rank=mesh.batch_index, world=nb, holdout_tokens=cfg.holdout, eos=mcfg.eos_token_id, accum=N)
    sampler = Sampler(sources, cfg.seq_len, cfg.batch_size, cfg.seed, plant=plant, windows=windows, **skw)
    data_offset = 0
    if resume_dir:
        check_resume_data(resume_dir, st, sampler, cfg, log)
        data_offset = int(st.get("data_offset", 0))
    elif cont_dir:
        same = st.get("data_hash_version", 1) >= 2 and st.get("data_hash") == sampler.hash
        if not same and st.get("data_hash_version", 1) >= 2:
            with open(os.path.join(cont_dir, "train_config.json")) as fh:
                old = json.load(fh)
            old_step = old["batch_size"] * old.get("grad_accum", 1)
            if old_step != sampler.step_batch and st.get("data_hash") == sampler.hash_at(old_step):
                raise ValueError(f"--continue_from {cont_dir}: the same data at another step batch ({old_step} -> {sampler.step_batch} "
                                 "sequences) would read the stream again from its first sample; keep batch_size x grad_accum")
        data_offset = int(st.get("data_offset", 0)) if same else start_step
        log("[ttt] data: " + ("the continued run's stream, read on" if same else
                              f"a new stream (hash {sampler.hash}), its first batch at step {start_step}"))
    log("[ttt] sources: " + ", ".join(f"{s.name}({s.num_tokens / 1e9:.2f}B, w={s.weight:.2f})" for s in sources))
    mask_maker = MaskMaker(cfg.inner_mask_mode, mcfg.chunk_size, mcfg.eos_token_id, mcfg.pad_token_id, cfg.data_path(cfg.unigram_path),
                           cfg.inner_target_frac, cfg.inner_generic_floor, cfg.seed, cfg.inner_task)

    def make_batch(ids, host=None, outer_t=None, loss_mask=None) -> Batch:
        ids_t = torch.as_tensor(np.asarray(ids)) if not torch.is_tensor(ids) else ids
        if host is None and mask_maker.active:
            host = mask_maker(np.asarray(ids_t))
        kw = {}
        if host is not None:
            kw["inner_perm" if cfg.inner_task == "split" else "inner_mask"] = torch.as_tensor(host)
        return Batch(input_ids=ids_t, outer_t=None if outer_t is None else torch.as_tensor(outer_t, dtype=torch.float32),
                     loss_mask=None if loss_mask is None else torch.as_tensor(loss_mask), **kw)

    # ---- evaluation programmes
    lc_base = loss_config(cfg)
    lc_train = dc.replace(lc_base, time_reweighting="none") if cfg.train_recall else lc_base
    eval_every = cfg.eval_interval or cfg.ckpt_interval
    groups = [(sampler, sources, True)]
    if cfg.eval_sources and cfg.holdout:
        ev_sources = parse_sources(cfg.eval_sources, cfg.data_root)
        check_vocab(ev_sources, mcfg.vocab_size)
        groups.append((Sampler(ev_sources, cfg.seq_len, cfg.batch_size, cfg.seed, eval_only=True, **skw), ev_sources, False))
    fn_for = lambda lc: (lambda b, keys, step: eng.eval_step(b, keys, step, lc))
    eval_fns = eval_fixed = planted_fns = None
    nc = cfg.seq_len // mcfg.chunk_size
    if cfg.holdout and cfg.eval_batches:
        lc = dc.replace(lc_base, per_sequence=True, per_token=cfg.eval_probes, mtp_weight=0.0, aux_causal_weight=0.0,
                        write_plan=write_plan(cfg, nc), window_drop=0.0, self_prior=0.0, outer_views=1)
        if cfg.eval_reread_chunks:
            n = cfg.eval_reread_chunks
            seg = lc.segment_chunks or n
            if n % seg:
                raise ValueError(f"eval_reread_chunks {n} must be a multiple of segment_chunks {seg}")
            lc = dc.replace(lc, score_from_chunk=n if cfg.eval_score_from_chunk < 0 else cfg.eval_score_from_chunk, segment_chunks=seg)
        scales = {1.0} | {float(x) for x in cfg.eval_inner_lr_scales.split(",") if x.strip()}
        if not cfg.no_write:
            scales.add(0.0)
        eval_fns = {sc: fn_for(at_scale(lc, sc)) for sc in scales}
        if cfg.eval_reread_chunks:
            eval_fns["reread"] = fn_for(dc.replace(lc, reread_chunks=cfg.eval_reread_chunks))
        eval_fixed = {}
        for t_fixed in [float(x) for x in cfg.eval_fixed_t.split(",") if x.strip()]:
            lc_t = dc.replace(lc, outer_t=t_fixed, time_reweighting="none", per_token=False, reread_chunks=0, score_from_chunk=0)
            eval_fixed[t_fixed] = {sc: fn_for(at_scale(lc_t, sc)) for sc in ((0.0, 1.0) if not cfg.no_write else (1.0,))}
        if cfg.eval_planted_recall:
            PR.planted_chunks(nc, mcfg.window_chunks)
            if cfg.eval_planted_len > mcfg.chunk_size:
                raise ValueError(f"eval_planted_len {cfg.eval_planted_len} > chunk_size {mcfg.chunk_size}")
            lc_p = dc.replace(lc_base, per_sequence=True, per_token=True, mtp_weight=0.0, aux_causal_weight=0.0, time_reweighting="none",
                              outer_t=-1.0, write_plan=write_plan(cfg, nc), window_drop=0.0, self_prior=0.0, outer_views=1)
            planted_fns = {sc: fn_for(at_scale(lc_p, sc)) for sc in ((0.0, 1.0) if not cfg.no_write else (1.0,))}

    def all_reduce(t):
        t = t.to(device)
        return eng.store.all_reduce_scalar(t)

    wb_holder = [None]                                           # set once the tracker is up (it starts after this definition)

    def run_eval(step):
        if eval_fns is None:
            return {}
        ar = all_reduce if nb > 1 else None
        ev = EV.evaluate(eval_fns, groups, cfg, mcfg, make_batch, step, log, is_main=is_main, all_reduce=ar)
        for t_fixed, fns in (eval_fixed or {}).items():
            ev.update(EV.evaluate(fns, groups, cfg, mcfg, make_batch, step, log, is_main=is_main, tag=f" t={t_fixed:g}", all_reduce=ar))
        if planted_fns is not None:
            ev.update(EV.evaluate_planted(planted_fns, groups, cfg, mcfg, make_batch, step, log, is_main=is_main))
        if wb_holder[0] is not None:
            wb_holder[0].log({k: v for k, v in ev.items() if isinstance(v, (int, float))}, step=step)
        return ev

    # ---- memory probe: one dry step, report the allocator's peak, exit
    if cfg.probe_memory:
        b = [make_batch(sampler.batch(m)) for m in range(N)]
        if device.type == "cuda":
            torch.cuda.reset_peak_memory_stats()
        eng.train_step(b, 0, lc_train)
        if device.type == "cuda":
            log(f"[probe] peak allocated {torch.cuda.max_memory_allocated() / 2**30:.2f} GiB  reserved "
                f"{torch.cuda.max_memory_reserved() / 2**30:.2f} GiB per GPU (one step: forward, backward, optimiser)")
        return 0

    # ---- experiment tracker (main process only, optional): continue the checkpoint's run only when this run writes into the
    # same checkpoint directory; a branch into another directory is a new run (reference train.py:1049-1056)
    wb = None
    wb_id = None
    if cfg.wandb_project and is_main:
        try:
            import wandb
            same_run = bool(resume_dir) and os.path.dirname(os.path.abspath(resume_dir)) == os.path.abspath(cfg.ckpt_dir)
            wb = wandb.init(project=cfg.wandb_project, config={**dc.asdict(cfg), **dc.asdict(mcfg)}, resume="allow",
                            id=st.get("wandb_run_id") if same_run else None)
            wb_id = wb.id
            wb_holder[0] = wb
        except Exception as e:                                   # noqa: BLE001 - not installed, offline, no credentials
            log(f"[ttt] wandb_project={cfg.wandb_project} but the tracker is unavailable ({type(e).__name__}: {e}); logging to stdout only")
    prefetch = Prefetcher(sampler, (start_step - data_offset) * N, max(cfg.prefetch, N), mask_maker if mask_maker.active else None)
    save_state = lambda: {"data_offset": data_offset, **({"wandb_run_id": wb_id} if wb_id else {})}
    tokens_per_step = cfg.batch_size * cfg.seq_len * N
    t_last, last_log = time.time(), start_step - 1
    trace = None
    try:
        if cfg.eval_only:
            run_eval(start_step)
            return 0
        if (start_step == 0 or cont_dir) and cfg.eval_step0:
            run_eval(start_step)
        profile_stop = -1
        for step in range(start_step, cfg.steps):
            if cfg.profile_dir and is_main:
                trig = os.path.join(cfg.profile_dir, "TRIGGER")
                if step == start_step + 2 or (step % cfg.log_interval == 0 and os.path.exists(trig)):
                    if os.path.exists(trig):
                        os.remove(trig)
                    prof.enable(True)
                    profile_stop = step + 2
                elif step == profile_stop:
                    rep = prof.report()
                    prof.enable(False)
                    os.makedirs(cfg.profile_dir, exist_ok=True)
                    with open(os.path.join(cfg.profile_dir, f"phases_step{step - 2}.txt"), "w") as fh:
                        fh.write(prof.format_report(rep) + "\n")
                    log(f"[ttt] profile (steps {step - 2}-{step - 1}) -> {cfg.profile_dir}")
            ds = step - data_offset
            if cfg.train_recall:
                local_ids, host = prefetch.get(ds)
                j0 = ds * sampler.G + sampler.rank * sampler.local
                ids_r, lm_r = PR.recall_train_batch(local_ids, range(j0, j0 + len(local_ids)), cfg.seed, mcfg.chunk_size,
                                                    mcfg.window_chunks, cfg.plant_len_min, cfg.plant_len_max, cfg.train_recall_cue,
                                                    eos=mcfg.eos_token_id)
                batches = [make_batch(ids_r, host, outer_t=np.ones(len(ids_r), np.float32), loss_mask=lm_r)]
            else:
                batches = []
                for m in range(N):
                    ids_t, host = prefetch.get_tensor(ds * N + m)
                    batches.append(make_batch(ids_t.clone(), host))
            m = eng.train_step(batches, step, lc_train)
            if step % cfg.log_interval == 0 or step == cfg.steps - 1:
                now = time.time()
                dt = (now - t_last) / max(1, step - last_log)
                t_last, last_log = now, step
                tps = tokens_per_step / max(dt, 1e-9)
                log(f"[{step:>7}] loss {m['main_loss']:.4f}  inner {m['inner_loss']:.4f}  drift {m['ttt_drift_rel']:.2e}  "
                    f"gnorm {m['grad_norm']:.3f}  lr {m['lr']:.2e}  {dt:.3f}s/step  {tps / 1e3:.0f}k tok/s"
                    + (f"  feat {m['inner_feat']:.3f}" if cfg.inner_feat != "off" else "")
                    + (f"  distill {m['inner_distill']:.3f}" if cfg.distill else "")
                    + (f"  mtp {m['mtp_loss']:.3f}/{m['inner_mtp']:.3f}" if cfg.mtp else "")
                    + (f"  aux x{cfg.aux_causal_weight:g}" if cfg.aux_causal_weight > 0 else "")
                    + (f"  kvb {m['inner_kvb']:.3f}" if cfg.inner_kvb_weight > 0 else "")
                    + (f"  noise {m['grad_noise_scale']:.0f}" if "grad_noise_scale" in m else "")
                    + (f"  overflow {m['overflow']}" if m["overflow"] else "")
                    + (f"  gn[e/p/s/w/o] {m['gnorm_embed']:.2f}/{m['gnorm_prefix']:.2f}/{m['gnorm_suffix']:.2f}/"
                       f"{m['gnorm_fast_weight']:.2f}/{m['gnorm_other']:.2f}" if m["grad_norm"] > 2.0 or step < 2 else ""))
                if wb:
                    wb.log({**{f"train/{k}": v for k, v in m.items() if isinstance(v, (int, float))}, "train/s_per_step": dt,
                            "train/tokens_per_s": tps}, step=step)
            saved_here = False
            if cfg.ckpt_interval and ((step + 1) % cfg.ckpt_interval == 0 or step == cfg.steps - 1):
                d = ckpt.save(cfg.ckpt_dir, step, eng, sampler.hash, keep=cfg.keep_checkpoints, extra_state=save_state())
                log(f"[ttt] checkpoint -> {d}  (keeping the newest {cfg.keep_checkpoints})")
                saved_here = True
            flag = poll_trigger()
            if world > 1:
                ft = torch.tensor([flag], device=device)
                dist.all_reduce(ft, op=dist.ReduceOp.MAX)
                flag = int(ft.item())
            if flag:
                if not saved_here:
                    d = ckpt.save(cfg.ckpt_dir, step, eng, sampler.hash, keep=cfg.keep_checkpoints, extra_state=save_state())
                    log(f"[ttt] triggered checkpoint -> {d}")
                clear_trigger()
                if flag == TRIGGER_STOP:
                    log(f"[ttt] triggered stop after step {step}: checkpoint written, exiting (--resume auto continues)")
                    break
            if eval_every and ((step + 1) % eval_every == 0 or step == cfg.steps - 1):
                run_eval(step + 1)
    finally:
        prefetch.close()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
