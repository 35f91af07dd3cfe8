"""Open a finished (or running) run for analysis: the engine with a checkpoint's weights, the run's own loss
configuration, its sources / sampler and the host-side batch builder -- what the offline tools share.

The reference's tools do the same by importing ``train.loss_config`` and the sampler with the checkpoint's
``train_config.json`` (``tools/elbo_eval.py:70-110``, ``tools/grad_noise.py:150-180``).
"""
from __future__ import annotations

import dataclasses as dc
import json
import os
from typing import Optional

import numpy as np
import torch


@dc.dataclass
class RunContext:
    engine: object
    cfg: object                  # TrainConfig
    mcfg: object                 # ModelConfig
    lcfg: object                 # LossConfig of the run
    sampler: object
    sources: list
    make_batch: object
    step: int


def open_run(ckpt_dir: str, device: Optional[torch.device] = None, seq_len: int = 0, batch_size: int = 0, sources: str = "",
             data_root: str = "", trainable: bool = False, **overrides) -> RunContext:
    """``ckpt_dir``: a step directory (``.../ckpt/<step>``) written by ``python -m dttt_b200.train``."""
    from ..ckpt import store as ckpt
    from ..data.host_masks import MaskMaker
    from ..data.streams import Sampler, parse_sources
    from ..engine import Engine, loss_config
    from ..parallel.mesh import make_mesh
    from ..schema import ModelConfig, TrainConfig
    from ..ttt.scan import Batch

    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cfg_path = next((p for p in (os.path.join(ckpt_dir, "train_config.json"), os.path.join(os.path.dirname(ckpt_dir.rstrip("/")), "train_config.json"))
                     if os.path.exists(p)), None)
    if cfg_path is None:
        raise FileNotFoundError(f"no train_config.json in or above {ckpt_dir}")
    raw = json.load(open(cfg_path))
    known = {f.name for f in dc.fields(TrainConfig)}
    kw = {k: v for k, v in raw.items() if k in known}
    kw.update({k: v for k, v in overrides.items() if k in known})
    if seq_len:
        kw["seq_len"] = seq_len
    if batch_size:
        kw["batch_size"] = batch_size
    if sources:
        kw["sources"] = sources
    if data_root:
        kw["data_root"] = data_root
    kw["grad_accum"] = 1
    cfg = TrainConfig(**kw)
    mc_path = os.path.join(ckpt_dir, "model_config.json")
    mcfg = ModelConfig.load(mc_path if os.path.exists(mc_path) else cfg.model_config)
    mesh = make_mesh(0, 1, device)
    eng = Engine(mcfg, cfg, mesh, device, init=False, trainable=trainable)
    st = ckpt.read_state(ckpt_dir)
    ckpt.load_weights(ckpt_dir, eng, lambda *_: None)
    eng.store.sync_compute()
    srcs = parse_sources(cfg.sources, cfg.data_root)
    sampler = Sampler(srcs, cfg.seq_len, cfg.batch_size, cfg.seed, rank=0, world=1, holdout_tokens=cfg.holdout, eos=mcfg.eos_token_id, accum=1)
    mm = MaskMaker(cfg.inner_mask_mode, mcfg.chunk_size, mcfg.eos_token_id, mcfg.pad_token_id, cfg.data_path(cfg.unigram_path),
                   cfg.inner_target_frac, cfg.inner_generic_floor, cfg.seed, cfg.inner_task)

    def make_batch(ids, outer_t=None, loss_mask=None):
        ids_t = torch.as_tensor(np.asarray(ids))
        kw2 = {}
        if mm.active:
            kw2["inner_perm" if cfg.inner_task == "split" else "inner_mask"] = torch.as_tensor(mm(np.asarray(ids_t)))
        return Batch(input_ids=ids_t, outer_t=None if outer_t is None else torch.as_tensor(outer_t, dtype=torch.float32),
                     loss_mask=None if loss_mask is None else torch.as_tensor(loss_mask), **kw2)

    return RunContext(eng, cfg, mcfg, loss_config(cfg), sampler, srcs, make_batch, int(st.get("step", 0)))


def heldout_sequences(ctx: RunContext, n_per_source: int):
    """``(ids [n, T], source names [n])``: the first ``n_per_source`` held-out sequences of every source, in the order the
    training-time evaluation reads them."""
    ids, names = [], []
    B = ctx.cfg.batch_size
    for si, s in enumerate(ctx.sources):
        got = 0
        k = 0
        nb = ctx.sampler.eval_batches(si)
        while got < n_per_source and k < nb:
            b = ctx.sampler.eval_batch(si, k)
            take = min(len(b), n_per_source - got)
            ids.append(np.asarray(b[:take]))
            names += [s.name] * take
            got += take
            k += 1
    return np.concatenate(ids), np.array(names)
