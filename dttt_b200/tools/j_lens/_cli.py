"""Shared pieces of the ``tools.j_lens`` command lines: options, model and data loading."""
from __future__ import annotations

import argparse
from typing import Tuple

import numpy as np
import torch

from .core import Reader


def add_common(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--ckpt", default=None, help="checkpoint step directory (model, train_config.json, state.json)")
    ap.add_argument("--model_config", default=None, help="default: the checkpoint's own")
    ap.add_argument("--random_init", action="store_true", help="tests: an untrained model of --model_config")
    ap.add_argument("--inner_lr", type=float, default=None, help="default: the checkpoint's ramp at its step")
    ap.add_argument("--inner_task", default=None, help="default: the checkpoint's")
    ap.add_argument("--sources", default="")
    ap.add_argument("--data_root", default="")
    ap.add_argument("--n_per_source", type=int, default=2)
    ap.add_argument("--seq_len", type=int, default=8192)
    ap.add_argument("--synthetic", type=int, default=0, help="tests: random sequences over this many token ids")
    ap.add_argument("--dtype", default="float32", choices=("float32", "bfloat16"))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="")


def load(a) -> Tuple[Reader, np.ndarray, np.ndarray]:
    """``(reader, ids [n, T], source names [n])``: held-out sequences of every source (never training data), or random
    ones with ``--synthetic``."""
    if a.random_init:
        from ...engine import Engine
        from ...parallel.mesh import make_mesh
        from ...schema import ModelConfig, TrainConfig
        dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
        mc = ModelConfig.load(a.model_config)
        tc = TrainConfig(model_config=a.model_config, seq_len=a.seq_len, batch_size=1, seed=a.seed, compute_dtype=a.dtype,
                         inner_task=a.inner_task or "causal", outer_shift=True, inner_lr_warmup_steps=0, fused_ce_block=0)
        eng = Engine(mc, tc, make_mesh(0, 1, dev), dev, trainable=False)
        reader = Reader(eng, tc, 0, a.inner_lr, a.inner_task)
        step = 0
    else:
        from ..runctx import heldout_sequences, open_run
        ctx = open_run(a.ckpt, seq_len=a.seq_len, batch_size=1, sources=a.sources, data_root=a.data_root, compute_dtype=a.dtype)
        reader = Reader(ctx.engine, ctx.cfg, ctx.step, a.inner_lr, a.inner_task)
    if a.synthetic:
        g = np.random.default_rng(a.seed)
        n = max(1, a.n_per_source)
        ids = g.integers(3, a.synthetic, size=(n, a.seq_len)).astype(np.int64)
        return reader, ids, np.array(["synthetic"] * n)
    ids, names = heldout_sequences(ctx, a.n_per_source)
    return reader, np.asarray(ids, np.int64), names
