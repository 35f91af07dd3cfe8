"""Checkpoints: f32 master weights, optimiser state and the metadata a resume needs.

Layout (the reference's, ``src/ttt/checkpoint.py:5-12``)::

    {ckpt_dir}/step_{N:08d}/
        model.eqx.part*      .npy records of the parameter leaves, f32, in ``models.params.param_spec`` order
        opt.eqx.part*        .npy records: Adam count (int32), first moments, second moments (parameter order each),
                             schedule count (int32) - the leaf order of ``optax.chain(clip, adamw)``
        model_config.json    train_config.json
        state.json           {step, data_hash, data_hash_version: 2, git, time, data_offset, ...}
        DONE                 written last; a directory without it is ignored

Every rank takes part in ``save`` (the shards of each parameter are gathered one parameter at a time), rank 0
writes, a barrier follows (``checkpoint.py:97-120``).  ``load_weights`` tolerates optional heads the saved
model did not have and narrows a wider saved fast weight by magnitude pruning (``:143-221``).  Three ways in
(``docs/config.md:40-57``): ``resume`` (same run, data hash checked), ``continue_from`` (another run's step
directory: weights, optimiser state and step), ``init_from`` (weights only).
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import time
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..models.params import param_spec
from ..schema import ModelConfig
from . import npystream as NS

# optional model fields -> (config key, value meaning "absent")
OPTIONAL = {"inner_gate": ("inner_lr_gate", False), "inner_token_gate": ("inner_token_gate", False),
            "inner_decay_logit": ("inner_decay", 0.0), "inner_precond": ("inner_optimizer", False),
            "inner_step_log": ("inner_optimizer", False), "inner_temp_log": ("inner_optimizer", False),
            "inner_feat_head": ("inner_feat_head", False), "mtp_head": ("mtp_head", False),
            "inner_kvb_value": ("inner_kvb_head", False)}


def git_info() -> dict:
    env = os.environ
    commit = env.get("DTTT_GIT_COMMIT") or env.get("TTT_GIT_COMMIT")
    if commit:
        return {"commit": commit, "branch": env.get("DTTT_GIT_BRANCH", env.get("TTT_GIT_BRANCH", "")),
                "dirty": env.get("DTTT_GIT_DIRTY", env.get("TTT_GIT_DIRTY", "0")) == "1"}
    try:
        run = lambda *a: subprocess.run(["git", *a], capture_output=True, text=True, timeout=5).stdout.strip()
        return {"commit": run("rev-parse", "HEAD"), "branch": run("rev-parse", "--abbrev-ref", "HEAD"),
                "dirty": bool(run("status", "--porcelain"))}
    except Exception:
        return {}


def step_dir(ckpt_dir: str, step: int) -> str:
    return os.path.join(ckpt_dir, f"step_{step:08d}")


def complete_steps(ckpt_dir: str) -> List[str]:
    if not os.path.isdir(ckpt_dir):
        return []
    return sorted(d for d in os.listdir(ckpt_dir) if d.startswith("step_") and os.path.exists(os.path.join(ckpt_dir, d, "DONE")))


def latest_complete(ckpt_dir: str) -> Optional[str]:
    done = complete_steps(ckpt_dir)
    return os.path.join(ckpt_dir, done[-1]) if done else None


def prune(ckpt_dir: str, keep: int) -> List[str]:
    if keep <= 0:
        return []
    gone = complete_steps(ckpt_dir)[:-keep]
    for d in gone:
        shutil.rmtree(os.path.join(ckpt_dir, d), ignore_errors=True)
    return gone


def resolve_resume(ckpt_dir: str, spec: str) -> Optional[str]:
    if not spec:
        return None
    if spec == "auto":
        return latest_complete(ckpt_dir)
    if not os.path.exists(os.path.join(spec, "DONE")):
        raise FileNotFoundError(f"{spec} is not a complete checkpoint (no DONE marker)")
    return spec


def read_state(d: str) -> dict:
    with open(os.path.join(d, "state.json")) as fh:
        return json.load(fh)


def _barrier() -> None:
    if dist.is_initialized():
        dist.barrier()


def save(ckpt_dir: str, step: int, engine, data_hash: str, keep: int = 0, extra_state: Optional[dict] = None) -> str:
    """Write a complete checkpoint (collective: every rank calls it)."""
    d = step_dir(ckpt_dir, step)
    st, opt = engine.store, engine.opt
    main = engine.mesh.rank == 0

    def leaves(buf=None):
        for name in st.names():
            t = st.gather_full(name, buf)                      # collective, one parameter at a time
            yield t.cpu().numpy() if main else None

    if main:
        os.makedirs(d, exist_ok=True)
        NS.write_records(os.path.join(d, "model.eqx"), leaves())
    else:
        for _ in leaves():
            pass
    if opt is not None:
        def opt_leaves():
            yield np.asarray(opt.count, np.int32)
            yield from leaves(opt.m)
            yield from leaves(opt.v)
            yield np.asarray(opt.count, np.int32)
        if main:
            NS.write_records(os.path.join(d, "opt.eqx"), opt_leaves())
        else:
            for _ in opt_leaves():
                pass
    if main:
        engine.mc.save(os.path.join(d, "model_config.json"))
        engine.tc.save(os.path.join(d, "train_config.json"))
        with open(os.path.join(d, "state.json"), "w") as fh:
            json.dump({"step": int(step), "data_hash": data_hash, "data_hash_version": 2, "git": git_info(), "time": time.time(),
                       **(extra_state or {})}, fh, indent=2)
        with open(os.path.join(d, "DONE"), "w") as fh:
            fh.write("ok\n")
        prune(ckpt_dir, keep)
    _barrier()
    return d


def _saved_config(d: str) -> Optional[dict]:
    p = os.path.join(d, "model_config.json")
    if not os.path.exists(p):
        return None
    with open(p) as fh:
        return json.load(fh)


def prune_fast_weight(gate: np.ndarray, up: np.ndarray, down: np.ndarray, inter: int):
    """Narrow a stacked SwiGLU fast weight ``[F,H,I] / [F,I,H]`` to ``inter`` hidden units per layer, keeping the
    units of largest ``|gate_j| |up_j| |down_j|`` in their original order (reference checkpoint.py:170-180)."""
    imp = np.linalg.norm(gate, axis=1) * np.linalg.norm(up, axis=1) * np.linalg.norm(down, axis=2)
    keep = np.sort(np.argsort(-imp, axis=1)[:, :inter], axis=1)
    g = np.stack([gate[f][:, keep[f]] for f in range(gate.shape[0])])
    u = np.stack([up[f][:, keep[f]] for f in range(up.shape[0])])
    dn = np.stack([down[f][keep[f], :] for f in range(down.shape[0])])
    return g, u, dn


def load_weights(d: str, engine, log=print) -> None:
    """Weights only, into the engine's sharded store (every rank reads the file)."""
    mc: ModelConfig = engine.mc
    saved = _saved_config(d)
    # through the schema loader: a file written by the reference or by an older run may still carry retired keys at their "off" value
    saved_spec = param_spec(ModelConfig.load(os.path.join(d, "model_config.json"))) if saved is not None else engine.spec
    missing = [n for n in engine.spec if n not in saved_spec]
    for n in missing:
        field = n.split(".")[0]
        if field not in OPTIONAL:
            raise ValueError(f"checkpoint {d} has no parameter {n}")
        log(f"[ttt] checkpoint {d} has no {n}: keeping its initialisation")
    saved_w = None if saved is None else (saved.get("ttt_intermediate_size") or saved.get("intermediate_size"))
    narrow = mc.memory == "ttt" and saved_w is not None and saved_w != mc.prime_intermediate_size
    if narrow and saved_w < mc.prime_intermediate_size:
        raise ValueError(f"checkpoint fast weight ({saved_w}) narrower than the model's ({mc.prime_intermediate_size})")
    held: Dict[str, np.ndarray] = {}
    for (name, (shape, _)), arr in zip(saved_spec.items(), NS.read_records(os.path.join(d, "model.eqx"))):
        if tuple(arr.shape) != tuple(shape):
            raise ValueError(f"checkpoint {d}: {name} has shape {arr.shape}, its config says {shape}")
        if name not in engine.spec:
            continue
        arr = arr.astype(np.float32) if np.issubdtype(arr.dtype, np.floating) else arr
        if narrow and name.startswith("fast_weight."):
            held[name] = arr
            if len(held) == 3:
                g, u, dn = prune_fast_weight(held["fast_weight.gate.weight"], held["fast_weight.up.weight"],
                                             held["fast_weight.down.weight"], mc.prime_intermediate_size)
                for n2, a2 in (("fast_weight.gate.weight", g), ("fast_weight.up.weight", u), ("fast_weight.down.weight", dn)):
                    engine.store.load_full(n2, torch.from_numpy(np.ascontiguousarray(a2)))
                log(f"[ttt] checkpoint {d}: fast weight narrowed {saved_w} -> {mc.prime_intermediate_size} hidden units per "
                    f"layer (magnitude pruning)")
            continue
        engine.store.load_full(name, torch.from_numpy(np.ascontiguousarray(arr)))


def load_opt(d: str, engine) -> None:
    """Optimiser state into the engine's shards (same model structure required).  The file holds whole tensors (``save``
    re-assembles tensor-parallel slices), so under tensor parallelism every moment is cut to this rank's slice first, exactly
    as ``ParamStore.load_full`` cuts the weights."""
    from ..models.params import tp_slice
    st, opt = engine.store, engine.opt
    names = list(st.names())
    it = NS.read_records(os.path.join(d, "opt.eqx"))
    count = int(next(it))
    for buf in (opt.m, opt.v):
        for name in names:
            arr = next(it)
            space, off, n, shape = st.slots[name]
            full = torch.from_numpy(np.ascontiguousarray(arr.astype(np.float32)))
            if st.tp_layout.get(name) is not None and tuple(full.shape) != tuple(shape):
                full = tp_slice(name, full, engine.mesh.tp, engine.mesh.tp_index)
            v = full.reshape(-1)
            if v.numel() != n:
                raise ValueError(f"checkpoint {d}: optimiser leaf of {name} has {v.numel()} elements, this rank stores {n}")
            lo, hi = st.shard_range(space)
            a, b = max(off, lo), min(off + n, hi)
            if a < b:
                st.master_part(space, buf)[a - lo:b - lo].copy_(v[a - off:b - off])
    sched_count = int(next(it))
    opt.count = count
    assert sched_count == count, (sched_count, count)
