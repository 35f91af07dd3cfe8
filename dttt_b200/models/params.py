"""The parameter tree: names, shapes, order, initialisation and the per-step compute copies.

The on-disk form of a model is the reference's: one array per leaf of its ``Model`` pytree, every
per-layer parameter stacked on a leading layer axis, in dataclass-field order
(``src/ttt/model.py:448-468`` for the model, ``:262-266`` block, ``:190-196`` attention, ``:157-159``
MLP, ``src/ttt/gdn.py:57-66`` GDN).  ``param_spec`` reproduces that order and those shapes, which is
what makes checkpoints interchangeable (``dttt_b200.ckpt``).  Names are the pytree paths joined by
dots, e.g. ``prefix.attn.q.weight [L-S, H, nh*d]``.

In memory the parameters live in ``parallel.store.ParamStore`` (sharded f32 masters, full compute
copies, full f32 gradient buffers); ``is_small`` says which parameters are used in f32 (norm weights,
biases, gates, scalars) rather than through a compute-dtype copy.
"""
from __future__ import annotations

import math
import re
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch

from ..schema import ModelConfig
from ..utils import rng as trng


def _block_spec(prefix: str, n: int, cfg: ModelConfig) -> List[Tuple[str, Tuple[int, ...], str]]:
    H, I = cfg.hidden_size, cfg.intermediate_size
    nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    out = [(f"{prefix}.attn_norm.weight", (n, H), "ones")]
    for nm, width in (("q", nh * d), ("k", nkv * d), ("v", nkv * d)):
        out.append((f"{prefix}.attn.{nm}.weight", (n, H, width), "normal"))
        if cfg.attention_bias:
            out.append((f"{prefix}.attn.{nm}.bias", (n, width), "zeros"))
    out.append((f"{prefix}.attn.o.weight", (n, nh * d, H), "normal"))
    if cfg.qk_norm:
        out.append((f"{prefix}.attn.q_norm.weight", (n, d), "ones"))
        out.append((f"{prefix}.attn.k_norm.weight", (n, d), "ones"))
    out.append((f"{prefix}.mlp_norm.weight", (n, H), "ones"))
    out.append((f"{prefix}.mlp.gate.weight", (n, H, I), "normal"))
    out.append((f"{prefix}.mlp.up.weight", (n, H, I), "normal"))
    out.append((f"{prefix}.mlp.down.weight", (n, I, H), "normal"))
    return out


_TP_COL = re.compile(r"^(prefix|suffix)\.(attn\.(q|k|v)|mlp\.(gate|up))\.(weight|bias)$")
_TP_ROW = re.compile(r"^(prefix|suffix)\.(attn\.o|mlp\.down)\.weight$")


def tp_layout(name: str) -> Optional[Tuple[str, int]]:
    """How a parameter is split over a tensor-parallel group: ``("col", axis)`` for the output features of the Q / K / V and
    MLP gate / up projections (whole heads per rank), ``("row", axis)`` for the input features of the attention-out and MLP
    down projections, ``None`` for everything that stays whole on every rank (norms, embedding, the fast-weight template:
    the fast-weight MLP runs per sequence and sequences, not its features, are divided over the group)."""
    if _TP_COL.match(name):
        return "col", (1 if name.endswith("bias") else 2)
    if _TP_ROW.match(name):
        return "row", 1
    return None


def tp_slice(name: str, t: torch.Tensor, tp: int, index: int) -> torch.Tensor:
    lay = tp_layout(name)
    if tp == 1 or lay is None:
        return t
    n = t.shape[lay[1]] // tp
    return t.narrow(lay[1], index * n, n).contiguous()


def param_spec(cfg: ModelConfig, tp: int = 1) -> "OrderedDict[str, Tuple[Tuple[int, ...], str]]":
    """Ordered ``name -> (shape, init kind)``; the order is the checkpoint's leaf order.  ``tp > 1``: the shapes one rank
    of a tensor-parallel group holds (``tp_layout``)."""
    if tp > 1:
        if cfg.num_key_value_heads % tp or cfg.intermediate_size % tp:
            raise ValueError(f"tensor parallel {tp}: needs kv heads and MLP width divisible by it")
        out = OrderedDict()
        for n, (shape, kind) in param_spec(cfg).items():
            lay = tp_layout(n)
            if lay is not None:
                shape = tuple(d // tp if a == lay[1] else d for a, d in enumerate(shape))
            out[n] = (shape, kind)
        return out
    H, V = cfg.hidden_size, cfg.vocab_size
    S, F, Ip = cfg.suffix_len, cfg.fast_len, cfg.prime_intermediate_size
    spec: List[Tuple[str, Tuple[int, ...], str]] = [("embed", (V, H), "normal")]
    if cfg.prefix_len:
        spec += _block_spec("prefix", cfg.prefix_len, cfg)
    spec += _block_spec("suffix", S, cfg)
    if cfg.memory == "gdn":
        nh, dk = cfg.gdn_heads, cfg.gdn_head_dim
        spec += [("mem_norm.weight", (F, H), "ones"),
                 ("gdn.q.weight", (F, H, nh * dk), "normal"), ("gdn.k.weight", (F, H, nh * dk), "normal"),
                 ("gdn.v.weight", (F, H, nh * dk), "normal"),
                 ("gdn.beta.weight", (F, H, nh), "normal"), ("gdn.beta.bias", (F, nh), "zeros"),
                 ("gdn.dt.weight", (F, H, nh), "normal"),
                 ("gdn.dt_bias", (F, nh), "gdn_dt"), ("gdn.A_log", (F, nh), "gdn_A"),
                 ("gdn.gate.weight", (F, H, nh * dk), "normal"), ("gdn.o_norm_w", (F, dk), "ones"),
                 ("gdn.o.weight", (F, nh * dk, H), "normal")]
        if cfg.gdn_conv:
            spec.append(("gdn.conv.weight", (F, 3 * nh * dk, cfg.gdn_conv), "conv"))
    else:
        spec += [("prime_norm.weight", (F, H), "ones"), ("prime_post_norm.weight", (F, H), "ones"),
                 ("fast_weight.gate.weight", (F, H, Ip), "normal"), ("fast_weight.up.weight", (F, H, Ip), "normal"),
                 ("fast_weight.down.weight", (F, Ip, H), "normal")]
    if cfg.inner_lr_gate:
        spec += [("inner_gate.weight", (F, H + 2, 1), "zeros"), ("inner_gate.bias", (F, 1), "zeros")]
    if cfg.inner_token_gate:
        spec += [("inner_token_gate.weight", (H, 1), "zeros"), ("inner_token_gate.bias", (1,), "zeros")]
    if cfg.inner_decay > 0:
        spec.append(("inner_decay_logit", (F,), "decay_logit"))
    if cfg.inner_optimizer:
        spec += [("inner_precond.0.gate.weight", (F, H), "zeros"), ("inner_precond.0.up.weight", (F, H), "zeros"),
                 ("inner_precond.0.down.weight", (F, Ip), "zeros"),
                 ("inner_precond.1.gate.weight", (F, Ip), "zeros"), ("inner_precond.1.up.weight", (F, Ip), "zeros"),
                 ("inner_precond.1.down.weight", (F, H), "zeros"),
                 ("inner_step_log", (F,), "zeros"), ("inner_temp_log", (), "zeros")]
    if cfg.inner_feat_head:
        spec.append(("inner_feat_head.weight", (H, H), "normal"))
    if cfg.mtp_head:
        spec.append(("mtp_head.weight", (H, H), "normal"))
    if cfg.inner_kvb_head:
        spec.append(("inner_kvb_value.weight", (F, H, H), "normal"))
    spec.append(("final_norm.weight", (H,), "ones"))
    if not cfg.tie_word_embeddings:
        spec.append(("lm_head", (V, H), "normal"))
    return OrderedDict((n, (s, k)) for n, s, k in spec)


def count_params(cfg: ModelConfig) -> int:
    return sum(math.prod(s) if s else 1 for s, _ in param_spec(cfg).values())


def init_params(cfg: ModelConfig, seed: int, device="cpu") -> "OrderedDict[str, torch.Tensor]":
    """All parameters at once (small models, tests); see ``iter_init``."""
    return OrderedDict(iter_init(cfg, seed, device))


def iter_init(cfg: ModelConfig, seed: int, device="cpu", tp: int = 1, tp_index: int = 0):
    """Yield ``(name, f32 tensor)`` in checkpoint order, one parameter at a time.  Every leaf draws from its own counter-based key (the seed folded with
    the leaf's index, then with the layer index for stacked leaves), so the values do not depend on the
    device, the process count or how the tree is later sharded.  Normal leaves have std
    ``initializer_range`` (reference model.py:137-148), norm weights are 1, gates / biases 0, the GDN
    decay is initialised long (reference gdn.py:74-88)."""
    # keys are derived on the host (a few integers each); only the bulk draws run on `device`, where a GPU uses the
    # counter-RNG kernel (same bits as the host statement)
    base = trng.key(seed)
    on = lambda key: key.to(device)
    for idx, (name, (shape, kind)) in enumerate(param_spec(cfg).items()):
        k = trng.fold_in(base, idx + 1)
        if kind == "ones":
            t = torch.ones(shape)
        elif kind == "zeros":
            t = torch.zeros(shape)
        elif kind == "normal":
            if len(shape) >= 3:        # stacked: one key per layer, so slicing the stack leaves values unchanged
                t = torch.stack([trng.normal(on(trng.fold_in(k, l)), shape[1:]) for l in range(shape[0])]) * cfg.initializer_range
            else:
                t = trng.normal(on(k), shape) * cfg.initializer_range
        elif kind == "gdn_dt":
            u = trng.uniform(k, shape, math.log(1e-4), math.log(1e-2))
            dt0 = torch.exp(u)
            t = dt0 + torch.log(-torch.expm1(-dt0))            # inverse softplus
        elif kind == "gdn_A":
            t = torch.log(trng.uniform(k, shape, 1.0, 4.0))
        elif kind == "decay_logit":
            p = cfg.inner_decay / 0.1
            t = torch.full(shape, math.log(p / (1 - p)))
        elif kind == "conv":
            t = torch.zeros(shape)
            t[..., -1] = 1.0                                     # identity filter: the option starts as "no conv"
        else:
            raise ValueError(kind)
        yield name, tp_slice(name, t, tp, tp_index).to(device=device, dtype=torch.float32).contiguous()


# parameters that stay f32 leaves in the compute view (everything that is not a matrix operand of a GEMM)
_SMALL = re.compile(r"norm|bias|inner_gate|inner_token_gate|inner_decay_logit|inner_precond|inner_step_log|"
                    r"inner_temp_log|dt_bias|A_log|o_norm_w|conv")


def is_small(name: str) -> bool:
    return bool(_SMALL.search(name))
