"""Block masked-diffusion decoding with test-time training:
``python -m dttt_b200.generate --ckpt <step dir> --prompt "..."``.

Generation proceeds in blocks of ``chunk_size`` tokens, left to right (reference ``src/ttt/generate.py:1-21``):
a block starts masked (prompt positions stay clean) and is unmasked over ``steps`` iterations, each running
the model on the current block against the clean K/V windows of the previous blocks and the live fast
weight, sampling every masked slot and committing the most confident share; a finished block is then treated
as a clean chunk in training: its K/V shift into the windows (forward B) and the write updates the fast
weight (forward C) with the same ``inner_update`` / ``write_chunk`` the training scan calls, so training and
decoding cannot drift apart.  State per sequence: the clean K/V window of every layer and the f32 fast weight.

Sampler options (``DecodeOpts``): confidence or random commit order, Gumbel sampling, probability threshold
(parallel decoding), presence penalty, a re-masking corrector loop, sub-block (semi-autoregressive) filling,
and the priority measure (log-probability, top-2 margin or negative entropy) - reference ``generate.py:196-355``.
With the outer shift slot ``i`` predicts token ``i+1`` and the first token of a block comes from the previous
block's tail logit.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from .ckpt import store as ckpt
from .engine import Engine
from .models.blocks import Net
from .ops import attention as A
from .ops import functional as Fn
from .schema import ModelConfig, TrainConfig
from .ttt import inner as IN
from .ttt import objective as OBJ
from .utils import rng


@dataclass
class DecodeState:
    kv: List[Tuple[torch.Tensor, torch.Tensor]]      # per layer (prefix then suffix): clean K/V windows [B, W*C, nkv, d]
    W: IN.FastW                                      # live fast weight, f32, per fast layer (gate, up, down) [B, ...]
    chunk: int                                       # index of the next block


def init_state(net: Net, batch: int = 1) -> DecodeState:
    cfg = net.cfg
    if cfg.memory != "ttt":
        raise NotImplementedError("decoding with the gdn memory is not implemented (training / evaluation only)")
    dev = net.p("final_norm.weight").device
    z = lambda: torch.zeros(batch, cfg.window_chunks * cfg.chunk_size, cfg.num_key_value_heads, cfg.head_dim, dtype=net.dtype, device=dev)
    W = [tuple(t.detach().clone() for t in w) for w in net.template_fast(batch)]
    return DecodeState([(z(), z()) for _ in range(cfg.num_hidden_layers)], W, 0)


@torch.no_grad()
def block_forward(net: Net, ids: torch.Tensor, pos: torch.Tensor, state: DecodeState, pos_q=None, own: str = "full", own_mask=None,
                  return_prime: bool = False, own_kv=None):
    """One block ``ids [B, C]`` through all layers against the state's windows: ``(logits [B, C, V] f32, the
    suffix input [B, C, H], own K/V per layer, extras)``."""
    cfg = net.cfg
    C = cfg.chunk_size
    if cfg.read_block and own_kv is None and own_mask is None and own == "full":
        raise ValueError("read_block: the read needs the block's clean K/V (own_kv); the clean pass is clean_forward")
    if own_kv is not None and own_mask is None:
        own_mask = A.read_mask_matrix(C, cfg.read_block, ids.device)
    nv = A.valid_window_chunks(state.chunk, cfg.window_chunks, cfg.reach)
    Lp = cfg.prefix_len
    h = net.embed_tokens(ids)
    kv_own = []
    for l in range(Lp):
        h, kvo, _ = net.block("prefix", l, h, pos, state.kv[l], nv, pos_q=pos_q, own=own, own_mask=own_mask,
                              own_kv=None if own_kv is None else own_kv[l])
        kv_own.append(kvo)
    h_in = h
    Wc = IN.cast_fast(state.W, net.dtype)
    hn, kvs, extra = net.suffix_forward(h, pos, state.kv[Lp:], Wc, nv, pos_q=pos_q, own=own, own_mask=own_mask,
                                        return_prime=return_prime, own_kv=None if own_kv is None else own_kv[Lp:])
    return net.logits(hn).float(), h_in, kv_own + list(kvs), extra


def clean_forward(net: Net, ids, pos, state, return_prime: bool = False):
    rb = net.cfg.read_block
    return block_forward(net, ids, pos, state, own=f"block:{rb}" if rb else "full", return_prime=return_prime)


def block_tail(net: Net, ids, pos, state) -> torch.Tensor:
    """``[B, V]``: the logit the last slot of the complete block gives the next block's first token (outer shift)."""
    own = clean_forward(net, ids, pos, state)[2] if net.cfg.read_block else None
    return block_forward(net, ids, pos, state, pos_q=pos + 1, own_kv=own)[0][:, -1]


def commit_block(net: Net, clean_ids, pos, state: DecodeState, key, inner_lr: float, inner_clip: float, inner_mask_ratio: float,
                 fused_ce_block: int = 8192, inner_views: int = 1, inner_mask_span: float = 0.0, inner_update_rule: str = "sgd",
                 inner_mask=None, inner_task: str = "mask", inner_perm=None, inner_context_frac: float = 0.5,
                 wc: IN.WriteConfig = IN.WriteConfig()) -> DecodeState:
    """A finished block becomes context: forward B shifts its K/V into the windows, forward C writes the fast weight."""
    cfg = net.cfg
    C, Lp = cfg.chunk_size, cfg.prefix_len
    B = clean_ids.shape[0]
    nv = A.valid_window_chunks(state.chunk, cfg.window_chunks, cfg.reach)
    clean_values = (not wc.plain) and wc.kvb_weight > 0 and wc.kvb_value == "clean"
    _, h_clean, kv_own, extra = clean_forward(net, clean_ids, pos, state, return_prime=clean_values)
    kv_next = [(torch.cat([ck[:, C:], ok], 1), torch.cat([cv[:, C:], ov], 1)) if ck.shape[1] else (ck, cv)
               for (ck, cv), (ok, ov) in zip(state.kv, kv_own)]
    kv_suf = state.kv[Lp:]
    pos_in, pos_q, own, targets = pos, None, "full", clean_ids
    if inner_task == "mask":
        if inner_mask is not None:
            x_inner = torch.where(inner_mask, torch.full_like(clean_ids, cfg.mask_token_id), clean_ids)
        else:
            keys = key if key.dim() == 2 else key.unsqueeze(0).expand(B, 2)
            x_inner, inner_mask = OBJ.inner_masks(keys, clean_ids, inner_mask_ratio, (inner_mask_ratio, inner_mask_ratio),
                                                  cfg.mask_token_id, cfg.pad_token_id, inner_views, inner_mask_span)
        if inner_views == 1:
            h_inner = block_forward(net, x_inner, pos, state)[1]
        else:
            h_inner = torch.stack([block_forward(net, x_inner[:, v], pos, state)[1] for v in range(inner_views)], 1)
        weights = inner_mask
    else:
        if inner_task == "causal":
            perm, K, own = torch.arange(C, device=clean_ids.device)[None].expand(B, C), 0, "causal"
        else:
            perm, K = inner_perm - pos[:, :1], int(round(inner_context_frac * C))
            own = f"split:{K}"
        x_inner, pos_in = torch.gather(clean_ids, 1, perm), torch.gather(pos, 1, perm)
        targets = torch.cat([x_inner[:, 1:], x_inner[:, -1:]], 1)
        pos_q = torch.cat([pos_in[:, 1:], pos_in[:, -1:]], 1)
        slot = torch.arange(C, device=clean_ids.device)
        weights = ((slot >= max(K - 1, 0)) & (slot <= C - 2))[None].expand(B, C)
        h_inner = block_forward(net, x_inner, pos_in, state, pos_q=pos_q, own=own)[1]
    if not wc.plain:
        if inner_task != "causal":
            raise ValueError("the write schemes (WriteConfig) are defined for the causal write")
        W_next, _ = IN.write_chunk(state.W, net, h_inner, targets, weights, kv_suf, pos_in, nv, inner_lr, inner_clip, fused_ce_block,
                                   inner_update_rule, h_clean, pos_q, own, wc, create_graph=False, W0=net.template_fast(B),
                                   kvb_src=extra[0] if clean_values else None)
    else:
        W_next, _ = IN.inner_update(state.W, net, h_inner, targets, weights, kv_suf, pos_in, nv, inner_lr, inner_clip, fused_ce_block,
                                    inner_update_rule, create_graph=False, h_clean=h_clean, pos_q=pos_q, own=own)
    W_next = [tuple(t.detach() for t in w) for w in W_next]
    return DecodeState(kv_next, W_next, state.chunk + 1)


@dataclass(frozen=True)
class DecodeOpts:
    order: str = "confidence"         # confidence | random
    gumbel_high: bool = False         # kept for interface parity: sampling here always uses full-resolution Gumbel noise
    threshold: float = 0.0
    presence_penalty: float = 0.0
    remask_loop: int = 0
    remask_k: int = 16
    subblock: int = 0
    priority: str = "logp"            # logp | margin | entropy


# ---- confidence unmasking of one block (reference generate.py:227-355: LLaDA-style, with the options of ``DecodeOpts``)
def _rank_of(priority: torch.Tensor) -> torch.Tensor:
    """Position of every slot when its row is sorted by descending priority (earlier slot first among equals)."""
    return torch.argsort(torch.argsort(-priority, dim=-1, stable=True), dim=-1)


def _gumbel(key: torch.Tensor, shape, device) -> torch.Tensor:
    u = rng.uniform(key.to("cpu"), shape).to(device).clamp_(1e-20, 1 - 1e-7)
    return -torch.log(-torch.log(u))


# how sure a slot's proposal is, from the log-probabilities over the vocabulary and the log-probability of the proposed token
_PRIORITY = {
    "logp": lambda logp, chosen: chosen,
    "margin": lambda logp, chosen: (lambda top: top[..., 0].exp() - top[..., 1].exp())(logp.topk(2, -1).values),
    "entropy": lambda logp, chosen: (logp.exp() * torch.where(torch.isfinite(logp), logp, torch.zeros_like(logp))).sum(-1),
}


class _KeyChain:
    """One fresh key per request: ``(carry, out) = split(carry)``."""

    def __init__(self, key: torch.Tensor):
        self.carry = key

    def take(self) -> torch.Tensor:
        self.carry, out = rng.split(self.carry, 2).unbind(0)
        return out


class BlockUnmasker:
    """The state of one block while it is being decoded: the tokens committed so far, the log-probability each was
    committed with, and the read-only context (positions, caches, previous block's tail logit)."""

    def __init__(self, net: Net, ids, known, pos, state: DecodeState, key, temperature: float, outer_shift: bool, prev_tail_logit,
                 opts: DecodeOpts):
        self.net, self.pos, self.state, self.opts = net, pos, state, opts
        self.temperature, self.outer_shift, self.prev_tail = temperature, outer_shift, prev_tail_logit
        self.ids, self.known, self.given = ids, known, known.clone()
        self.B, self.C = ids.shape
        self.dev, self.mask_id, self.V = ids.device, net.cfg.mask_token_id, net.cfg.vocab_size
        self.pos_q = pos + 1 if outer_shift else None
        self.blank = torch.full_like(ids, self.mask_id)
        self.committed_logp = torch.zeros(self.B, self.C, device=self.dev)
        self.keys = _KeyChain(key)

    def masked_input(self, visible: torch.Tensor) -> torch.Tensor:
        return torch.where(visible, self.ids, self.blank)

    def propose(self, visible: torch.Tensor, key: torch.Tensor, own_kv=None):
        """A token for every slot given the ``visible`` ones: ``(tokens, their log-probability, their priority)``."""
        o = self.opts
        x = self.masked_input(visible)
        logits = block_forward(self.net, x, self.pos, self.state, pos_q=self.pos_q, own_kv=own_kv)[0]
        logits[..., self.mask_id] = float("-inf")
        if self.outer_shift:                                        # slot i is predicted at slot i - 1; slot 0 by the previous block's tail
            lead = self.prev_tail.clone() if self.prev_tail is not None else torch.zeros(self.B, self.V, device=self.dev)
            lead[..., self.mask_id] = float("-inf")
            logits = torch.cat([lead[:, None], logits[:, :-1]], 1)
        if o.presence_penalty > 0:
            seen = torch.zeros(self.B, self.V, device=self.dev).scatter_(1, x, 1.0)
            seen[:, self.mask_id] = 0
            logits = logits - o.presence_penalty * seen[:, None]
        logp = torch.log_softmax(logits, -1)
        if self.temperature > 0:
            tokens = (logits / self.temperature + _gumbel(key, (self.B, self.C, self.V), self.dev)).argmax(-1)
        else:
            tokens = logits.argmax(-1)
        chosen = logp.gather(-1, tokens[..., None])[..., 0]
        return tokens, chosen, _PRIORITY[o.priority](logp, chosen)

    def pick(self, priority: torch.Tensor, key: torch.Tensor, quota: torch.Tensor, allowed=None) -> torch.Tensor:
        """The ``quota [B]`` open (and allowed) slots of highest priority; with ``order = random`` the priority is a draw."""
        if self.opts.order == "random":
            priority = rng.uniform(rng.fold_in(key, 1).to("cpu"), (self.B, self.C)).to(self.dev)
        shut = self.known if allowed is None else (self.known | ~allowed)
        priority = torch.where(shut, torch.full_like(priority, float("-inf")), priority)
        return (_rank_of(priority) < quota[:, None]) & ~shut

    def commit(self, where: torch.Tensor, tokens: torch.Tensor, logp: torch.Tensor) -> None:
        self.ids = torch.where(where, tokens, self.ids)
        self.committed_logp = torch.where(where, logp, self.committed_logp)
        self.known = self.known | where

    # ---- schedules
    def sweep(self, n_steps: int, allowed=None, own_kv=None) -> None:
        """Fill the open (allowed) slots in ``n_steps`` rounds, an equal share of what is left per round."""
        for i in range(n_steps):
            key = self.keys.take()
            tokens, logp, priority = self.propose(self.known, key, own_kv)
            open_ = ~self.known if allowed is None else (~self.known & allowed)
            quota = torch.ceil(open_.sum(-1).float() / (n_steps - i)).long()
            self.commit(self.pick(priority, key, quota, allowed), tokens, logp)

    def until_confident(self, threshold: float) -> None:
        """Each round commits every slot whose proposal reaches ``threshold`` probability, and at least the best one."""
        one = torch.ones(self.B, dtype=torch.long, device=self.dev)
        rounds = 0
        while (~self.known).any() and rounds < self.C:
            key = self.keys.take()
            tokens, logp, priority = self.propose(self.known, key)
            sure = (logp >= float(np.log(threshold))) & ~self.known
            self.commit(sure | self.pick(priority, key, one), tokens, logp)
            rounds += 1

    def revise(self, rounds: int, k: int) -> None:
        """Re-predict, ``rounds`` times, the ``k`` generated slots that were committed least surely (Gumbel-perturbed)."""
        for _ in range(rounds):
            k_pick, k_draw = self.keys.take(), self.keys.take()
            doubt = torch.where(self.given, torch.full_like(self.committed_logp, float("-inf")),
                                -self.committed_logp + _gumbel(k_pick, (self.B, self.C), self.dev))
            again = (_rank_of(doubt) < k) & ~self.given
            tokens, logp, _ = self.propose(~again, k_draw)
            self.ids = torch.where(again, tokens, self.ids)
            self.committed_logp = torch.where(again, logp, self.committed_logp)


def _check_decode_opts(opts: DecodeOpts, C: int, read_block: int, outer_shift: bool) -> None:
    if opts.order not in ("confidence", "random") or opts.priority not in _PRIORITY:
        raise ValueError(f"DecodeOpts order {opts.order!r} / priority {opts.priority!r}")
    if opts.subblock < 0 or (opts.subblock and (C % opts.subblock or opts.threshold > 0)):
        raise ValueError(f"DecodeOpts.subblock {opts.subblock}: a divisor of the block size {C}, without threshold")
    if read_block and (opts.threshold > 0 or opts.remask_loop > 0 or opts.subblock not in (0, read_block) or not outer_shift):
        raise ValueError(f"read_block {read_block}: its groups are decoded in order, with the outer shift")


@torch.no_grad()
def decode_block(net: Net, ids, known, pos, state: DecodeState, key, steps: int, temperature: float = 0.0, outer_shift: bool = False,
                 prev_tail_logit=None, opts: DecodeOpts = DecodeOpts()):
    """Unmask one block: ``ids [B, C]`` carry the known tokens, ``known [B, C]`` marks them.  Returns ``(ids, tail logit)``."""
    cfg = net.cfg
    C, rb = cfg.chunk_size, cfg.read_block
    _check_decode_opts(opts, C, rb, outer_shift)
    work = BlockUnmasker(net, ids, known, pos, state, key, temperature, outer_shift, prev_tail_logit, opts)
    slot = torch.arange(C, device=ids.device)
    whole_rows = lambda m: m[None].expand(work.B, C)
    if opts.threshold > 0:
        work.until_confident(opts.threshold)
    elif rb:
        # group g holds the slots predicted from sub-block g of the clean stream (shifted by one); its own clean keys are refreshed first
        per_group = max(1, -(-steps * rb // C))
        for g in range(C // rb):
            members = ((slot >= g * rb + 1) & (slot <= (g + 1) * rb)) | ((slot == 0) & (g == 0))
            own = clean_forward(net, work.masked_input(work.known), pos, state)[2]
            work.sweep(per_group, whole_rows(members), own)
    elif opts.subblock:
        per_group = max(1, -(-steps * opts.subblock // C))
        for g in range(C // opts.subblock):
            work.sweep(per_group, whole_rows((slot // opts.subblock) == g))
    else:
        work.sweep(steps)
    work.revise(opts.remask_loop, opts.remask_k)
    tail = block_tail(net, work.ids, pos, state) if outer_shift else torch.zeros(work.B, cfg.vocab_size, device=ids.device)
    return work.ids, tail


@torch.no_grad()
def generate(net: Net, prompt: torch.Tensor, max_new_tokens: int, key: torch.Tensor, steps: int = 16, temperature: float = 0.0,
             inner_lr: float = 1.0, inner_clip: float = 1.0, inner_mask_ratio: float = 0.75, fused_ce_block: int = 8192,
             inner_views: int = 1, inner_mask_span: float = 0.0, inner_update_rule: str = "sgd", inner_mask_mode: str = "random",
             unigram=None, inner_target_frac: float = 0.5, inner_generic_floor: float = 0.1, inner_task: str = "mask",
             outer_shift: bool = False, wc: IN.WriteConfig = IN.WriteConfig(), opts: DecodeOpts = DecodeOpts()) -> torch.Tensor:
    """``prompt [P]`` -> ``[P + max_new_tokens]`` token ids.  Blocks inside the prompt are only committed; the block
    holding the prompt's end is decoded around its known tokens; later blocks are decoded from all-masked."""
    from .data.host_masks import inner_mask_rule, split_perm
    cfg = net.cfg
    C = cfg.chunk_size
    dev = net.p("final_norm.weight").device
    P = int(prompt.shape[0])
    total = P + max_new_tokens
    n_blocks = -(-total // C)
    ids_all = torch.cat([prompt.long().to(dev), torch.full((n_blocks * C - P,), cfg.mask_token_id, dtype=torch.long, device=dev)])
    known_all = torch.arange(n_blocks * C, device=dev) < P
    state = init_state(net, 1)
    out = []
    tail = torch.zeros(1, cfg.vocab_size, device=dev)
    for b in range(n_blocks):
        sl = slice(b * C, (b + 1) * C)
        pos = torch.arange(b * C, (b + 1) * C, device=dev)[None]
        ids, known = ids_all[sl][None], known_all[sl][None]
        ks = rng.split(key, 3)
        key, k_dec, k_inner = ks[0], ks[1], ks[2]
        if not bool(known.all()):
            ids, tail = decode_block(net, ids, known, pos, state, k_dec, steps, temperature, outer_shift, tail, opts)
        elif outer_shift:
            tail = block_tail(net, ids, pos, state)
        host_mask = host_perm = None
        prefix = np.concatenate([x.cpu().numpy() for x in out]) if out else None
        if inner_task == "split":
            host_perm = torch.as_tensor(split_perm(ids[0].cpu().numpy(), inner_mask_mode, C, cfg.eos_token_id, cfg.pad_token_id,
                                                   1.0 - inner_target_frac, unigram, inner_generic_floor, seed=b, prefix=prefix),
                                        dtype=torch.long, device=dev)[None] + b * C
        elif inner_mask_mode != "random":
            host_mask = torch.as_tensor(inner_mask_rule(ids[0].cpu().numpy(), inner_mask_mode, C, cfg.eos_token_id, cfg.pad_token_id,
                                                        unigram, inner_target_frac, inner_generic_floor, seed=b, prefix=prefix),
                                        device=dev)[None]
        state = commit_block(net, ids, pos, state, k_inner, inner_lr, inner_clip, inner_mask_ratio, fused_ce_block, inner_views,
                             inner_mask_span, inner_update_rule, host_mask, inner_task, host_perm, 1.0 - inner_target_frac, wc)
        out.append(ids[0])
    return torch.cat(out)[:total]


def load_model(ckpt_dir: str, model_config: Optional[str] = None, device=None, dtype: str = "bfloat16") -> Engine:
    """An inference engine (no optimiser state, no gradient buffers) holding the checkpoint's weights on one device."""
    if model_config is None and os.path.exists(os.path.join(ckpt_dir, "model_config.json")):
        model_config = os.path.join(ckpt_dir, "model_config.json")
    if model_config is None:
        model_config = "configs/1b_e2e"
        for p in (os.path.join(ckpt_dir, "train_config.json"), os.path.join(os.path.dirname(ckpt_dir), "train_config.json")):
            if os.path.exists(p):
                with open(p) as fh:
                    model_config = json.load(fh).get("model_config", model_config)
                break
    mc = ModelConfig.load(model_config)
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if device.type == "cpu":
        dtype = "float32"
    eng = Engine(mc, TrainConfig(compute_dtype=dtype), device=device, init=False, trainable=False)
    ckpt.load_weights(ckpt_dir, eng, log=lambda *a: None)
    return eng


def main(argv=None) -> None:
    import argparse
    pre = argparse.ArgumentParser(add_help=False)
    pre.add_argument("--ckpt", default=None)
    known, _ = pre.parse_known_args(argv)
    dflt = {}
    if known.ckpt:
        for p in (os.path.join(known.ckpt, "train_config.json"), os.path.join(os.path.dirname(known.ckpt), "train_config.json")):
            if os.path.exists(p):
                with open(p) as fh:
                    dflt = json.load(fh)
                break
    g = lambda k, d: dflt.get(k, d)
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.generate")
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--model_config", default=None)
    ap.add_argument("--tokenizer", default="", help="directory with tokenizer.json (default: the model config's directory)")
    ap.add_argument("--prompt", default="The history of the Roman Empire")
    ap.add_argument("--prompt_ids", default="", help="comma-separated token ids instead of text (no tokenizer needed)")
    ap.add_argument("--max_new_tokens", type=int, default=256)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--inner_lr", type=float, default=g("inner_lr", 1.0))
    ap.add_argument("--inner_clip", type=float, default=g("inner_clip", 1.0))
    ap.add_argument("--inner_mask_ratio", type=float, default=0.75)
    ap.add_argument("--inner_views", type=int, default=g("inner_views", 1))
    ap.add_argument("--inner_mask_span", type=float, default=0.0)
    ap.add_argument("--inner_update", default="sgd", choices=["sgd", "sign", "muon2"])
    ap.add_argument("--inner_mask_mode", default=g("inner_mask_mode", "random"), choices=["random", "rare", "docaware"])
    ap.add_argument("--inner_target_frac", type=float, default=g("inner_target_frac", 0.5))
    ap.add_argument("--inner_task", default=g("inner_task", "mask"), choices=["mask", "causal", "split"])
    ap.add_argument("--outer_shift", type=lambda s: s.lower() in ("1", "true", "yes"), default=g("outer_shift", False))
    for k, typ, d in (("inner_subchunks", int, 1), ("inner_subchunk_scale", float, 1.0), ("inner_surprise_gamma", float, 0.0),
                      ("inner_kvb_weight", float, 0.0), ("inner_kvb_value", str, "self"), ("inner_fast_frac", float, 0.0),
                      ("inner_fast_lr_scale", float, 1.0), ("inner_fast_decay", float, 0.0), ("inner_norm_alpha", float, 0.0),
                      ("inner_norm_cap", float, 1.0)):
        ap.add_argument(f"--{k}", type=typ, default=g(k, d))
    ap.add_argument("--order", default="confidence"); ap.add_argument("--threshold", type=float, default=0.0)
    ap.add_argument("--presence_penalty", type=float, default=0.0); ap.add_argument("--remask_loop", type=int, default=0)
    ap.add_argument("--remask_k", type=int, default=16); ap.add_argument("--subblock", type=int, default=0)
    ap.add_argument("--priority", default="logp")
    ap.add_argument("--unigram_path", default="bucket/data/tokens/unigram_llama3.i64")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    wc = IN.WriteConfig(subchunks=a.inner_subchunks, subchunk_scale=a.inner_subchunk_scale, surprise_gamma=a.inner_surprise_gamma,
                        kvb_weight=a.inner_kvb_weight, kvb_value=a.inner_kvb_value, fast_frac=a.inner_fast_frac,
                        fast_lr_scale=a.inner_fast_lr_scale, fast_decay=a.inner_fast_decay, norm_alpha=a.inner_norm_alpha,
                        norm_cap=a.inner_norm_cap)
    eng = load_model(a.ckpt, a.model_config)
    tok = None
    if a.prompt_ids:
        prompt = torch.tensor([int(x) for x in a.prompt_ids.split(",")])
    else:
        from transformers import PreTrainedTokenizerFast
        tdir = a.tokenizer or (a.model_config or g("model_config", "configs/1b_e2e"))
        tok = PreTrainedTokenizerFast.from_pretrained(tdir)
        prompt = torch.tensor(tok(a.prompt, add_special_tokens=False)["input_ids"])
    uni = np.fromfile(a.unigram_path, dtype=np.int64) if a.inner_mask_mode != "random" and os.path.exists(a.unigram_path) else None
    out = generate(eng.net(train=False), prompt, a.max_new_tokens, rng.key(a.seed), steps=a.steps, temperature=a.temperature,
                   inner_lr=a.inner_lr, inner_clip=a.inner_clip, inner_mask_ratio=a.inner_mask_ratio, inner_views=a.inner_views,
                   inner_mask_span=a.inner_mask_span, inner_update_rule=a.inner_update, inner_mask_mode=a.inner_mask_mode,
                   inner_target_frac=a.inner_target_frac, inner_task=a.inner_task, outer_shift=a.outer_shift, wc=wc, unigram=uni,
                   opts=DecodeOpts(a.order, False, a.threshold, a.presence_penalty, a.remask_loop, a.remask_k, a.subblock, a.priority))
    new = out[len(prompt):].tolist()
    print(tok.decode(new) if tok is not None else ",".join(map(str, new)))


if __name__ == "__main__":
    main()
