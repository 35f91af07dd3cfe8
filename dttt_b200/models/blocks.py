"""The transformer, written batch-first over explicit layer loops.

Shapes carry the batch: a chunk of hidden states is ``[B, C, H]``, a KV window ``[B, W*C, nkv, d]``,
the live fast weight of a layer ``[B, H, I]`` / ``[B, I, H]`` (one per sequence).  The reference states
the same model for one sequence and vmaps it (``src/ttt/model.py:1-33``); here the batch is folded
into the rows of every GEMM with shared weights, and the per-sequence fast-weight products are one
batched GEMM launch.

Layer semantics (``model.py:276-333``): attention residual, then the memory residual
``h += post_norm(W(pre_norm(h)))`` (fast weight) or the GDN state read, then the base SwiGLU MLP
residual.  The prefix layers run all chunks and all streams at once (``model.py:335-442``): a stream's
chunk ``c`` attends to the CLEAN stream's K/V of chunks ``[c-W, c)`` plus its own K/V of chunk ``c``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import functional as Fn
from ..ops import attention as A
from ..schema import ModelConfig

OUTER, CLEAN, INNER = 0, 1, 2      # stream indices of the prefix (inner views occupy INNER, INNER+1, ...)


def cast_like(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x if x.dtype == dtype else x.to(dtype)


class Net:
    """Stateless forward functions over a ``ComputeWeights`` view."""

    def __init__(self, cfg: ModelConfig, cw, tp_ctx=None):
        """``tp_ctx`` (``parallel.tp.TPContext``): the trunk's projections are tensor parallel.  Hidden states, fast weights and
        losses then cover this rank's ``B / tp`` sequences, while Q / K / V, the KV windows and the attention cover all ``B``
        sequences of the group for this rank's ``heads / tp`` heads (``parallel/tp.py``)."""
        self.cfg, self.cw = cfg, cw
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.dtype = cw.dtype
        self.tp = tp_ctx
        self.tp_size = 1 if tp_ctx is None else tp_ctx.size

    def group_rows(self, pos: torch.Tensor) -> torch.Tensor:
        """Positions of the ``B / tp`` local sequences -> positions for all ``B`` sequences of the tensor-parallel group.  The
        sequences of a group share their positions (``loss_fn`` refuses per-sequence position ids under tensor parallelism)."""
        if self.tp_size == 1:
            return pos
        return pos[:1].expand(pos.shape[0] * self.tp_size, *pos.shape[1:])

    # ---- parameter access
    def p(self, name: str, layer: Optional[int] = None) -> torch.Tensor:
        return self.cw.get(name, layer)

    def lm_weight(self) -> torch.Tensor:
        return self.p("embed") if self.cfg.tie_word_embeddings else self.p("lm_head")

    # ---- pieces
    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        """Embedding lookup whose gradient is a f32 scatter-add (reference model.py:534-542)."""
        from ..ops import embed as E
        return E.embedding(self.p("embed"), ids, self.dtype, self.cw.grad_buffer("embed") if self.cw.train else None)

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        w = self.lm_weight()
        return Fn.mm(h.reshape(-1, h.shape[-1]), cast_like(w, h.dtype), False, True, out_dtype=torch.float32) \
            .view(*h.shape[:-1], -1)

    def norm(self, name: str, layer: Optional[int], x: torch.Tensor) -> torch.Tensor:
        return Fn.rms_norm(x, self.p(name, layer), self.cfg.rms_norm_eps)

    def qkv(self, stack: str, l: int, x: torch.Tensor, pos: torch.Tensor, pos_q: Optional[torch.Tensor] = None):
        """``x [..., T, H]``, ``pos [..., T]`` -> ``q [..., T, nh, d]``, ``k, v [..., T, nkv, d]`` (RoPE applied;
        ``pos_q``: query positions when they differ from the keys', reference model.py:219-233)."""
        cfg = self.cfg
        nh, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        b = (lambda n: self.p(f"{stack}.attn.{n}.bias", l)) if cfg.attention_bias else (lambda n: None)
        q = Fn.linear(x, self.p(f"{stack}.attn.q.weight", l), b("q")).unflatten(-1, (-1, d))       # heads / tp under tensor parallelism
        k = Fn.linear(x, self.p(f"{stack}.attn.k.weight", l), b("k")).unflatten(-1, (-1, d))
        v = Fn.linear(x, self.p(f"{stack}.attn.v.weight", l), b("v")).unflatten(-1, (-1, d))
        pos = self.group_rows(pos)
        pos_q = None if pos_q is None else self.group_rows(pos_q)
        if cfg.qk_norm:
            q = Fn.rms_norm(q, self.p(f"{stack}.attn.q_norm.weight", l), cfg.rms_norm_eps)
            k = Fn.rms_norm(k, self.p(f"{stack}.attn.k_norm.weight", l), cfg.rms_norm_eps)
        rope = lambda t, p_: Fn.rope(t, p_, d, cfg.rope_theta, cfg.rope_scaling)
        return rope(q, pos if pos_q is None else pos_q), rope(k, pos), v

    def mlp(self, stack: str, l: int, x: torch.Tensor) -> torch.Tensor:
        g = Fn.linear(x, self.p(f"{stack}.mlp.gate.weight", l))
        u = Fn.linear(x, self.p(f"{stack}.mlp.up.weight", l))
        return Fn.linear(Fn.glu(g, u, self.cfg.hidden_act), self.p(f"{stack}.mlp.down.weight", l))

    def fast_mlp(self, W: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], x: torch.Tensor,
                 return_hidden: bool = False):
        """Per-sequence SwiGLU: ``W = (gate [B,H,I], up [B,H,I], down [B,I,H])`` (or unbatched ``[H,I]``)."""
        g, u = Fn.linear(x, W[0]), Fn.linear(x, W[1])
        a = Fn.glu(g, u, self.cfg.hidden_act)
        y = Fn.linear(a, W[2])
        return (y, a) if return_hidden else y

    # ---- one chunk through one layer (suffix; reference Block.__call__)
    def block(self, stack: str, l: int, h: torch.Tensor, pos: torch.Tensor, kv_prev: Tuple[torch.Tensor, torch.Tensor],
              n_valid: int, *, prime=None, memory=None, update_memory: bool = False, inner: bool = False,
              pos_q: Optional[torch.Tensor] = None, own: str = "full", own_mask: Optional[torch.Tensor] = None,
              own_kv=None, return_prime: bool = False, attention: bool = True):
        """``h [B, C, H]``, ``pos [B, C]``, ``kv_prev = (k, v) [B, W*C, nkv, d]`` of which the newest ``n_valid``
        chunks are visible.  ``prime = (f, W)``: fast-weight layer index ``f`` and its live weights;
        ``memory = (f, gdn, S)``: GDN layer index, module and state.  Returns ``(h, (k, v), extra)`` where
        ``extra`` is the updated GDN state, the fast weight's ``(x, p_out)`` or None."""
        cfg = self.cfg
        C = cfg.chunk_size
        extra = None
        if attention:
            q, k, v = self.qkv(stack, l, self.norm(f"{stack}.attn_norm.weight", l, h), pos, pos_q)
            a = A.attend_window(q, k, v, kv_prev[0], kv_prev[1], n_valid, C, self.scale, own=own, inner=inner,
                                own_mask=own_mask, extra_own=own_kv)
            h = h + Fn.linear(a.flatten(-2), self.p(f"{stack}.attn.o.weight", l))
        else:
            k = v = None
        if prime is not None:
            f, W = prime
            x_p = self.norm("prime_norm.weight", f, h)
            p_out = self.norm("prime_post_norm.weight", f, self.fast_mlp(W, x_p))
            h = h + p_out
            if return_prime:
                extra = (x_p, p_out)
        elif memory is not None:
            f, gdn, S = memory
            xm = self.norm("mem_norm.weight", f, h)
            h = h + gdn.read(self, f, xm, S)
            if update_memory:
                extra = gdn.update(self, f, xm, S)
        h = h + self.mlp(stack, l, self.norm(f"{stack}.mlp_norm.weight", l, h))
        return h, (k, v), extra

    # ---- the prefix: all chunks, all streams, one layer (reference Block.prefix_call)
    def prefix_layer(self, l: int, h: torch.Tensor, pos_k: torch.Tensor, pos_q: Optional[torch.Tensor], first_chunk: int,
                     kv_win: Optional[Tuple[torch.Tensor, torch.Tensor]], owns: Sequence[str], reach: Optional[int],
                     read_block: int = 0):
        """``h [B, S, T, H]`` (S streams), ``pos_k/pos_q [B, S, T]``; ``kv_win``: clean K/V of the ``W`` chunks before
        this segment ``[B, W*C, nkv, d]`` x2 (None at the sequence start); ``first_chunk``: global index of the
        segment's first chunk.  Returns ``(h, (k_tail, v_tail))`` with the clean K/V of the segment's last W chunks."""
        cfg = self.cfg
        B, S, T, H = h.shape
        C, Wn = cfg.chunk_size, cfg.window_chunks
        nc = T // C
        x = self.norm("prefix.attn_norm.weight", l, h)
        q, k, v = self.qkv("prefix", l, x, pos_k, pos_q)                       # [B, S, T, heads, d]
        if not read_block and A.segment_attention_ok(q, C, Wn, owns):
            # one launch for all chunks and streams; the clean windows are read in place (ops.attention._SegmentAttention)
            a_seg, k_tail, v_tail = A.segment_attention(q, k, v, kv_win, C, Wn, first_chunk, reach, owns, self.scale)
            h = h + Fn.linear(a_seg.flatten(-2), self.p("prefix.attn.o.weight", l))
            h = h + self.mlp("prefix", l, self.norm("prefix.mlp_norm.weight", l, h))
            return h, (k_tail, v_tail)
        kc, vc = k[:, CLEAN], v[:, CLEAN]
        k_prev, v_prev = (None, None) if kv_win is None else kv_win
        B = q.shape[0]                                                         # all sequences of the tensor-parallel group
        nv_of = [A.valid_window_chunks(first_chunk + c, Wn, reach) for c in range(nc)]
        groups: Dict[int, List[int]] = {}
        for c, nv in enumerate(nv_of):
            groups.setdefault(nv, []).append(c)
        # the clean KV windows of every run of chunks with the same number of visible window chunks, [B * run, nv * C, nkv, d]
        glist = [(nv, cs[0], len(cs)) for nv, cs in groups.items()]
        k_wins = dict(zip(groups, A.window_groups(kc, C, Wn, k_prev, glist)))
        v_wins = dict(zip(groups, A.window_groups(vc, C, Wn, v_prev, glist)))
        outs = []
        for s in range(S):
            qs = q[:, s].unflatten(1, (nc, C))                                  # [B, nc, C, nh, d]
            ks = k[:, s].unflatten(1, (nc, C))
            vs = v[:, s].unflatten(1, (nc, C))
            own, own_mask, extra = owns[s], None, None
            if read_block and s == OUTER:
                own, own_mask = "read", A.read_mask_matrix(C, read_block, q.device)
            elif read_block and s == CLEAN:
                own = f"block:{read_block}"
            a_s = [None] * nc
            for nv, cs in groups.items():
                sel = (lambda t, _a=cs[0], _b=cs[-1] + 1: t[:, _a:_b])        # chunks sharing a valid length are contiguous
                fl = lambda t: t.flatten(0, 1)
                if read_block and s == OUTER:
                    extra = (fl(sel(kc.unflatten(1, (nc, C)))), fl(sel(vc.unflatten(1, (nc, C)))))
                a = A.attend_window(fl(sel(qs)), fl(sel(ks)), fl(sel(vs)), k_wins[nv], v_wins[nv], nv, C,
                                    self.scale, own=own if own != "read" else "full", own_mask=own_mask, extra_own=extra)
                a = a.unflatten(0, (-1, len(cs)))
                for j, c in enumerate(cs):
                    a_s[c] = a[:, j]
            outs.append(torch.stack(a_s, dim=1).flatten(1, 2))                  # [B, T, nh, d]
        a_all = torch.stack(outs, dim=1).flatten(-2)                             # [B, S, T, nh*d]
        h = h + Fn.linear(a_all, self.p("prefix.attn.o.weight", l))
        h = h + self.mlp("prefix", l, self.norm("prefix.mlp_norm.weight", l, h))
        WC = Wn * C
        if WC == 0:
            tail = (kc[:, :0], vc[:, :0])
        elif T >= WC:
            tail = (kc[:, T - WC:], vc[:, T - WC:])
        else:
            pk = kc.new_zeros((B, WC - T) + tuple(kc.shape[2:])) if k_prev is None else k_prev[:, T:]
            pv = vc.new_zeros((B, WC - T) + tuple(vc.shape[2:])) if v_prev is None else v_prev[:, T:]
            tail = (torch.cat([pk, kc], 1), torch.cat([pv, vc], 1))
        return h, tail

    # ---- the suffix: one chunk through all suffix layers with the live memory (reference suffix_forward)
    def suffix_forward(self, h: torch.Tensor, pos: torch.Tensor, kv: Sequence[Tuple[torch.Tensor, torch.Tensor]], W,
                       n_valid: int, *, inner: bool = False, pos_q: Optional[torch.Tensor] = None, own: str = "full",
                       own_mask: Optional[torch.Tensor] = None, memory_state: Optional[torch.Tensor] = None,
                       update_memory: bool = False, return_prime: bool = False, own_kv=None):
        """``h [B, C, H]``; ``kv``: per suffix layer ``(k, v) [B, W*C, nkv, d]``; ``W``: per fast layer
        ``(gate, up, down)`` in the compute dtype (None with memory gdn); ``memory_state [B, S, nh, dv, dk]``.
        Returns ``(final_norm(h), kv_own, extra)``: ``kv_own`` per layer ``(k, v) [B, C, nkv, d]``; ``extra`` is the
        new GDN states ``[B, S, ...]`` (``update_memory``), ``(xs, p_outs)`` per fast layer (``return_prime``) or None."""
        cfg = self.cfg
        gdn = None
        if cfg.memory == "gdn":
            from .gdn import GDN
            gdn = GDN
        kv_own, xs, ps, states = [], [], [], []
        f = 0
        for i in range(cfg.suffix_len):
            okv = None if own_kv is None else own_kv[i]
            kw = dict(inner=inner, pos_q=pos_q, own=own, own_mask=own_mask, own_kv=okv)
            if gdn is not None:
                attn_here = not (cfg.gdn_alternate and i % 2 == 0)
                h, kvo, ex = self.block("suffix", i, h, pos, kv[i], n_valid, memory=(i, gdn, memory_state[:, i]),
                                        update_memory=update_memory, attention=attn_here, **kw)
                if update_memory:
                    states.append(ex)
                if not attn_here:
                    kvo = (kv[i][0][:, :h.shape[1]] * 0, kv[i][1][:, :h.shape[1]] * 0) if kv[i][0].shape[1] >= h.shape[1] \
                        else (kv[i][0].new_zeros(h.shape[0], h.shape[1], *kv[i][0].shape[2:]),) * 2
            elif cfg.fast_mask[i]:
                h, kvo, ex = self.block("suffix", i, h, pos, kv[i], n_valid, prime=(f, W[f]), return_prime=return_prime, **kw)
                if return_prime:
                    xs.append(ex[0]); ps.append(ex[1])
                f += 1
            else:
                h, kvo, _ = self.block("suffix", i, h, pos, kv[i], n_valid, **kw)
            kv_own.append(kvo)
        hn = self.norm("final_norm.weight", None, h)
        if update_memory:
            return hn, kv_own, torch.stack(states, dim=1)
        if return_prime:
            return hn, kv_own, (xs, ps)
        return hn, kv_own, None

    def suffix_forward_streams(self, h: torch.Tensor, pos: torch.Tensor, pos_q: Optional[torch.Tensor],
                               kv: Sequence[Tuple[torch.Tensor, torch.Tensor]], W, n_valid: int, owns: Sequence[str],
                               return_prime: bool = False):
        """Several streams of one chunk through the suffix in ONE pass: ``h [B, S, C, H]`` with stream ``CLEAN`` (index 1) the
        clean one, ``pos / pos_q [B, S, C]`` (key and query positions per stream), the same window ``kv`` and the same fast
        weights ``W`` for all of them, one own-chunk pattern per stream.  Equal to ``suffix_forward`` stream by stream (the
        read and the clean pass of a chunk step use the same memory when no row takes the self-prior), but every projection
        sees ``S`` times the rows, the fast-weight products ``S C`` rows per sequence, and on the GPU the attention of all
        streams is one launch (``ops.attention.segment_attention`` over a one-chunk segment).  Returns ``(final_norm(h)
        [B, S, C, H], kv_own of the clean stream per layer, (xs, p_outs) of the clean stream per fast layer or None)``.
        Not for the GDN memory or the sub-block read."""
        cfg = self.cfg
        B, S, C, H = h.shape
        Wn = cfg.window_chunks
        kv_own, xs, ps = [], [], []
        f = 0
        for i in range(cfg.suffix_len):
            q, k, v = self.qkv("suffix", i, self.norm("suffix.attn_norm.weight", i, h), pos, pos_q)      # [B, S, C, heads, d]
            kw, vw = kv[i]
            if kw.shape[1] == Wn * C and A.segment_attention_ok(q, C, Wn, owns):
                # a one-chunk segment whose window holds `n_valid` chunks: first = n_valid makes exactly those visible
                a, _, _ = A.segment_attention(q, k, v, (kw, vw) if Wn else None, C, Wn, n_valid, None, owns, self.scale)
            else:
                a = torch.stack([A.attend_window(q[:, s], k[:, s], v[:, s], kw, vw, n_valid, C, self.scale, own=owns[s])
                                 for s in range(S)], dim=1)
            h = h + Fn.linear(a.flatten(-2), self.p("suffix.attn.o.weight", i))
            if cfg.fast_mask[i]:
                x_p = self.norm("prime_norm.weight", f, h)
                p_out = self.norm("prime_post_norm.weight", f, self.fast_mlp(W[f], x_p.flatten(1, 2)).unflatten(1, (S, C)))
                h = h + p_out
                if return_prime:
                    xs.append(x_p[:, CLEAN]); ps.append(p_out[:, CLEAN])
                f += 1
            h = h + self.mlp("suffix", i, self.norm("suffix.mlp_norm.weight", i, h))
            kv_own.append((k[:, CLEAN], v[:, CLEAN]))
        hn = self.norm("final_norm.weight", None, h)
        return hn, kv_own, ((xs, ps) if return_prime else None)

    # ---- whole sequence with a FIXED memory (tests, evaluation tools; reference Model.hidden)
    def hidden(self, ids: torch.Tensor, pos: Optional[torch.Tensor] = None, W=None) -> torch.Tensor:
        """Final-normed hidden states ``[B, T, H]`` for clean ``ids [B, T]`` with the KV window applied and a fixed
        fast weight (``W`` batched, or the ``W_0`` template); the training path threads a per-chunk ``W`` instead."""
        cfg = self.cfg
        B, T = ids.shape
        C, Wn = cfg.chunk_size, cfg.window_chunks
        if T % C:
            raise ValueError(f"T={T} not a multiple of chunk_size={C}")
        if cfg.read_block:
            raise NotImplementedError("read_block: a fixed-memory forward of clean ids has no noisy read")
        nc = T // C
        pos = torch.arange(T, device=ids.device)[None].expand(B, T) if pos is None else pos
        h = self.embed_tokens(ids)
        for l in range(cfg.prefix_len):
            h, _ = self._single_stream_layer("prefix", l, h, pos, None)
        if cfg.memory != "gdn":
            if W is None:
                W = self.template_fast(B)
            W = [tuple(cast_like(t, self.dtype) for t in w) for w in W]
        f = 0
        for i in range(cfg.suffix_len):
            prime = None
            if cfg.memory != "gdn" and cfg.fast_mask[i]:
                prime = (f, W[f]); f += 1
            h, _ = self._single_stream_layer("suffix", i, h, pos, prime)
        return self.norm("final_norm.weight", None, h)

    def _single_stream_layer(self, stack: str, l: int, h: torch.Tensor, pos: torch.Tensor, prime):
        cfg = self.cfg
        B, T, H = h.shape
        C, Wn = cfg.chunk_size, cfg.window_chunks
        nc = T // C
        q, k, v = self.qkv(stack, l, self.norm(f"{stack}.attn_norm.weight", l, h), pos)
        k_win, v_win = A.window_gather(k, C, Wn), A.window_gather(v, C, Wn)
        outs = []
        for c in range(nc):
            nv = A.valid_window_chunks(c, Wn, cfg.reach)
            sl = slice(c * C, (c + 1) * C)
            outs.append(A.attend_window(q[:, sl], k[:, sl], v[:, sl], k_win[:, c], v_win[:, c], nv, C, self.scale))
        a = torch.cat(outs, dim=1).flatten(-2)
        h = h + Fn.linear(a, self.p(f"{stack}.attn.o.weight", l))
        if prime is not None:
            f, W = prime
            h = h + self.norm("prime_post_norm.weight", f, self.fast_mlp(W, self.norm("prime_norm.weight", f, h)))
        h = h + self.mlp(stack, l, self.norm(f"{stack}.mlp_norm.weight", l, h))
        return h, (k, v)

    def template_fast(self, B: int):
        """The ``W_0`` template broadcast to the batch, f32: the fast weight at the sequence start."""
        out = []
        for f in range(self.cfg.fast_len):
            out.append(tuple(self.p(f"fast_weight.{n}.weight", f).float().unsqueeze(0).expand(B, -1, -1)
                             for n in ("gate", "up", "down")))
        return out

    def forward_logits(self, ids: torch.Tensor, **kw) -> torch.Tensor:
        return self.logits(self.hidden(ids, **kw))
