"""Model and run configuration.

Field names, defaults and JSON form are those of the reference (``src/ttt/config.py:68-122`` for the
model, ``:229-377`` for a run) so that its ``configs/*/config.json`` and ``runs/*.json`` files load
here unchanged and a ``train_config.json`` / ``model_config.json`` written here loads there.  What this
package adds (tensor parallelism, the GDN short convolution, ...) lives in fields that are only
written to JSON when they differ from their default, which keeps saved files readable by the
reference as long as the additions are off.

Rules carried over: an unknown key is an error, not a warning (``config.py:32-42``); six retired
options still load when set to their "off" value (``:26-29``); a run config may name ``"base"`` files
that are read first and overridden key by key, keys starting with ``#`` are comments (``:49-65``).
"""
from __future__ import annotations

import dataclasses as dc
import json
import os
from typing import Any, Dict, Optional, Tuple

# option -> the value that meant "off" when the option still existed
RETIRED = {"inner_assoc_scale": 1.0, "inner_prior_units": "", "inner_prior_k": 0, "inner_prior_dims": 0,
           "inner_norm_whiten": False, "self_prior_delay": [0, 0]}


def _read_json(path: str) -> Dict[str, Any]:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as fh:
        return json.load(fh)


def _accept(cls, raw: Dict[str, Any]) -> Dict[str, Any]:
    names = {f.name for f in dc.fields(cls)}
    in_use = sorted(k for k in raw if k not in names and k in RETIRED and raw[k] != RETIRED[k])
    if in_use:
        raise ValueError(f"{cls.__name__}: removed options in use: " + ", ".join(f"{k}={raw[k]!r}" for k in in_use))
    kept = {k: v for k, v in raw.items() if k in names or k not in RETIRED}
    extra = sorted(set(kept) - names)
    if extra:
        raise ValueError(f"{cls.__name__}: unknown keys {extra}. Known: {sorted(names)}")
    return kept


def load_run_config(path: str, _chain: Tuple[str, ...] = ()) -> Dict[str, Any]:
    """Flatten a run configuration file and its ``base`` chain into one dict of ``TrainConfig`` fields."""
    path = os.path.abspath(path)
    if path in _chain:
        raise ValueError(f"run config {path}: 'base' cycle")
    with open(path) as fh:
        raw = json.load(fh)
    bases = raw.pop("base", [])
    merged: Dict[str, Any] = {}
    for rel in ([bases] if isinstance(bases, str) else bases):
        merged.update(load_run_config(os.path.join(os.path.dirname(path), rel), _chain + (path,)))
    merged.update({k: v for k, v in raw.items() if not k.startswith("#")})
    return _accept(TrainConfig, merged)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


@dc.dataclass(frozen=True)
class ModelConfig:
    # architecture (Hugging Face names)
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    hidden_act: str = "silu"
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    rope_scaling: Optional[Tuple[Tuple[str, Any], ...]] = None    # llama3 only; kept as sorted pairs, saved as a dict
    initializer_range: float = 0.02
    tie_word_embeddings: bool = True
    attention_bias: bool = False
    qk_norm: bool = True
    # test-time training
    suffix_len: int = 6                   # the top layers that run chunk by chunk
    suffix_plain_top: int = 0             # the top this-many suffix layers carry no fast weight
    fast_layers: Optional[Tuple[int, ...]] = None   # explicit fast-weight layers (absolute indices)
    ttt_intermediate_size: Optional[int] = None
    inner_lr_gate: bool = False
    inner_token_gate: bool = False
    inner_decay: float = 0.0
    inner_optimizer: bool = False
    inner_feat_head: bool = False
    mtp_head: bool = False
    inner_kvb_head: bool = False
    memory: str = "ttt"                   # ttt (fast-weight MLP) | gdn (Gated DeltaNet state)
    gdn_heads: int = 16
    gdn_head_dim: int = 128
    # chunk / window geometry
    chunk_size: int = 1024
    window_chunks: int = 7
    window_reach: int = -1
    read_block: int = 0
    # special tokens
    mask_token_id: int = 0
    pad_token_id: int = 0
    eos_token_id: int = 0
    bos_token_id: Optional[int] = None
    # --- additions of this package (omitted from JSON while at their defaults) ---
    gdn_conv: int = 0                     # > 0: causal depthwise short convolution of this width on the GDN q/k/v
    gdn_alternate: bool = False           # memory gdn: suffix layers alternate GDN-only and attention layers
    gdn_chunk: int = 64                   # block length of the chunked delta rule

    _ADDED = ("gdn_conv", "gdn_alternate", "gdn_chunk")

    def __post_init__(self):
        _need(self.num_attention_heads % self.num_key_value_heads == 0,
              "num_attention_heads must be a multiple of num_key_value_heads")
        _need(self.head_dim % 2 == 0, "head_dim must be even for RoPE")
        if self.rope_scaling is not None:
            rs = dict(self.rope_scaling)
            keys = {"rope_type", "factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"}
            _need(rs.get("rope_type") == "llama3" and set(rs) == keys,
                  f"rope_scaling {rs}: llama3 only, with exactly the keys {sorted(keys)}")
            _need(rs["factor"] >= 1 and 0 < rs["low_freq_factor"] < rs["high_freq_factor"]
                  and rs["original_max_position_embeddings"] > 0,
                  f"rope_scaling {rs}: factor >= 1, 0 < low_freq_factor < high_freq_factor, "
                  "original_max_position_embeddings > 0")
            object.__setattr__(self, "rope_scaling", tuple(sorted(rs.items())))
        _need(0 < self.suffix_len <= self.num_hidden_layers, "suffix_len must be in (0, num_hidden_layers]")
        _need(0 <= self.suffix_plain_top < self.suffix_len, "suffix_plain_top must be in [0, suffix_len)")
        _need(not (self.suffix_plain_top and (self.memory == "gdn" or self.inner_kvb_head)),
              "suffix_plain_top > 0: TTT only, without the key-value-binding head")
        if self.fast_layers is not None:
            fl = tuple(sorted(int(x) for x in self.fast_layers))
            object.__setattr__(self, "fast_layers", fl)
            _need(len(fl) > 0 and len(set(fl)) == len(fl) and fl[-1] < self.num_hidden_layers,
                  f"fast_layers {fl}: distinct layer indices below num_hidden_layers")
            _need(fl[0] == self.num_hidden_layers - self.suffix_len,
                  f"fast_layers {fl}: the lowest must be the suffix's first layer "
                  f"(suffix_len = {self.num_hidden_layers - fl[0]})")
            _need(not (self.suffix_plain_top or self.memory == "gdn" or self.inner_kvb_head),
                  "fast_layers: TTT only, without suffix_plain_top or the key-value-binding head")
        _need(self.mask_token_id < self.vocab_size, f"mask_token_id {self.mask_token_id} >= vocab_size {self.vocab_size}")
        _need(0.0 <= self.inner_decay < 0.1, "inner_decay must be in [0, 0.1) (parameterised as 0.1 * sigmoid)")
        _need(self.hidden_act in ("silu", "gelu"), f"unsupported hidden_act {self.hidden_act!r}")
        _need(self.memory in ("ttt", "gdn"), f"memory {self.memory!r} (ttt | gdn)")
        _need(-1 <= self.window_reach <= self.window_chunks,
              f"window_reach {self.window_reach}: -1 (all) or 0 .. window_chunks ({self.window_chunks})")
        _need(self.read_block >= 0 and (self.read_block == 0 or self.chunk_size % self.read_block == 0),
              f"read_block {self.read_block}: 0 or a divisor of chunk_size {self.chunk_size}")
        _need(not (self.memory == "gdn" and (self.inner_lr_gate or self.inner_token_gate or self.inner_decay > 0
                                             or self.inner_optimizer or self.inner_feat_head or self.inner_kvb_head)),
              "memory gdn has no fast weight: the write controls / feature head do not apply")
        _need(self.gdn_conv >= 0 and self.gdn_chunk > 0, "gdn_conv >= 0 and gdn_chunk > 0")
        _need(not (self.gdn_alternate or self.gdn_conv) or self.memory == "gdn", "gdn_alternate / gdn_conv need memory gdn")

    # ---- derived quantities (reference config.py:172-215)
    @property
    def prefix_len(self) -> int:
        return self.num_hidden_layers - self.suffix_len

    @property
    def fast_mask(self) -> Tuple[bool, ...]:
        if self.fast_layers is not None:
            return tuple((self.prefix_len + i) in self.fast_layers for i in range(self.suffix_len))
        n_fast = self.suffix_len - self.suffix_plain_top
        return tuple(i < n_fast for i in range(self.suffix_len))

    @property
    def fast_len(self) -> int:
        return sum(self.fast_mask)

    @property
    def fast_layer_indices(self) -> Tuple[int, ...]:
        return tuple(self.prefix_len + i for i, f in enumerate(self.fast_mask) if f)

    @property
    def suffix_runs(self) -> Tuple[Tuple[bool, int, int], ...]:
        mask, out, start = self.fast_mask, [], 0
        for i in range(1, len(mask) + 1):
            if i == len(mask) or mask[i] != mask[start]:
                out.append((mask[start], start, i))
                start = i
        return tuple(out)

    @property
    def prime_intermediate_size(self) -> int:
        return self.ttt_intermediate_size or self.intermediate_size

    @property
    def reach(self) -> Optional[int]:
        return None if self.window_reach < 0 else self.window_reach

    @property
    def window_len(self) -> int:
        return self.window_chunks * self.chunk_size

    def to_json_dict(self) -> Dict[str, Any]:
        d = dc.asdict(self)
        d.pop("_ADDED", None)
        if d["rope_scaling"] is not None:
            d["rope_scaling"] = dict(d["rope_scaling"])
        defaults = {f.name: f.default for f in dc.fields(self)}
        for k in self._ADDED:
            if d[k] == defaults[k]:
                d.pop(k)
        return d

    @classmethod
    def load(cls, path: str) -> "ModelConfig":
        return cls(**_accept(cls, _read_json(path)))

    def save(self, path: str) -> None:
        with open(path, "w") as fh:
            json.dump(self.to_json_dict(), fh, indent=2)

    def replace(self, **kw) -> "ModelConfig":
        d = {f.name: getattr(self, f.name) for f in dc.fields(self)}
        if d["rope_scaling"] is not None:
            d["rope_scaling"] = dict(d["rope_scaling"])
        d.update(kw)
        return ModelConfig(**d)


# ModelConfig is frozen: the class attribute above is not a field
ModelConfig.__dataclass_fields__.pop("_ADDED", None)


@dc.dataclass(frozen=True)
class TrainConfig:
    # what to train on
    model_config: str = "configs/1b_e2e"
    sources: str = ""
    data_root: str = ""
    seq_len: int = 8192
    batch_size: int = 64
    grad_accum: int = 1
    steps: int = 50_000
    seed: int = 42
    plant_frac: float = 0.0
    plant_len_min: int = 32
    plant_len_max: int = 128
    train_recall: bool = False
    train_recall_cue: int = 16
    doc_windows: bool = False
    # outer optimiser
    lr: float = 1e-3
    end_lr: float = 1e-5
    warmup_steps: int = 5000
    decay_start: int = -1
    decay_end: int = -1
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    adam_b1: float = 0.9
    adam_b2: float = 0.95
    no_decay_pattern: str = r"embed|norm|bias|inner_|A_log"
    fast_weight_lr_scale: float = 1.0
    # inner loop
    inner_lr: float = 1.0
    inner_clip: float = 1.0
    inner_lr_warmup_steps: int = 5000
    inner_mask_range: Tuple[float, float] = (0.5, 1.0)
    inner_mask_ratio: float = -1.0
    second_order: bool = True
    # objective
    time_reweighting: str = "cart"
    cart_p: float = 0.1
    cart_window: int = 512
    # memory / speed
    remat_levels: int = 1
    remat_prefix: bool = False
    prefix_remat_levels: int = 1
    keep_prefix_layers: int = 0             # this many prefix layers keep their activations instead of recomputing (180 GB parts); < 0: as many as fit
    keep_suffix_chunks: int = 0             # this many chunk steps per segment keep their graph instead of running twice; < 0: as many as fit
    segment_chunks: int = 0
    truncate_fast_weight: bool = False
    inner_views: int = 1
    inner_view_mode: str = "complement"
    inner_views_sequential: bool = False
    inner_cart: bool = False
    inner_mask_span: float = 0.0
    inner_update: str = "sgd"
    inner_task: str = "mask"
    inner_from_outer: bool = False
    inner_mask_mode: str = "random"
    inner_target_frac: float = 0.5
    inner_generic_floor: float = 0.1
    no_write: bool = False
    write_off: bool = False
    aux_causal_weight: float = 0.0
    inner_feat: str = "off"
    inner_feat_weight: float = 1.0
    inner_update_frac: float = 1.0
    # write schemes of the causal write
    inner_subchunks: int = 1
    inner_subchunk_scale: float = 1.0
    inner_surprise_gamma: float = 0.0
    inner_kvb_weight: float = 0.0
    inner_kvb_value: str = "self"
    inner_fast_frac: float = 0.0
    inner_fast_lr_scale: float = 1.0
    inner_fast_decay: float = 0.0
    inner_write_steps: int = 1
    inner_norm_alpha: float = 0.0
    inner_norm_cap: float = 1.0
    window_drop: float = 0.0
    window_drop_frac: float = 0.9
    self_prior: float = 0.0
    outer_views: int = 1
    distill: bool = False
    distill_t_range: Tuple[float, float] = (0.1, 0.3)
    distill_weight: float = 1.0
    distill_topk: int = 64
    distill_meta: bool = True
    distill_warmup_steps: int = 0
    mtp: bool = False
    mtp_weight: float = 0.3
    inner_mtp_weight: float = 0.5
    fused_ce_block: int = 8192
    attn_chunk_batch: int = 2
    replicate_weights: str = "suffix,embed"
    # checkpoints / logging
    ckpt_dir: str = "bucket/checkpoints"
    ckpt_interval: int = 1000
    keep_checkpoints: int = 3
    resume: str = ""
    resume_legacy_root: str = ""
    init_from: str = ""
    continue_from: str = ""
    log_interval: int = 10
    # evaluation
    holdout: int = 4_194_304
    eval_seed: int = 12345
    outer_t: float = -1.0
    outer_shift: bool = False
    log_dir: str = ""
    eval_batches: int = 1
    eval_interval: int = 0
    eval_inner_lr_scales: str = "1"
    eval_only: bool = False
    eval_step0: bool = True
    eval_probes: bool = False
    eval_sources: str = ""
    unigram_path: str = "bucket/data/tokens/unigram_llama3.i64"
    eval_fixed_t: str = ""
    eval_reread_chunks: int = 0
    eval_score_from_chunk: int = -1
    eval_planted_recall: bool = False
    eval_planted_batches: int = 1
    eval_planted_len: int = 64
    eval_planted_cue: int = 16
    eval_write_plan: str = ""
    prefetch: int = 4
    wandb_project: str = ""
    probe_memory: bool = False
    profile_dir: str = ""
    fsdp_size: int = 0
    # --- additions of this package (omitted from JSON while at their defaults) ---
    tp_size: int = 1                      # tensor-parallel group size inside a node (heads / MLP width / vocab)
    compute_dtype: str = "bfloat16"       # bfloat16 | float32 (CPU checks)
    fused_comm: bool = True               # fused compute+collective kernels over peer memory (else NCCL)
    shard_compute: bool = False           # prefix matrices: bf16 copies current only in the owner's slice, gathered inside each GEMM

    _ADDED = ("tp_size", "compute_dtype", "fused_comm", "shard_compute")

    def __post_init__(self):
        c = self
        _need(c.fsdp_size >= 0, f"fsdp_size must be non-negative, got {c.fsdp_size}")
        _need(c.tp_size >= 1, "tp_size >= 1")
        _need(c.compute_dtype in ("bfloat16", "float32"), f"compute_dtype {c.compute_dtype!r}")
        _need(c.seq_len > 0, "seq_len must be positive")
        _need(c.time_reweighting in ("cart", "linear", "original", "none"), f"time_reweighting {c.time_reweighting!r}")
        lo, hi = c.inner_mask_range
        _need(0.0 <= lo <= hi <= 1.0, "inner_mask_range must satisfy 0 <= lo <= hi <= 1")
        _need(c.inner_view_mode in ("complement", "strata"), f"inner_view_mode {c.inner_view_mode!r} (complement | strata)")
        _need(c.inner_view_mode != "complement" or c.inner_views in (1, 2),
              "inner_views must be 1 or 2 with complementary views (use inner_view_mode strata for more)")
        _need(c.inner_view_mode != "strata" or c.inner_views >= 2, "inner_view_mode strata needs inner_views >= 2")
        _need(c.inner_update in ("sgd", "sign", "muon2"), f"inner_update {c.inner_update!r} (sgd | sign | muon2)")
        _need(c.inner_mask_mode in ("random", "rare", "docaware"),
              f"inner_mask_mode {c.inner_mask_mode!r} (random | rare | docaware)")
        _need(0.0 < c.inner_update_frac <= 1.0, "inner_update_frac in (0, 1]")
        _need(c.inner_feat in ("off", "add", "only") and c.inner_feat_weight >= 0,
              f"inner_feat {c.inner_feat!r} (off | add | only), weight >= 0")
        _need(c.inner_task in ("mask", "causal", "split"), f"inner_task {c.inner_task!r} (mask | causal | split)")
        dlo, dhi = c.distill_t_range
        _need(0.0 <= dlo <= dhi <= 1.0 and c.distill_topk >= 1 and c.distill_weight >= 0,
              "distill_t_range must satisfy 0 <= lo <= hi <= 1, distill_topk >= 1, distill_weight >= 0")
        _need(not (c.distill and (c.inner_task == "split" or c.inner_views != 1 or c.no_write or c.inner_from_outer
                                  or c.eval_reread_chunks)),
              "distill needs inner_task mask | causal, one inner view, a write (not no_write / inner_from_outer) "
              "and no re-read evaluation")
        _need(c.aux_causal_weight >= 0, "aux_causal_weight must be >= 0")
        _need(0.0 <= c.plant_frac < 1.0 and 2 <= c.plant_len_min <= c.plant_len_max,
              "plant_frac in [0, 1) and 2 <= plant_len_min <= plant_len_max")
        _need(not (c.train_recall and (c.plant_frac > 0 or c.grad_accum != 1
                                       or not 0 < c.train_recall_cue < c.plant_len_min)),
              "train_recall plants itself (plant_frac 0), needs grad_accum 1 and 0 < train_recall_cue < plant_len_min")
        if c.eval_write_plan:
            try:
                plan = [tuple(int(v) for v in e.split(":")) for e in c.eval_write_plan.split(",") if e.strip()]
                good = all(len(e) == 2 and min(e) >= 0 for e in plan)
            except ValueError:
                good = False
            _need(good and c.inner_task == "causal",
                  "eval_write_plan: 'chunk:steps,...' with chunk, steps >= 0 (causal write)")
        _need(not c.eval_planted_recall or (0 < c.eval_planted_cue < c.eval_planted_len and c.eval_planted_batches >= 1),
              "eval_planted_recall needs 0 < eval_planted_cue < eval_planted_len and eval_planted_batches >= 1")
        _need(all(0.0 <= v <= 1.0 for v in (c.window_drop, c.window_drop_frac, c.self_prior)),
              "window_drop, window_drop_frac and self_prior are in [0, 1]")
        _need(not (c.self_prior > 0 and (c.no_write or c.write_off or c.inner_from_outer)),
              "self_prior reads a chunk after its own write: it needs a write")
        _need(c.fast_weight_lr_scale >= 0, "fast_weight_lr_scale >= 0")
        _need(c.outer_views >= 1 and not (c.outer_views > 1 and (c.distill or c.mtp or c.inner_from_outer)),
              "outer_views >= 1, and > 1 not with distill / mtp / inner_from_outer")
        schemes = (c.inner_subchunks != 1 or c.inner_subchunk_scale != 1.0 or c.inner_surprise_gamma > 0
                   or c.inner_kvb_weight > 0 or c.inner_fast_frac > 0 or c.inner_write_steps != 1
                   or c.inner_norm_alpha > 0)
        _need(not (schemes and (c.inner_task != "causal" or c.inner_views != 1 or c.no_write or c.inner_from_outer
                                or c.write_off or c.distill or c.mtp or c.inner_feat != "off"
                                or c.inner_update_frac < 1.0)),
              "the write schemes (inner_subchunks / surprise / kvb / fast / write_steps) need the plain causal write "
              "(inner_task causal, one view, no no_write / inner_from_outer / write_off / distill / mtp / "
              "inner_feat / inner_update_frac)")
        _need(not (c.write_off and (c.no_write or c.inner_from_outer or c.distill or c.mtp or c.inner_views != 1
                                    or c.inner_feat != "off")),
              "write_off keeps one plain inner stream (not no_write / inner_from_outer / distill / mtp / views / feat)")
        _need(not (c.aux_causal_weight > 0 and (c.no_write or c.inner_from_outer)),
              "aux_causal_weight needs an inner stream (not no_write / inner_from_outer)")
        _need(c.mtp_weight >= 0 and c.inner_mtp_weight >= 0, "mtp_weight and inner_mtp_weight must be >= 0")
        _need(not (c.mtp and (not c.outer_shift or c.inner_task != "causal" or c.no_write or c.inner_from_outer)),
              "mtp needs outer_shift, inner_task causal and a causal write (not no_write / inner_from_outer)")
        _need(not (c.resume and c.resume != "auto" and c.init_from),
              "--resume <path> and --init_from are mutually exclusive (use --resume auto)")
        _need(not (c.continue_from and (c.continue_from == "auto" or c.init_from or c.resume not in ("", "auto"))),
              "--continue_from <step dir> resumes this run's own newest checkpoint first (resume auto): "
              "not with --init_from or --resume <path>")
        if c.continue_from:
            parent = os.path.dirname(os.path.abspath(c.continue_from.rstrip("/")))
            _need(parent != os.path.abspath(c.ckpt_dir),
                  f"--continue_from {c.continue_from} is in this run's own ckpt_dir: a branch or stage "
                  "needs a ckpt_dir of its own (to restart a run, use --resume auto)")
        if c.decay_start >= 0 or c.decay_end >= 0:
            _need(max(1, c.warmup_steps) <= c.decay_start < c.decay_end,
                  f"decay_start {c.decay_start}, decay_end {c.decay_end}: "
                  "warmup_steps <= decay_start < decay_end, or both -1 (no decay)")
        _need(c.eval_reread_chunks >= 0 and c.eval_score_from_chunk >= -1,
              "eval_reread_chunks >= 0 and eval_score_from_chunk >= -1")

    def to_json_dict(self) -> Dict[str, Any]:
        d = dc.asdict(self)
        defaults = {f.name: f.default for f in dc.fields(self)}
        for k in self._ADDED:
            if d[k] == defaults[k]:
                d.pop(k)
        return d

    @classmethod
    def load(cls, path: str) -> "TrainConfig":
        raw = _read_json(path)
        for k in ("inner_mask_range", "distill_t_range"):
            if k in raw:
                raw[k] = tuple(raw[k])
        return cls(**_accept(cls, raw))

    def save(self, path: str) -> None:
        with open(path, "w") as fh:
            json.dump(self.to_json_dict(), fh, indent=2)

    def data_path(self, path: str) -> str:
        return os.path.join(self.data_root, path) if path and self.data_root else path

    def replace(self, **kw) -> "TrainConfig":
        return dc.replace(self, **kw)


TrainConfig.__dataclass_fields__.pop("_ADDED", None)
